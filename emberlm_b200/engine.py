"""Host-side driver of the training-step engine (libctdk.so's ctdk_engine_* entry points).

torch is used for device memory, streams and torch.distributed only; every arithmetic
kernel of the step is a ctdk kernel. Names and grouping follow the reference:
parameters in Model::collect_parameters order with the decay / no-decay split
(emberlm src/nn/model.cpp:63-100), AdamW hyper-parameters and bias corrections as
optim::AdamW (src/core/optim.cu:132-168), clipping as optim::clip_grad_norm_
(src/core/optim.cu:248-293), micro-batch semantics as tools/ctd_train/main.cpp:346-373.
"""
from __future__ import annotations

import ctypes as C
import os
import math
from dataclasses import dataclass

import numpy as np
import torch

from . import lib

_L = lib.raw()


class ModelConfig(C.Structure):
    """ctdk_model_config; field names follow LlamaConfig (include/ctd/nn/model.h:19-37)."""
    _fields_ = [
        ("vocab_size", C.c_int), ("hidden_size", C.c_int), ("intermediate_size", C.c_int),
        ("num_hidden_layers", C.c_int), ("num_attention_heads", C.c_int),
        ("num_key_value_heads", C.c_int), ("head_dim", C.c_int),
        ("rms_norm_eps", C.c_float), ("rope_theta", C.c_float), ("qk_norm", C.c_int),
        ("rope_scaling_factor", C.c_float), ("rope_scaling_low_freq_factor", C.c_float),
        ("rope_scaling_high_freq_factor", C.c_float), ("rope_scaling_original_max_pos", C.c_int),
        ("gradient_checkpointing", C.c_int), ("precision", C.c_int),
    ]


def make_config(vocab_size, hidden_size, intermediate_size, num_hidden_layers, num_attention_heads,
                num_key_value_heads, head_dim, rms_norm_eps=1e-5, rope_theta=100000.0,
                qk_norm=False, rope_scaling_factor=0.0, rope_scaling_low_freq_factor=1.0,
                rope_scaling_high_freq_factor=4.0, rope_scaling_original_max_pos=8192,
                gradient_checkpointing=False, precision=lib.GEMM_TF32, **_ignored) -> ModelConfig:
    return ModelConfig(vocab_size, hidden_size, intermediate_size, num_hidden_layers,
                       num_attention_heads, num_key_value_heads, head_dim, rms_norm_eps, rope_theta,
                       int(qk_norm), rope_scaling_factor, rope_scaling_low_freq_factor,
                       rope_scaling_high_freq_factor, rope_scaling_original_max_pos,
                       int(gradient_checkpointing), precision)


# The five presets of include/ctd/nn/model.h:39-124.
PRESETS = {
    "smollm2_135m": dict(vocab_size=49152, hidden_size=576, intermediate_size=1536, num_hidden_layers=30,
                         num_attention_heads=9, num_key_value_heads=3, head_dim=64, rms_norm_eps=1e-5,
                         rope_theta=100000.0),
    "smollm2_360m": dict(vocab_size=49152, hidden_size=960, intermediate_size=2560, num_hidden_layers=32,
                         num_attention_heads=15, num_key_value_heads=5, head_dim=64, rms_norm_eps=1e-5,
                         rope_theta=100000.0),
    "qwen3_0_6b": dict(vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28,
                       num_attention_heads=16, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6,
                       rope_theta=1000000.0, qk_norm=True),
    "qwen3_1_7b": dict(vocab_size=151936, hidden_size=2048, intermediate_size=6144, num_hidden_layers=28,
                       num_attention_heads=16, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6,
                       rope_theta=1000000.0, qk_norm=True),
    "llama3_2_1b": dict(vocab_size=128256, hidden_size=2048, intermediate_size=8192, num_hidden_layers=16,
                        num_attention_heads=32, num_key_value_heads=8, head_dim=64, rms_norm_eps=1e-5,
                        rope_theta=500000.0, rope_scaling_factor=32.0, rope_scaling_low_freq_factor=1.0,
                        rope_scaling_high_freq_factor=4.0, rope_scaling_original_max_pos=8192),
}


def param_names(cfg: ModelConfig) -> list[str]:
    """HF names in Model::collect_parameters order (src/nn/model.cpp:78-98)."""
    names = ["model.embed_tokens.weight"]
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        names += [p + "input_layernorm.weight", p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight",
                  p + "self_attn.v_proj.weight", p + "self_attn.o_proj.weight"]
        if cfg.qk_norm:
            names += [p + "self_attn.q_norm.weight", p + "self_attn.k_norm.weight"]
        names += [p + "post_attention_layernorm.weight", p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight",
                  p + "mlp.down_proj.weight"]
    names.append("model.norm.weight")
    return names


def param_shapes(cfg: ModelConfig) -> list[tuple[int, ...]]:
    hid, I, D = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    H, Hk = cfg.num_attention_heads, cfg.num_key_value_heads
    shapes = [(cfg.vocab_size, hid)]
    for _ in range(cfg.num_hidden_layers):
        shapes += [(hid,), (H * D, hid), (Hk * D, hid), (Hk * D, hid), (hid, H * D)]
        if cfg.qk_norm:
            shapes += [(D,), (D,)]
        shapes += [(hid,), (I, hid), (I, hid), (hid, I)]
    shapes.append((hid,))
    return shapes


@dataclass
class Layout:
    names: list
    shapes: list
    offsets: list
    numels: list
    decay: list
    total: int


def model_layout(cfg: ModelConfig) -> Layout:
    n = _L.ctdk_model_num_tensors(C.byref(cfg))
    if n < 0:
        raise lib.CtdkError(-1, lib.last_error())
    off = (C.c_int64 * n)()
    num = (C.c_int64 * n)()
    dec = (C.c_int * n)()
    total = C.c_int64()
    lib.check(_L.ctdk_model_layout(C.byref(cfg), off, num, dec, C.byref(total)))
    names, shapes = param_names(cfg), param_shapes(cfg)
    assert len(names) == n and all(int(np.prod(s)) == num[i] for i, s in enumerate(shapes))
    return Layout(names, shapes, list(off), list(num), list(dec), total.value)


def padded_total(layout_total: int, world: int) -> int:
    """Arena length padded so that it splits evenly over `world` ranks in 64-float units."""
    unit = 64 * world
    return (layout_total + unit - 1) // unit * unit


def shard_bounds(total_padded: int, world: int, rank: int) -> tuple[int, int]:
    """ZeRO-1 ownership: rank r owns the contiguous slice r of parameters, gradients, m and v."""
    shard = total_padded // world
    return rank * shard, (rank + 1) * shard


def tensor_layer(name: str, num_layers: int) -> int:
    """Backward-completion index of a parameter: the layer number for decoder-layer tensors,
    num_layers for the final norm, -1 for the (tied) embedding, whose gradient is final only after
    the embedding backward at the very end (the layer callback of the engine uses the same
    numbering)."""
    if name.startswith("model.layers."):
        return int(name.split(".")[2])
    return num_layers if name == "model.norm.weight" else -1


def make_buckets(layout: Layout, total_padded: int, world: int, num_layers: int, layers_per_bucket: int = 4):
    """Cuts the arena into contiguous buckets [lo, hi) whose lengths are multiples of 64 * world:
    the embedding, then groups of `layers_per_bucket` decoder layers (the last one also takes the
    final norm and the padding). Cuts are rounded down to the unit, so a bucket may begin inside the
    last tensor of the previous group. Returns [(lo, hi, ready)] in arena order; `ready` is the
    lowest completion index (see tensor_layer) of the tensors the bucket overlaps: the bucket's
    gradients are final once the layer callback has fired for `ready` (backward runs from the
    last layer down to the embedding). Rank r owns slice r of every bucket."""
    unit = 64 * world
    layer_of = [tensor_layer(n, num_layers) for n in layout.names]
    first = {}
    for o, l in zip(layout.offsets, layer_of):
        first[l] = min(first.get(l, o), o)
    cuts = [0]
    if layers_per_bucket > 0:       # 0: one bucket = the whole arena (reduced after the backward pass)
        for l in range(0, num_layers, layers_per_bucket):
            c = first[l] // unit * unit
            if c > cuts[-1]:
                cuts.append(c)
    cuts.append(total_padded)
    out = []
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        ready = min((l for o, k, l in zip(layout.offsets, layout.numels, layer_of) if o < hi and o + k > lo),
                    default=num_layers)
        out.append((lo, hi, ready))
    return out


def bucket_slice(lo: int, hi: int, world: int, rank: int) -> tuple[int, int]:
    """Arena range of bucket [lo, hi) that `rank` owns."""
    n = (hi - lo) // world
    return lo + rank * n, lo + (rank + 1) * n


def deal_micro_batches(accum: int, world: int, rank: int) -> list[int]:
    """The step's `accum` micro-batches are dealt round-robin: rank r runs r, r+world, ..."""
    if accum % world:
        raise ValueError(f"{accum} micro-batches do not divide over {world} ranks")
    return list(range(rank, accum, world))


def build_segments(layout: Layout, weight_decay: float, lo: int, hi: int):
    """Weight-decay segments of the arena slice [lo, hi): decay group gets weight_decay, norm
    weights 0 (the two ParamGroups of tools/ctd_train/main.cpp:304-311); padding counts as
    no-decay. Returns (exclusive end offsets relative to lo, decay per segment)."""
    ends, wds = [], []
    pos = lo
    for o, k, d in zip(layout.offsets, layout.numels, layout.decay):
        padded_end = o + (k + 63) // 64 * 64
        if padded_end <= lo or o >= hi:
            continue
        end = min(padded_end, hi)
        wd = weight_decay if d else 0.0
        if ends and wds[-1] == wd:
            ends[-1] = end - lo
        else:
            ends.append(end - lo)
            wds.append(wd)
        pos = end
    if pos < hi:
        if ends and wds[-1] == 0.0:
            ends[-1] = hi - lo
        else:
            ends.append(hi - lo)
            wds.append(0.0)
    if not ends:
        ends, wds = [hi - lo], [0.0]
    ends[-1] = hi - lo
    return ends, wds


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


_L.ctdk_model_num_tensors.restype = C.c_int64
_L.ctdk_model_num_tensors.argtypes = [C.POINTER(ModelConfig)]
_L.ctdk_model_layout.restype = C.c_int
_L.ctdk_model_layout.argtypes = [C.POINTER(ModelConfig), C.POINTER(C.c_int64), C.POINTER(C.c_int64),
                                 C.POINTER(C.c_int), C.POINTER(C.c_int64)]
_L.ctdk_engine_workspace_bytes.restype = C.c_int64
_L.ctdk_engine_workspace_bytes.argtypes = [C.POINTER(ModelConfig), C.c_int64, C.c_int64]
_L.ctdk_engine_create.restype = C.c_int
_L.ctdk_engine_create.argtypes = [C.POINTER(ModelConfig), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                  C.c_int64, C.c_int64, C.POINTER(C.c_void_p)]
_L.ctdk_engine_destroy.restype = C.c_int
_L.ctdk_engine_destroy.argtypes = [C.c_void_p]
_L.ctdk_engine_forward_backward.restype = C.c_int
_L.ctdk_engine_forward_backward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                            C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]
_L.ctdk_engine_forward_loss.restype = C.c_int
_L.ctdk_engine_forward_loss.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                        C.c_void_p, C.c_void_p]
_L.ctdk_engine_set_active_rows.restype = C.c_int
_L.ctdk_engine_set_active_rows.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
LAYER_CALLBACK = C.CFUNCTYPE(None, C.c_int, C.c_void_p)
_L.ctdk_engine_set_forward_callback.restype = C.c_int
_L.ctdk_engine_set_forward_callback.argtypes = [C.c_void_p, C.CFUNCTYPE(None, C.c_int, C.c_void_p), C.c_void_p]
_L.ctdk_engine_set_layer_callback.restype = C.c_int
_L.ctdk_engine_set_layer_callback.argtypes = [C.c_void_p, LAYER_CALLBACK, C.c_void_p]


class TrainerHParams(C.Structure):
    """ctdk_trainer_hparams."""
    _fields_ = [("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
                ("weight_decay", C.c_float), ("clip", C.c_float), ("layers_per_bucket", C.c_int)]


_L.ctdk_dp_arena_floats.restype = C.c_int64
_L.ctdk_dp_arena_floats.argtypes = [C.POINTER(ModelConfig), C.c_int]
_L.ctdk_dp_num_buckets.restype = C.c_int
_L.ctdk_dp_num_buckets.argtypes = [C.POINTER(ModelConfig), C.c_int, C.c_int]
_L.ctdk_dp_buckets.restype = C.c_int
_L.ctdk_dp_buckets.argtypes = [C.POINTER(ModelConfig), C.c_int, C.c_int, C.c_int] + [C.POINTER(C.c_int64)] * 5 + [
    C.POINTER(C.c_int)]
_L.ctdk_dp_segments.restype = C.c_int
_L.ctdk_dp_segments.argtypes = [C.POINTER(ModelConfig), C.c_float, C.c_int64, C.c_int64, C.POINTER(C.c_int64),
                                C.POINTER(C.c_float), C.c_int]
_L.ctdk_trainer_unique_id.restype = C.c_int
_L.ctdk_trainer_unique_id.argtypes = [C.c_void_p]
_L.ctdk_trainer_create.restype = C.c_int
_L.ctdk_trainer_create.argtypes = [C.POINTER(ModelConfig), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_void_p,
                                   C.POINTER(TrainerHParams), C.POINTER(C.c_void_p)]
_L.ctdk_trainer_destroy.restype = C.c_int
_L.ctdk_trainer_destroy.argtypes = [C.c_void_p]
_L.ctdk_trainer_engine.restype = C.c_void_p
_L.ctdk_trainer_engine.argtypes = [C.c_void_p]
_L.ctdk_trainer_set_layer_callback.restype = C.c_int
_L.ctdk_trainer_set_layer_callback.argtypes = [C.c_void_p, LAYER_CALLBACK, C.c_void_p]
_L.ctdk_trainer_step.restype = C.c_int
_L.ctdk_trainer_step.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                 C.c_void_p, C.c_int64, C.c_float, C.c_void_p]
_L.ctdk_trainer_zero_loss.restype = C.c_int
_L.ctdk_trainer_zero_loss.argtypes = [C.c_void_p, C.c_void_p]
_L.ctdk_trainer_forward_backward.restype = C.c_int
_L.ctdk_trainer_forward_backward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                             C.c_int64, C.c_int, C.c_int, C.c_void_p]
_L.ctdk_trainer_forward_loss.restype = C.c_int
_L.ctdk_trainer_forward_loss.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
_L.ctdk_trainer_optimizer_step.restype = C.c_int
_L.ctdk_trainer_optimizer_step.argtypes = [C.c_void_p, C.c_float, C.c_void_p]
_L.ctdk_trainer_allreduce_loss.restype = C.c_int
_L.ctdk_trainer_allreduce_loss.argtypes = [C.c_void_p, C.c_void_p]
_L.ctdk_trainer_wait_parameters.restype = C.c_int
_L.ctdk_trainer_wait_parameters.argtypes = [C.c_void_p, C.c_void_p]
_L.ctdk_trainer_read_metrics.restype = C.c_int
_L.ctdk_trainer_read_metrics.argtypes = [C.c_void_p, C.POINTER(C.c_float), C.c_void_p]
_L.ctdk_trainer_loss_sums.restype = C.c_void_p
_L.ctdk_trainer_loss_sums.argtypes = [C.c_void_p]
_L.ctdk_trainer_step_count.restype = C.c_int64
_L.ctdk_trainer_step_count.argtypes = [C.c_void_p]
_L.ctdk_trainer_set_step_count.restype = C.c_int
_L.ctdk_trainer_set_step_count.argtypes = [C.c_void_p, C.c_int64]
_L.ctdk_trainer_gather_state.restype = C.c_int
_L.ctdk_trainer_gather_state.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
_L.ctdk_trainer_scatter_state.restype = C.c_int
_L.ctdk_trainer_scatter_state.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
_L.ctdk_batch_widen.restype = C.c_int
_L.ctdk_batch_widen.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]


def dp_plan(cfg: ModelConfig, world: int, rank: int, layers_per_bucket: int = 4):
    """The library's bucket plan (ctdk_dp_buckets) as a list of dicts: lo, hi, a, b (the slice `rank`
    owns), state (offset of that slice in the rank's m / v), ready."""
    n = _L.ctdk_dp_num_buckets(C.byref(cfg), world, layers_per_bucket)
    if n < 0:
        raise lib.CtdkError(-1, lib.last_error())
    arr = [(C.c_int64 * n)() for _ in range(5)]
    ready = (C.c_int * n)()
    lib.check(_L.ctdk_dp_buckets(C.byref(cfg), world, rank, layers_per_bucket, *arr, ready))
    return [dict(lo=arr[0][i], hi=arr[1][i], a=arr[2][i], b=arr[3][i], state=arr[4][i], ready=ready[i])
            for i in range(n)]


def dp_segments(cfg: ModelConfig, weight_decay: float, lo: int, hi: int):
    """The library's weight-decay segments of the arena range [lo, hi) (ctdk_dp_segments)."""
    n = _L.ctdk_dp_segments(C.byref(cfg), weight_decay, lo, hi, None, None, 0)
    if n < 0:
        raise lib.CtdkError(-1, lib.last_error())
    ends, wds = (C.c_int64 * n)(), (C.c_float * n)()
    _L.ctdk_dp_segments(C.byref(cfg), weight_decay, lo, hi, ends, wds, n)
    return list(ends), list(wds)


def nccl_unique_id() -> bytes:
    """128-byte NCCL unique id (rank 0 makes it, every rank passes the same bytes to TrainEngine)."""
    buf = C.create_string_buffer(128)
    lib.check(_L.ctdk_trainer_unique_id(buf))
    return buf.raw


class TrainEngine:
    """One rank's training state on top of the library's data-parallel trainer (ctdk_trainer_*):
    torch owns the device memory (parameter / gradient arenas, this rank's ZeRO-1 slices of AdamW's
    m / v, the workspace); the step, the bucketed reduce-scatter / all-gather over NCCL and the
    optimizer run inside libctdk.so. `group` is a torch.distributed process group (None = 1 GPU),
    used only to hand rank 0's NCCL unique id to the other ranks; pass `nccl_id` to do that yourself."""

    def __init__(self, cfg: ModelConfig, batch: int, seq: int, device="cuda:0", group=None,
                 lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, clip=1.0, train=True,
                 rank=None, world=None, nccl_id: bytes | None = None):
        self.cfg, self.B, self.T = cfg, batch, seq
        self.device = torch.device(device)
        self.group = group
        if group is not None:
            import torch.distributed as dist
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        else:
            self.world, self.rank = (world or 1), (rank or 0)
        if self.world > 1:
            # The collectives run beside the backward pass on their own stream and hold a few SMs
            # while they do; a persistent GEMM that wants every SM would then run in two waves.
            lib.check(_L.ctdk_reserve_sms(int(os.environ.get("CTDK_DP_RESERVED_SMS", "0"))))
            if nccl_id is None:
                import torch.distributed as dist
                box = [nccl_unique_id() if self.rank == 0 else None]
                dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0), group=group)
                nccl_id = box[0]
        self.layout = model_layout(cfg)
        # arena padded so that it splits evenly over ranks in 64-float units
        self.total = _L.ctdk_dp_arena_floats(C.byref(cfg), self.world)
        assert self.total == padded_total(self.layout.total, self.world)
        self.shard = self.total // self.world
        self.params = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        self.grads = torch.zeros(self.total, dtype=torch.float32, device=self.device) if train else None
        ws = _L.ctdk_engine_workspace_bytes(C.byref(cfg), batch, seq)
        if ws < 0:
            raise lib.CtdkError(-1, lib.last_error())
        self.workspace = torch.empty(ws, dtype=torch.uint8, device=self.device)
        self.hp = dict(lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, clip=clip)
        self._t = None
        self._h = C.c_void_p()
        self._cb = None
        self.device_status = 0
        if train:
            self.m = torch.zeros(self.shard, dtype=torch.float32, device=self.device)
            self.v = torch.zeros(self.shard, dtype=torch.float32, device=self.device)
            per = int(os.environ.get("CTDK_DP_BUCKET_LAYERS", "4"))
            thp = TrainerHParams(lr, beta1, beta2, eps, weight_decay, clip, per)
            self._t = C.c_void_p()
            with torch.cuda.device(self.device):
                lib.check(_L.ctdk_trainer_create(C.byref(cfg), self.params.data_ptr(), self.grads.data_ptr(),
                                                 self.m.data_ptr(), self.v.data_ptr(), self.workspace.data_ptr(), ws,
                                                 batch, seq, self.rank, self.world, nccl_id, C.byref(thp),
                                                 C.byref(self._t)))
            self._h = C.c_void_p(_L.ctdk_trainer_engine(self._t))
            self.buckets = dp_plan(cfg, self.world, self.rank, per if self.world > 1 else 0)
            # device float[2] {sum mask*loss, sum mask} the passes add to (inside the trainer)
            self.loss_sums = _view_device_floats(_L.ctdk_trainer_loss_sums(self._t), 2, self.device)
        else:
            lib.check(_L.ctdk_engine_create(C.byref(cfg), self.params.data_ptr(), None,
                                            self.workspace.data_ptr(), ws, batch, seq, C.byref(self._h)))
            self.buckets = []
            self.loss_sums = torch.zeros(2, dtype=torch.float32, device=self.device)

    def __del__(self):
        t, h = getattr(self, "_t", None), getattr(self, "_h", None)
        if _L is None:
            return
        if t:
            _L.ctdk_trainer_destroy(t)
            self._t = self._h = None
        elif h:
            _L.ctdk_engine_destroy(h)
            self._h = None

    @property
    def step_count(self) -> int:
        return int(_L.ctdk_trainer_step_count(self._t)) if self._t else 0

    @step_count.setter
    def step_count(self, n: int) -> None:
        lib.check(_L.ctdk_trainer_set_step_count(self._t, int(n)))

    # ---- parameters -------------------------------------------------------------------
    def named_parameters(self) -> dict:
        self.wait_parameters()
        lo = self.layout
        return {n: self.params[o:o + k].view(s) for n, s, o, k in zip(lo.names, lo.shapes, lo.offsets, lo.numels)}

    def named_grads(self) -> dict:
        lo = self.layout
        return {n: self.grads[o:o + k].view(s) for n, s, o, k in zip(lo.names, lo.shapes, lo.offsets, lo.numels)}

    def load_parameters(self, tensors: dict) -> None:
        views = self.named_parameters()
        for n, v in views.items():
            src = tensors[n]
            src = torch.from_numpy(np.ascontiguousarray(src)) if isinstance(src, np.ndarray) else src
            if tuple(src.shape) != tuple(v.shape):
                raise RuntimeError(f"load_parameters: shape mismatch for {n}")
            v.copy_(src.to(torch.float32))

    def init_parameters(self, seed=1234, std=0.02) -> None:
        """Random-init N(0, std) for embedding / linear weights, 1.0 for every norm weight."""
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)
        self.params.zero_()
        for (n, v), dec in zip(self.named_parameters().items(), self.layout.decay):
            if dec:
                v.normal_(0.0, std, generator=gen)
            else:
                v.fill_(1.0)

    def wait_parameters(self) -> None:
        """Makes the current stream wait for every all-gather that optimizer_step() left in flight.
        Called before anything other than the engine's own forward pass reads self.params."""
        if self._t:
            lib.check(_L.ctdk_trainer_wait_parameters(self._t, _stream_ptr()))

    def gather_state(self, shard_state: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """m or v in arena order, assembled from every rank's slices (for checkpoints)."""
        out = torch.empty(self.total, dtype=torch.float32, device=self.device) if out is None else out
        lib.check(_L.ctdk_trainer_gather_state(self._t, shard_state.data_ptr(), out.data_ptr(), _stream_ptr()))
        return out

    def scatter_state(self, full: torch.Tensor, shard_state: torch.Tensor) -> None:
        lib.check(_L.ctdk_trainer_scatter_state(self._t, full.data_ptr(), shard_state.data_ptr(), _stream_ptr()))

    # ---- step -------------------------------------------------------------------------
    def set_layer_callback(self, fn) -> None:
        """fn(layer) is called when everything that writes layer `layer`'s gradients has been
        ordered before the current stream (see ctdk_engine_set_layer_callback)."""
        self._cb = LAYER_CALLBACK(lambda layer, _u: fn(layer)) if fn else LAYER_CALLBACK(0)
        if self._t:
            lib.check(_L.ctdk_trainer_set_layer_callback(self._t, self._cb, None))
        else:
            lib.check(_L.ctdk_engine_set_layer_callback(self._h, self._cb, None))

    def set_active_rows(self, rows: torch.Tensor | None) -> None:
        """Names the supervised positions (ascending int32 indices into the flattened batch) of the
        next forward_backward / forward_loss call, so the LM head skips the others."""
        self._active = rows  # keep alive until the kernels have run
        n = 0 if rows is None else rows.numel()
        lib.check(_L.ctdk_engine_set_active_rows(self._h, rows.data_ptr() if n else None, n))

    def forward_backward(self, ids, targets, loss_mask, row_weight, accumulate=False, last=False) -> None:
        """last=True (several ranks): this is the step's final backward pass, so each gradient
        bucket is reduce-scattered as soon as it is complete; optimizer_step() picks the results up."""
        B, T = ids.shape
        lib.check(_L.ctdk_trainer_forward_backward(
            self._t, ids.data_ptr(), targets.data_ptr(), loss_mask.data_ptr(), row_weight.data_ptr(),
            B, T, int(accumulate), int(last), _stream_ptr()))

    def forward_loss(self, ids, targets, loss_mask) -> None:
        B, T = ids.shape
        if self._t:
            lib.check(_L.ctdk_trainer_forward_loss(self._t, ids.data_ptr(), targets.data_ptr(), loss_mask.data_ptr(),
                                                   B, T, _stream_ptr()))
        else:
            lib.check(_L.ctdk_engine_forward_loss(self._h, ids.data_ptr(), targets.data_ptr(), loss_mask.data_ptr(),
                                                  B, T, self.loss_sums.data_ptr(), _stream_ptr()))

    def optimizer_step(self, lr=None) -> None:
        """reduce-scatter(grads) -> sum of squares (+ all-reduce) -> clip scale -> fused AdamW on
        this rank's slices -> all-gather(params), all inside ctdk_trainer_optimizer_step. No host
        synchronisation; the all-gathers are left in flight for the next forward pass."""
        lib.check(_L.ctdk_trainer_optimizer_step(self._t, self.hp["lr"] if lr is None else lr, _stream_ptr()))
        if os.environ.get("CTDK_DP_GATHER_OVERLAP", "1") != "1":
            self.wait_parameters()

    def train_step(self, ids, targets, loss_mask, row_weight, lr=None, active_rows=None) -> None:
        """One optimizer step on this rank's rows (already weighted per micro-batch). active_rows:
        optional int32 device tensor of the supervised positions (see set_active_rows)."""
        B, T = ids.shape
        self._active = active_rows
        n = 0 if active_rows is None else active_rows.numel()
        lib.check(_L.ctdk_trainer_step(self._t, ids.data_ptr(), targets.data_ptr(), loss_mask.data_ptr(),
                                       row_weight.data_ptr(), B, T, active_rows.data_ptr() if n else None, n,
                                       self.hp["lr"] if lr is None else lr, _stream_ptr()))
        if os.environ.get("CTDK_DP_GATHER_OVERLAP", "1") != "1":
            self.wait_parameters()

    def read_metrics(self) -> dict:
        """Synchronises and returns the logged loss (mask-weighted mean, main.cpp:365-380) and
        the pre-clip gradient norm of the last step. Raises CtdkError if a bounded device-side wait
        gave up since the last call (the results since then are not to be trusted)."""
        out = (C.c_float * 5)()
        lib.check(_L.ctdk_trainer_read_metrics(self._t, out, _stream_ptr()))
        self.device_status = 0
        return dict(loss=out[0] / out[1] if out[1] > 0 else 0.0, mask_sum=out[1], grad_norm=out[4], clip_scale=out[3])


class _DeviceFloats:
    """A few fp32 values in device memory that the library owns, exposed through the CUDA array
    interface so that torch can view them without copying."""

    def __init__(self, ptr: int, n: int):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 3,
                                         "strides": None}


def _view_device_floats(ptr: int, n: int, device) -> torch.Tensor:
    return torch.as_tensor(_DeviceFloats(ptr, n), device=device)


def check_device_status() -> int:
    """Reads (and clears) the device status word that the kernels' bounded waits write when one of
    them gives up; synchronises the current stream. Raises CtdkError (CTDK_ETIMEOUT) if a wait ran
    out since the last check: the results computed since then are not to be trusted."""
    lib.check(_L.ctdk_device_status(_stream_ptr(), None))
    return 0


def row_weights(loss_mask: torch.Tensor, micro_batch: int, accum_total: int) -> torch.Tensor:
    """w[i] = mask_i / (A * sum(mask of i's micro-batch)): the factor the reference applies
    through mul_scalar(loss, 1/A) and the masked-CE backward (main.cpp:346-361, loss.cu:388-411).
    loss_mask is [rows, T] with rows a multiple of micro_batch; A counts ALL micro-batches of
    the step (over every rank). Micro-batches with an empty mask get weight 0 (main.cpp:357)."""
    rows, T = loss_mask.shape
    m = loss_mask.view(rows // micro_batch, micro_batch * T)
    sm = m.sum(dim=1, keepdim=True)
    w = torch.where(sm > 0, m / (sm * accum_total), torch.zeros_like(m))
    return w.view(rows, T).contiguous()


# ----------------------------------------------------------------------------------------------
# KV-cache greedy decoding (the ctd_generate path)
# ----------------------------------------------------------------------------------------------
_L.ctdk_decode_workspace_bytes.restype = C.c_int64
_L.ctdk_decode_workspace_bytes.argtypes = [C.POINTER(ModelConfig), C.c_int64]
_L.ctdk_decode_create.restype = C.c_int
_L.ctdk_decode_create.argtypes = [C.POINTER(ModelConfig), C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                  C.POINTER(C.c_void_p)]
_L.ctdk_decode_destroy.restype = C.c_int
_L.ctdk_decode_destroy.argtypes = [C.c_void_p]
_L.ctdk_decode_prefill.restype = C.c_int
_L.ctdk_decode_prefill.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
_L.ctdk_decode_greedy.restype = C.c_int
_L.ctdk_decode_greedy.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
_L.ctdk_decode_logits.restype = C.c_int
_L.ctdk_decode_logits.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]


class Decoder:
    """Greedy KV-cache generation, batch 1, as ctd_generate with temperature <= 0
    (tools/ctd_generate/main.cpp:94-184): prefill the prompt, then one token per step."""

    def __init__(self, cfg: ModelConfig, max_seq_len: int, device="cuda:0", params: torch.Tensor | None = None):
        self.cfg, self.max_seq_len = cfg, max_seq_len
        self.device = torch.device(device)
        self.layout = model_layout(cfg)
        self.params = params if params is not None else torch.zeros(self.layout.total, dtype=torch.float32,
                                                                    device=self.device)
        ws = _L.ctdk_decode_workspace_bytes(C.byref(cfg), max_seq_len)
        if ws < 0:
            raise lib.CtdkError(-1, lib.last_error())
        self.workspace = torch.zeros(ws, dtype=torch.uint8, device=self.device)
        self._h = C.c_void_p()
        lib.check(_L.ctdk_decode_create(C.byref(cfg), self.params.data_ptr(), self.workspace.data_ptr(), ws,
                                        max_seq_len, C.byref(self._h)))
        self.stream = torch.cuda.Stream(device=self.device)

    def __del__(self):
        h = getattr(self, "_h", None)
        if h and _L is not None:
            _L.ctdk_decode_destroy(h)
            self._h = None

    def named_parameters(self) -> dict:
        lo = self.layout
        return {n: self.params[o:o + k].view(s) for n, s, o, k in zip(lo.names, lo.shapes, lo.offsets, lo.numels)}

    def load_parameters(self, tensors: dict) -> None:
        for n, v in self.named_parameters().items():
            src = tensors[n]
            src = torch.from_numpy(np.ascontiguousarray(src)) if isinstance(src, np.ndarray) else src
            v.copy_(src.to(torch.float32))

    def generate(self, input_ids, max_new_tokens: int) -> torch.Tensor:
        """Returns the generated token ids (device int64 [n]); n = min(max_new_tokens, room left in
        max_seq_len). An empty prompt raises, as the reference reports 'empty_prompt'."""
        ids = torch.as_tensor(input_ids, dtype=torch.int64, device=self.device).reshape(-1).contiguous()
        if ids.numel() == 0:
            raise RuntimeError("generate: empty_prompt")
        n = min(max_new_tokens, self.max_seq_len - ids.numel() + 1)   # the last token needs no cache position (as the reference's loop)
        out = torch.zeros(max(n, 1), dtype=torch.int64, device=self.device)
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            lib.check(_L.ctdk_decode_prefill(self._h, ids.data_ptr(), ids.numel(), self.stream.cuda_stream))
            if n > 0:
                lib.check(_L.ctdk_decode_greedy(self._h, n, out.data_ptr(), self.stream.cuda_stream))
            # a bounded wait that gave up inside a kernel of the generation is an error, not a result
            lib.check(_L.ctdk_device_status(self.stream.cuda_stream, None))
        torch.cuda.current_stream().wait_stream(self.stream)
        return out[:max(n, 0)]

    def last_logits(self) -> torch.Tensor:
        p = C.c_void_p()
        lib.check(_L.ctdk_decode_logits(self._h, C.byref(p)))
        base = self.workspace.data_ptr()
        off = p.value - base
        return self.workspace[off:off + 4 * self.cfg.vocab_size].view(torch.float32)
