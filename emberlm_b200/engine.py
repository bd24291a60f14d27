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


class TrainEngine:
    """One rank's training state: parameter / gradient arenas, ZeRO-1 shard of AdamW m/v,
    workspace, and the step. `group` is a torch.distributed process group (None = 1 GPU)."""

    def __init__(self, cfg: ModelConfig, batch: int, seq: int, device="cuda:0", group=None,
                 lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, clip=1.0, train=True):
        self.cfg, self.B, self.T = cfg, batch, seq
        self.device = torch.device(device)
        self.group = group
        if group is not None:
            import torch.distributed as dist
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        else:
            self.world, self.rank = 1, 0
        if self.world > 1:
            # The collectives run beside the backward pass on their own stream and hold a few SMs
            # while they do; a persistent GEMM that wants every SM would then run in two waves.
            lib.check(_L.ctdk_reserve_sms(int(os.environ.get("CTDK_DP_RESERVED_SMS", "0"))))
        self.layout = model_layout(cfg)
        # arena padded so that it splits evenly over ranks in 64-float units
        self.total = padded_total(self.layout.total, self.world)
        self.shard = self.total // self.world
        self.params = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        self.grads = torch.zeros(self.total, dtype=torch.float32, device=self.device) if train else None
        ws = _L.ctdk_engine_workspace_bytes(C.byref(cfg), batch, seq)
        if ws < 0:
            raise lib.CtdkError(-1, lib.last_error())
        self.workspace = torch.empty(ws, dtype=torch.uint8, device=self.device)
        self._h = C.c_void_p()
        lib.check(_L.ctdk_engine_create(C.byref(cfg), self.params.data_ptr(),
                                        self.grads.data_ptr() if train else None,
                                        self.workspace.data_ptr(), ws, batch, seq, C.byref(self._h)))
        self.loss_sums = torch.zeros(2, dtype=torch.float32, device=self.device)
        self.hp = dict(lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, clip=clip)
        self.step_count = 0
        self._cb = None
        self._user_cb = None
        if train:
            self.m = torch.zeros(self.shard, dtype=torch.float32, device=self.device)
            self.v = torch.zeros(self.shard, dtype=torch.float32, device=self.device)
            self._scalars = torch.zeros(4, dtype=torch.float32, device=self.device)  # sumsq, scale, norm
            self._build_segments()
            if self.world > 1:
                self._install_bucket_callback()

    def __del__(self):
        h = getattr(self, "_h", None)
        if h and _L is not None:
            _L.ctdk_engine_destroy(h)
            self._h = None

    # ---- parameters -------------------------------------------------------------------
    def named_parameters(self) -> dict:
        if getattr(self, "buckets", None):
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

    def _build_segments(self) -> None:
        """One rank: one segment table over the whole arena. Several ranks: the arena is cut into
        buckets (make_buckets), rank r owns slice r of each; m / v hold the slices back to back and
        every slice has its own weight-decay segment table."""
        wd = self.hp["weight_decay"]
        if self.world == 1:
            ends, wds = build_segments(self.layout, wd, 0, self.total)
            self.seg_end = torch.tensor(ends, dtype=torch.int64, device=self.device)
            self.seg_wd = torch.tensor(wds, dtype=torch.float32, device=self.device)
            self.buckets = []
            return
        self.buckets = []
        pos = 0
        per = int(os.environ.get("CTDK_DP_BUCKET_LAYERS", "4"))
        for lo, hi, ready in make_buckets(self.layout, self.total, self.world, self.cfg.num_hidden_layers, per):
            a, b = bucket_slice(lo, hi, self.world, self.rank)
            ends, wds = build_segments(self.layout, wd, a, b)
            self.buckets.append(dict(
                lo=lo, hi=hi, ready=ready, a=a, b=b, state=pos,
                seg_end=torch.tensor(ends, dtype=torch.int64, device=self.device),
                seg_wd=torch.tensor(wds, dtype=torch.float32, device=self.device), work=None))
            pos += b - a
        assert pos == self.shard

    def _install_bucket_callback(self) -> None:
        """Reduce-scatter of a bucket starts as soon as the backward kernels of the last layer it
        needs have been enqueued: the collective runs on the process group's own stream behind an
        event on the compute stream, so it overlaps the backward of the layers below."""
        import torch.distributed as dist

        def on_layer(layer: int) -> None:
            if self._user_cb is not None:
                self._user_cb(layer)
            if not self._reduce_in_backward:
                return
            for bk in self.buckets:
                if bk["ready"] == layer and bk["work"] is None:
                    bk["work"] = dist.reduce_scatter_tensor(self.grads[bk["a"]:bk["b"]], self.grads[bk["lo"]:bk["hi"]],
                                                            op=dist.ReduceOp.SUM, group=self.group, async_op=True)

        self._reduce_in_backward = False
        self._cb = LAYER_CALLBACK(lambda layer, _u: on_layer(layer))
        lib.check(_L.ctdk_engine_set_layer_callback(self._h, self._cb, None))

        # All-gathers of the updated parameters are left in flight by optimizer_step(); each part of
        # the next forward pass first makes the compute stream wait for the buckets it reads (the
        # embedding bucket is also the tied LM head, read again at the end).
        L = self.cfg.num_hidden_layers
        for bk in self.buckets:
            touched = [tensor_layer(n, L) for n, o, k in zip(self.layout.names, self.layout.offsets, self.layout.numels)
                       if o < bk["hi"] and o + k > bk["lo"]]
            bk["first_use"] = min(touched) if touched else L
            bk["gather"] = None

        def on_forward(layer: int) -> None:
            for bk in self.buckets:
                if bk["gather"] is not None and bk["first_use"] <= layer:
                    bk["gather"].wait()
                    bk["gather"] = None

        self._fcb = LAYER_CALLBACK(lambda layer, _u: on_forward(layer))
        lib.check(_L.ctdk_engine_set_forward_callback(self._h, self._fcb, None))

    def wait_parameters(self) -> None:
        """Makes the current stream wait for every all-gather that optimizer_step() left in flight.
        Called before anything other than the engine's own forward pass reads self.params."""
        for bk in getattr(self, "buckets", []):
            if bk.get("gather") is not None:
                bk["gather"].wait()
                bk["gather"] = None

    # ---- step -------------------------------------------------------------------------
    def set_layer_callback(self, fn) -> None:
        if self.world > 1 and self.grads is not None:
            self._user_cb = fn          # chained in front of the gradient-bucket callback
            return
        self._cb = LAYER_CALLBACK(lambda layer, _u: fn(layer)) if fn else LAYER_CALLBACK(0)
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
        self._reduce_in_backward = bool(last) and self.world > 1
        try:
            lib.check(_L.ctdk_engine_forward_backward(
                self._h, ids.data_ptr(), targets.data_ptr(), loss_mask.data_ptr(), row_weight.data_ptr(),
                B, T, int(accumulate), self.loss_sums.data_ptr(), _stream_ptr()))
        finally:
            self._reduce_in_backward = False

    def forward_loss(self, ids, targets, loss_mask) -> None:
        B, T = ids.shape
        lib.check(_L.ctdk_engine_forward_loss(self._h, ids.data_ptr(), targets.data_ptr(),
                                              loss_mask.data_ptr(), B, T, self.loss_sums.data_ptr(),
                                              _stream_ptr()))

    def optimizer_step(self, lr=None) -> None:
        """reduce-scatter(grads) -> sum of squares (+ all-reduce) -> clip scale -> fused AdamW on
        this rank's slices -> all-gather(params). No host synchronisation. With several ranks the
        arena is handled bucket by bucket: reduce-scatters that forward_backward(last=True) already
        started are only waited for (a stream dependency), the rest are issued here; the all-gather
        of a bucket overlaps the AdamW of the next."""
        hp = self.hp
        lr = hp["lr"] if lr is None else lr
        s = _stream_ptr()
        sc = self._scalars
        sc.zero_()
        if self.world > 1:
            import torch.distributed as dist
            order = sorted(self.buckets, key=lambda bk: -bk["ready"])   # the order backward completes them
            for bk in order:
                if bk["work"] is None:
                    bk["work"] = dist.reduce_scatter_tensor(self.grads[bk["a"]:bk["b"]], self.grads[bk["lo"]:bk["hi"]],
                                                            op=dist.ReduceOp.SUM, group=self.group, async_op=True)
            for bk in order:
                bk["work"].wait()
                bk["work"] = None
                lib.call("ctdk_sumsq", self.grads[bk["a"]:bk["b"]].data_ptr(), bk["b"] - bk["a"], sc.data_ptr(), s)
            dist.all_reduce(sc[0:1], group=self.group)
            dist.all_reduce(self.loss_sums, group=self.group)
        else:
            lib.call("ctdk_sumsq", self.grads.data_ptr(), self.shard, sc.data_ptr(), s)
        lib.call("ctdk_clip_scale", sc.data_ptr(), hp["clip"], 1e-6, sc[1:].data_ptr(), sc[2:].data_ptr(), s)
        self.step_count += 1
        t = np.float32(self.step_count)
        bc1 = np.float32(1.0) - np.power(np.float32(hp["beta1"]), t, dtype=np.float32)
        bc2 = np.float32(1.0) - np.power(np.float32(hp["beta2"]), t, dtype=np.float32)
        ap = lib.AdamWParams(lr, hp["beta1"], hp["beta2"], hp["eps"], 0.0, float(bc1), float(bc2))
        if self.world == 1:
            lib.call("ctdk_adamw", self.params.data_ptr(), self.grads.data_ptr(), self.m.data_ptr(),
                     self.v.data_ptr(), self.shard, C.byref(ap), sc[1:].data_ptr(), self.seg_end.data_ptr(),
                     self.seg_wd.data_ptr(), self.seg_end.numel(), s)
            return
        import torch.distributed as dist
        for bk in self.buckets:   # arena order = the order the next forward pass reads them
            n, st = bk["b"] - bk["a"], bk["state"]
            pslice = self.params[bk["a"]:bk["b"]]
            lib.call("ctdk_adamw", pslice.data_ptr(), self.grads[bk["a"]:bk["b"]].data_ptr(),
                     self.m[st:st + n].data_ptr(), self.v[st:st + n].data_ptr(), n, C.byref(ap), sc[1:].data_ptr(),
                     bk["seg_end"].data_ptr(), bk["seg_wd"].data_ptr(), bk["seg_end"].numel(), s)
            bk["gather"] = dist.all_gather_into_tensor(self.params[bk["lo"]:bk["hi"]], pslice, group=self.group,
                                                       async_op=True)
        if os.environ.get("CTDK_DP_GATHER_OVERLAP", "1") != "1":
            self.wait_parameters()

    def train_step(self, ids, targets, loss_mask, row_weight, lr=None, active_rows=None) -> None:
        """One optimizer step on this rank's rows (already weighted per micro-batch). active_rows:
        optional int32 device tensor of the supervised positions (see set_active_rows)."""
        self.loss_sums.zero_()
        if active_rows is not None:
            self.set_active_rows(active_rows)
        self.forward_backward(ids, targets, loss_mask, row_weight, accumulate=False, last=True)
        self.optimizer_step(lr)

    def read_metrics(self) -> dict:
        """Synchronises and returns the logged loss (mask-weighted mean, main.cpp:365-380) and
        the pre-clip gradient norm of the last step."""
        ls = self.loss_sums.tolist()
        sc = self._scalars.tolist()
        return dict(loss=ls[0] / ls[1] if ls[1] > 0 else 0.0, mask_sum=ls[1], grad_norm=sc[2], clip_scale=sc[1])


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
        n = min(max_new_tokens, self.max_seq_len - ids.numel())
        out = torch.zeros(max(n, 1), dtype=torch.int64, device=self.device)
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            lib.check(_L.ctdk_decode_prefill(self._h, ids.data_ptr(), ids.numel(), self.stream.cuda_stream))
            if n > 0:
                lib.check(_L.ctdk_decode_greedy(self._h, n, out.data_ptr(), self.stream.cuda_stream))
        torch.cuda.current_stream().wait_stream(self.stream)
        return out[:max(n, 0)]

    def last_logits(self) -> torch.Tensor:
        p = C.c_void_p()
        lib.check(_L.ctdk_decode_logits(self._h, C.byref(p)))
        base = self.workspace.data_ptr()
        off = p.value - base
        return self.workspace[off:off + 4 * self.cfg.vocab_size].view(torch.float32)
