#!/usr/bin/env python
"""Benchmark of the decoder training step (forward + backward + clip + AdamW), data-parallel
over N GPUs of one node. Prints ONE JSON line on rank 0.

  python bench.py --gpus 1 --steps 10 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
      --master-port P bench.py --gpus N --steps K --warmup W
  python bench.py --impl reference ...     # the reference's own CUDA build of the same step

Workload: the SmolLM2-360M-shaped decoder on a global batch of 32 rows x 1024 tokens (the step
sees T = 1023 positions per row, as the reference's loader shifts inputs/targets), random-init
fp32 weights, uniform synthetic token ids, ~50 % span loss masks. The batch is the reference's
8 micro-batches of 4 rows (each normalised by its own mask sum, weighted 1/8); rank r takes
micro-batches r, r+N, ... and runs them in one fused pass, gradients are reduce-scattered,
AdamW runs on the rank's ZeRO-1 shard, parameters are all-gathered. Total work is fixed as N
grows (strong scaling). `value` = positions/s with inputs resident in HBM; `e2e` = the same
with token / mask rows coming from pinned host memory every step and the loss read back.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import re
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (preset, global rows, seq_len, micro-batch rows, grad-accum micro-batches, checkpointing)
    "smollm2_135m_b4x512": ("smollm2_135m", 4, 512, 4, 1, False),
    "smollm2_360m_b32x1024": ("smollm2_360m", 32, 1024, 4, 8, False),
    # one rank's share of the 8-GPU step above (for single-GPU profiles of the small-M kernels)
    "smollm2_360m_b4x1024": ("smollm2_360m", 4, 1024, 4, 1, False),
    "qwen3_0_6b_b16x2048": ("qwen3_0_6b", 16, 2048, 2, 8, False),
    "llama3_2_1b_b32x2048": ("llama3_2_1b", 32, 2048, 4, 8, True),
    "qwen3_1_7b_b64x4096": ("qwen3_1_7b", 64, 4096, 2, 32, True),
}
DEFAULT_WORKLOAD = "smollm2_360m_b32x1024"
HP = dict(lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, clip=1.0)
METRIC = "train tokens/s (fwd+bwd+AdamW)"
NCU_GEMM_DRAM_BYTES_PER_FLOP = (74.0e6 + 115.7e6) / (2.0 * 16384 * 2560 * 960)


def workload_config(name: str) -> dict:
    """The `config` object both arms print: what the workload is, nothing about how an arm runs it."""
    preset, rows, S, mb, A, ckpt = WORKLOADS[name]
    return {"workload": name, "global_batch": rows, "seq_len": S, "positions_per_step": rows * (S - 1), "micro_batch": mb,
            "grad_accum": A, "gradient_checkpointing": ckpt}


def step_rows(vocab: int, rows: int, S: int, step: int):
    """The documents of step `step` (both arms train on the same rows; four distinct steps, then they repeat)."""
    return synth_rows(vocab, rows, S, seed=4321 + step % 4)


def algorithmic_flops_per_step(cfg: dict, rows: int, T: int) -> float:
    """3 * [2*tok*(P_mat + V*hid) + L*B*H*2*T^2*D]: forward + 2x backward, causal half of the
    attention square, recomputation and masked-row skipping not counted."""
    hid, I, D = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    H, Hk, L, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["num_hidden_layers"], cfg["vocab_size"]
    p_mat = L * (2 * hid * H * D + 2 * hid * Hk * D + 3 * hid * I)
    tok = rows * T
    return 3.0 * (2.0 * tok * (p_mat + V * hid) + L * rows * H * 2.0 * T * T * D)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16_burst=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_burst=1590.0, bf16_sustained=1400.0, source="fallback")


def synth_rows(vocab: int, rows: int, S: int, seed: int):
    """int32 token rows and int8 0/1 masks in the reference's bin format: mask[0] = 0, then
    alternating spans of 16..128 positions, 'assistant' spans = 1 (about half of the positions)."""
    import numpy as np
    rng = np.random.default_rng(seed)
    tok = rng.integers(0, vocab, size=(rows, S), dtype=np.int32)
    msk = np.zeros((rows, S), dtype=np.int8)
    for d in range(rows):
        pos, val = 1, 0
        while pos < S:
            ln = int(rng.integers(16, 129))
            msk[d, pos:pos + ln] = val
            pos += ln
            val ^= 1
        if msk[d].sum() == 0:
            msk[d, -1] = 1
    return tok, msk


# ----------------------------------------------------------------------------------------------
def run_ours(args) -> dict:
    import numpy as np
    import torch
    import torch.distributed as dist

    from emberlm_b200 import engine as E, lib

    preset, rows, S, mb, A, ckpt = WORKLOADS[args.workload]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        # NCCL may print a version banner on stdout at communicator creation: send everything written
        # to fd 1 before the result line to stderr, so stdout carries the one JSON line only.
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
        group = dist.group.WORLD
        warm = torch.zeros(1, device="cuda")
        dist.all_reduce(warm)
        torch.cuda.synchronize()
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        os.close(saved_stdout)
    if A % world != 0:
        raise SystemExit(f"{A} micro-batches do not divide over {world} ranks")
    T = S - 1
    my_mbs = list(range(rank, A, world))          # micro-batches dealt round-robin
    my_rows = len(my_mbs) * mb
    cfgd = dict(E.PRESETS[preset])
    precision = lib.GEMM_3XTF32 if args.precision == "3xtf32" else lib.GEMM_TF32
    cfg = E.make_config(**cfgd, gradient_checkpointing=ckpt, precision=precision)
    eng = E.TrainEngine(cfg, my_rows, T, device=f"cuda:{local}", group=group, **HP)
    eng.init_parameters(seed=1234)

    # synthetic documents: a different set of rows per step, same on every rank; a rank keeps the
    # rows of its own micro-batches
    n_steps = args.warmup + args.steps
    L_ = lib.raw()
    L_.ctdk_launch_count.restype = C.c_longlong
    L_.ctdk_prof_collect.argtypes = [C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_longlong)]

    def host_batch(step):
        tok, msk = step_rows(cfgd["vocab_size"], rows, S, step)
        sel = np.concatenate([np.arange(j * mb, (j + 1) * mb) for j in my_mbs])
        return tok[sel], msk[sel]

    pinned_tok = [torch.empty((my_rows, S), dtype=torch.int32).pin_memory() for _ in range(2)]
    pinned_msk = [torch.empty((my_rows, S), dtype=torch.int8).pin_memory() for _ in range(2)]
    pinned_act = [torch.empty(my_rows * T, dtype=torch.int32).pin_memory() for _ in range(2)]
    host = [host_batch(s) for s in range(min(n_steps, 4))]

    dev = torch.device(f"cuda:{local}")
    d_bufs = [dict(ids=torch.empty((my_rows, T), dtype=torch.int64, device=dev), tgt=torch.empty((my_rows, T), dtype=torch.int64, device=dev),
                   mask=torch.empty((my_rows, T), dtype=torch.float32, device=dev), w=torch.empty((my_rows, T), dtype=torch.float32, device=dev),
                   sums=torch.empty(len(my_mbs) + 1, dtype=torch.float32, device=dev)) for _ in range(max(2, len(host)))]

    def to_device(step, slot, keep=None):
        """One step's rows as they lie in the bins (int32 tokens, int8 masks: 5 bytes per token) and the
        supervised positions from pinned host memory to the device, then widened there by the library
        (ctdk_batch_widen: int64 ids / targets, fp32 mask, per-row weights). keep: index of a private
        set of output buffers (the device-resident arm keeps one per step); None = slot's."""
        t, m = host[step % len(host)]
        pinned_tok[slot].copy_(torch.from_numpy(t))
        pinned_msk[slot].copy_(torch.from_numpy(m))
        act = np.flatnonzero(m[:, 1:]).astype(np.int32)      # supervised positions, known to the loader
        pinned_act[slot][:act.size].copy_(torch.from_numpy(act))
        d_tok = pinned_tok[slot].cuda(non_blocking=True)
        d_msk = pinned_msk[slot].cuda(non_blocking=True)
        d_act = pinned_act[slot][:act.size].cuda(non_blocking=True)
        b = d_bufs[slot if keep is None else keep]
        lib.check(L_.ctdk_batch_widen(d_tok.data_ptr(), d_msk.data_ptr(), my_rows, S, mb, A, b["ids"].data_ptr(), b["tgt"].data_ptr(),
                                      b["mask"].data_ptr(), b["w"].data_ptr(), b["sums"].data_ptr(),
                                      torch.cuda.current_stream().cuda_stream))
        return b["ids"], b["tgt"], b["mask"], b["w"], d_act

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(run_step, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(steps):
            run_step(s)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    # ---- device-resident arm ------------------------------------------------------------
    resident = [to_device(s, s % 2, keep=s) for s in range(len(host))]
    torch.cuda.synchronize()

    def step_resident(s):
        ids, tgt, mask, w, act = resident[s % len(resident)]
        eng.train_step(ids, tgt, mask, w, active_rows=act)

    for s in range(args.warmup):
        step_resident(s)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    n0 = L_.ctdk_launch_count()
    ms_total = timed(step_resident, args.steps)
    launches = L_.ctdk_launch_count() - n0
    # The same K steps once more with every GEMM / attention / norm / AdamW launch bracketed by CUDA
    # events on its stream (about a thousand extra event records per step, which is why `value`
    # above is taken without them).
    L_.ctdk_prof_enable(1)
    ms_prof = timed(step_resident, args.steps)
    L_.ctdk_prof_enable(0)
    clocks = sampler.stop() if sampler else None
    prof = {}
    for name, cls in (("gemm", 0), ("attn", 1), ("adamw", 2), ("norm", 3), ("norm_bwd", 4), ("qk_norm_rope", 5), ("ce", 6), ("embedding", 7)):
        a, b, n = C.c_double(), C.c_double(), C.c_longlong()
        L_.ctdk_prof_collect(cls, C.byref(a), C.byref(b), C.byref(n))
        prof[name] = (a.value, b.value, n.value)
    metrics = eng.read_metrics()

    # ---- end-to-end arm: rows from pinned host memory every step, loss read back ------------
    losses = []

    def step_e2e(s):
        ids, tgt, mask, w, act = to_device(s, s % 2)
        eng.train_step(ids, tgt, mask, w, active_rows=act)
        losses.append(eng.read_metrics()["loss"])      # D2H read of the step's loss / grad norm

    step_e2e(0)
    ms_e2e = timed(step_e2e, args.steps)

    positions = rows * T
    act_mean = int(np.mean([int(m[:, 1:].sum()) for _, m in host]))
    value = positions * args.steps / (ms_total / 1e3)
    e2e_value = positions * args.steps / (ms_e2e / 1e3)
    peaks = measured_peaks()
    gemm_ms, gemm_flops, gemm_n = prof["gemm"]
    tf32_peak = peaks["bf16_sustained"] / 2.0      # TF32 runs at half the bf16 tensor rate
    achieved = gemm_flops / (gemm_ms / 1e3) / 1e12 if gemm_ms > 0 else 0.0
    flops_step = algorithmic_flops_per_step(cfgd, rows, T)
    out = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": ("3xtf32" if args.precision == "3xtf32" else "tf32") + " (fp32 storage, fp32 accumulate)",
        "data": "synthetic", "impl": "ours",
        "config": workload_config(args.workload),
        "notes": {"parallelism": f"dp{world}+zero1 (C++ trainer in libctdk.so, NCCL reduce-scatter / all-gather per bucket)",
                  "precision": args.precision, "supervised_positions_per_rank": act_mean,
                  "lm_head": "supervised rows only (masked rows have zero loss and gradient)",
                  "l2": "inputs larger than L2 (activations of several GB per step)",
                  "algorithmic_tflop_per_step": flops_step / 1e12,
                  "workspace_gib_per_rank": eng.workspace.numel() / 2**30},
        "step_tflops_per_gpu": flops_step / (ms_total / args.steps / 1e3) / 1e12 / world,
        "step_frac_of_tf32_peak": flops_step / (ms_total / args.steps / 1e3) / 1e12 / world / tf32_peak,
        "loss": metrics["loss"], "grad_norm": metrics["grad_norm"],
        "device_status": eng.device_status,     # 0: no bounded device-side wait gave up (checked every read_metrics)
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": my_rows * S * 5 + 4 * act_mean, "d2h_bytes_per_step": 24},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"kernel": "gemm_tf32_kernel (tcgen05)", "bound": "tensor", "achieved": achieved,
                     "peak": tf32_peak, "unit": "TFLOP/s", "frac": achieved / tf32_peak if tf32_peak else None,
                     "peak_source": f"{peaks['source']}: bf16_tflops_sustained/2 (TF32 = half the bf16 rate)",
                     "launches": int(gemm_n), "avg_launch_ms": gemm_ms / gemm_n if gemm_n else None,
                     "share_of_step": gemm_ms / ms_prof, "profiled_ms_per_step": ms_prof / args.steps,
                     # DRAM bytes per average launch, scaled by FLOPs from the one ncu capture of this
                     # kernel (16384 x 2560 x 960: 74.0 MB read + 115.7 MB written for 80.5 GFLOP)
                     "traffic": (NCU_GEMM_DRAM_BYTES_PER_FLOP * gemm_flops / gemm_n) if gemm_n else None,
                     "traffic_source": "ncu dram__bytes_read+write of gemm_tf32_2cta_kernel at 16384x2560x960, "
                                       "scaled to the average launch by FLOPs"},
        "kernel_classes": {k: {"ms_per_step": v[0] / args.steps, "launches_per_step": v[2] / args.steps,
                               "achieved": (v[1] / (v[0] / 1e3) / (1e12 if k in ("gemm", "attn") else 1e9)) if v[0] > 0 else None,
                               "unit": "TFLOP/s" if k in ("gemm", "attn") else "GB/s",
                               "frac_of_measured_peak": (v[1] / (v[0] / 1e3) / 1e12 / tf32_peak if k in ("gemm", "attn")
                                                         else v[1] / (v[0] / 1e3) / 1e9 / peaks["hbm_gbs"]) if v[0] > 0 else None}
                           for k, v in prof.items()},
    }
    if args.rank_invariance and world > 1:
        out["rank_invariance"] = rank_invariance(E, eng, cfg, cfgd, rows, S, mb, A, my_mbs, rank, world, dev)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_baseline(preset)
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else None


def rank_invariance(E, eng, cfg, cfgd, rows, S, mb, A, my_mbs, rank, world, dev) -> dict | None:
    """One optimizer step from identical weights on all ranks (data-parallel) and on rank 0 alone (every
    micro-batch in one pass): the updated weights must agree per tensor up to summation order.
    Reported as max|a-b| / max|b| per tensor; the worst one is named."""
    import numpy as np
    import torch
    import torch.distributed as dist
    T = S - 1
    tok, msk = step_rows(cfgd["vocab_size"], rows, S, 0)

    def device_batch(sel, engine):
        t = torch.from_numpy(tok[sel]).to(dev)
        m = torch.from_numpy(msk[sel]).to(dev)
        ids, tgt = t[:, :-1].to(torch.int64).contiguous(), t[:, 1:].to(torch.int64).contiguous()
        mask = m[:, 1:].to(torch.float32).contiguous()
        return ids, tgt, mask, E.row_weights(mask, mb, A)

    eng.init_parameters(seed=99)
    eng.m.zero_(); eng.v.zero_(); eng.step_count = 0
    sel = np.concatenate([np.arange(j * mb, (j + 1) * mb) for j in my_mbs])
    eng.train_step(*device_batch(sel, eng))
    eng.read_metrics()
    got = eng.params.clone()
    dist.barrier()
    if rank != 0:
        return None
    solo = E.TrainEngine(cfg, rows, T, device=str(dev), **HP)
    solo.init_parameters(seed=99)
    solo.train_step(*device_batch(np.arange(rows), solo))
    solo.read_metrics()
    worst, worst_name, over = 0.0, "", 0
    lay = solo.layout
    for n, o, k in zip(lay.names, lay.offsets, lay.numels):
        a, b = got[o:o + k], solo.params[o:o + k]
        e = float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))
        over += e > 1e-5
        if e > worst:
            worst, worst_name = e, n
    return {"ranks": world, "tensors": len(lay.names), "worst_tensor": worst_name, "worst_max_rel_err": worst,
            "tensors_above_1e-5": int(over),
            "note": "one AdamW step from identical weights, all ranks vs rank 0 alone; differences come from the order of the "
                    "gradient sums (reduce-scatter, split-K) and AdamW's sign-like first step on near-zero gradients (<= 2*lr)"}


def cpu_baseline(preset: str) -> dict:
    """The numpy oracle (a port: the reference has no CPU implementation of the step) timed on the
    host cores on a bounded sample: one row of 1024 tokens through the full model, fwd+bwd+AdamW."""
    import numpy as np
    from oracle import model as om
    cfg = om.PRESETS[preset]
    S = 1024
    params = om.init_params(cfg, seed=1234)
    tok, msk = om.synth_batch(cfg.vocab_size, 1, S, seed=7)
    opt = om.AdamWState()
    t0 = time.perf_counter()
    om.train_step(params, cfg, [om.make_batch(tok, msk, [0])], opt, HP["lr"], HP["beta1"], HP["beta2"], HP["eps"],
                  HP["weight_decay"], HP["clip"])
    dt = time.perf_counter() - t0
    return {"value": (S - 1) / dt, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"1 row x {S} tokens, all {cfg.num_hidden_layers} layers, fwd+bwd+clip+AdamW, numpy/BLAS fp32, {dt:.1f} s"}


# ----------------------------------------------------------------------------------------------
def run_reference(args) -> dict | None:
    """Times the UNMODIFIED reference (its CUDA build, oracle/_ref/ref_harness) on the same
    workload: same config, same micro-batch split (b rows x A micro-batches), same optimizer."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    import numpy as np
    from oracle import model as om, ref_run
    preset, rows, S, mb, A, ckpt = WORKLOADS[args.workload]
    base = {"impl": "reference", "metric": METRIC, "unit": "tokens/s", "higher_is_better": True}
    if not ref_run.available():
        return {**base, "unavailable": "oracle/_ref/ref_harness not built (reference sources absent at build time)"}
    cfg = om.PRESETS[preset]
    params = om.init_params(cfg, seed=1234)
    n_steps = args.warmup + args.steps
    parts = [step_rows(cfg.vocab_size, rows, S, st) for st in range(min(n_steps, 4))]    # the rows of the other arm
    tok, msk = np.concatenate([p_[0] for p_ in parts]), np.concatenate([p_[1] for p_ in parts])
    t0 = time.perf_counter()
    try:
        r = ref_run.run_reference(cfg, params, tok, msk, mb, A, steps=args.steps, warmup=args.warmup,
                                  gradient_checkpointing=ckpt, want_grads=False, want_params=False, **HP)
    except Exception as e:  # noqa: BLE001
        return {**base, "unavailable": f"reference run failed: {str(e)[:200]}"}
    ms = sum(r["step_ms"])
    positions = rows * (S - 1)
    value = positions * args.steps / (ms / 1e3)
    return {**base, "value": value, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp32 (cuBLAS SGEMM, default math mode)", "data": "synthetic",
            "config": workload_config(args.workload),
            "notes": {"parallelism": "single GPU (the reference has no data parallelism)"},
            "loss": r["loss"][-1], "grad_norm": r["grad_norm"][-1],
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": 0, "kind": "reference",
                             "sample": "the reference's own CUDA build on one B200 (it has no CPU path); "
                                       f"{args.steps} steps after {args.warmup} warm-up, wall clock with device sync; "
                                       f"whole run {time.perf_counter() - t0:.0f} s incl. weight load"},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def run_decode(args) -> dict:
    """KV-cache greedy decode, Qwen3-0.6B shape, batch 1: 256 uniform prompt ids, 512 new tokens.
    A "step" is one full generation (prefill + 512 tokens); value = new tokens/s."""
    import torch
    from emberlm_b200 import engine as E
    torch.cuda.set_device(0)
    cfgd = dict(E.PRESETS["qwen3_0_6b"])
    cfg = E.make_config(**cfgd)
    dec = E.Decoder(cfg, max_seq_len=1024)
    gen = torch.Generator(device="cuda").manual_seed(1234)
    for (_, v), dcy in zip(dec.named_parameters().items(), dec.layout.decay):
        v.normal_(0.0, 0.02, generator=gen) if dcy else v.fill_(1.0)
    prompt_len, new_tokens = 256, 512
    prompts = [torch.randint(0, cfgd["vocab_size"], (prompt_len,), generator=gen, device="cuda")
               for _ in range(args.warmup + args.steps)]
    for i in range(args.warmup):
        dec.generate(prompts[i], new_tokens)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        out = dec.generate(prompts[args.warmup + i], new_tokens)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    # end to end: prompt from pinned host memory, generated ids copied back to the host
    host_prompt = prompts[0].cpu().pin_memory()
    t0 = time.perf_counter()
    for i in range(args.steps):
        toks = dec.generate(host_prompt.cuda(non_blocking=True), new_tokens).cpu()
    e2e_s = time.perf_counter() - t0
    P = sum(dec.layout.numels)
    bytes_per_token = 4.0 * P
    peaks = measured_peaks()
    per_tok_ms = ms / args.steps / new_tokens
    return {"metric": "decode tokens/s (greedy, KV cache, batch 1)", "value": new_tokens * args.steps / (ms / 1e3),
            "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "replicas only", "vs_baseline": None, "dtype": "fp32 (GEMV), tf32 prefill",
            "data": "synthetic", "impl": "ours",
            "config": {"workload": "qwen3_0_6b_decode", "prompt_len": prompt_len, "new_tokens": new_tokens,
                       "l2": "weights (2.4 GB) larger than L2"},
            "e2e": {"value": new_tokens * args.steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": prompt_len * 8,
                    "d2h_bytes_per_step": new_tokens * 8},
            "roofline": {"kernel": "gemv_kernel (all weights streamed once per token)", "bound": "hbm",
                         "achieved": bytes_per_token / (per_tok_ms / 1e3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": bytes_per_token / (per_tok_ms / 1e3) / 1e9 / peaks["hbm_gbs"],
                         "note": "whole-token figure incl. prefill share, attention and launch gaps", "traffic": None},
            "last_tokens": toks[-4:].tolist()}


def run_decode_reference(args) -> dict:
    """The reference's own generator (tools/ctd_generate/main.cpp:104-184, built unmodified as
    oracle/_ref/ref_ctd_generate) on the same workload: same random weights written as a safetensors
    file, the same prompts as requests on its stdin (one process per request, as the tool reads its
    whole stdin), greedy, 512 new tokens. A step is the prefill plus the decode time the tool logs
    itself; its weight load is not counted."""
    import tempfile
    import torch
    from emberlm_b200 import engine as E, safetensors_io
    base = {"impl": "reference", "metric": "decode tokens/s (greedy, KV cache, batch 1)", "unit": "tokens/s", "higher_is_better": True}
    exe = ROOT / "oracle" / "_ref" / "ref_ctd_generate"
    if not exe.exists():
        return {**base, "unavailable": "oracle/_ref/ref_ctd_generate not built (reference sources absent at build time)"}
    torch.cuda.set_device(0)
    cfgd = dict(E.PRESETS["qwen3_0_6b"])
    dec = E.Decoder(E.make_config(**cfgd), max_seq_len=1024)
    gen = torch.Generator(device="cuda").manual_seed(1234)
    for (_, v), dcy in zip(dec.named_parameters().items(), dec.layout.decay):
        v.normal_(0.0, 0.02, generator=gen) if dcy else v.fill_(1.0)
    prompt_len, new_tokens = 256, 512
    prompts = [torch.randint(0, cfgd["vocab_size"], (prompt_len,), generator=gen, device="cuda").tolist()
               for _ in range(args.warmup + args.steps)]
    t_all = time.perf_counter()
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "model.safetensors")
        safetensors_io.save_safetensors([(n, v.cpu().numpy()) for n, v in dec.named_parameters().items()], path)
        del dec
        torch.cuda.empty_cache()
        # One request per process (the tool reads its whole stdin as one request); its own log gives the
        # prefill and decode times, so the weight load of every process is not counted.
        secs, last = [], []
        deadline = time.perf_counter() + 280.0   # the whole arm is bounded: a bench run must end within minutes
        try:
            for i, ids in enumerate(prompts):
                left = deadline - time.perf_counter()
                if left <= 5:
                    raise RuntimeError(f"time limit reached after {i} requests")
                r = subprocess.run([str(exe), "--model", path], capture_output=True, text=True, timeout=left,
                                   input=json.dumps(dict(input_ids=ids, max_new_tokens=new_tokens, max_seq_len=1024, temperature=0.0)))
                if r.returncode != 0:
                    raise RuntimeError("generator exited: " + r.stderr[-300:])
                out = [json.loads(ln) for ln in r.stdout.strip().splitlines()]
                got = [m["token"] for m in out if "token" in m]
                if len(got) != new_tokens:
                    raise RuntimeError(f"generator returned {len(got)} tokens: {out[-1]}")
                pre = re.search(r"prefill \(\d+ tok\) in ([0-9.eE+-]+) s", r.stderr)
                dcd = re.search(r"generated \d+ tok in ([0-9.eE+-]+) s", r.stderr)
                if not pre or not dcd:
                    raise RuntimeError("generator log without timings: " + r.stderr[-300:])
                if i >= args.warmup:
                    secs.append(float(pre.group(1)) + float(dcd.group(1)))
                last = got[-4:]
        except Exception as e:  # noqa: BLE001
            return {**base, "unavailable": f"reference generator failed: {str(e)[:200]}"}
    total = sum(secs)
    value = new_tokens * args.steps / total
    return {**base, "value": value, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3,
            "scaling": "replicas only", "vs_baseline": None, "dtype": "fp32 (cuBLAS SGEMM, default math mode)", "data": "synthetic",
            "config": {"workload": "qwen3_0_6b_decode", "prompt_len": prompt_len, "new_tokens": new_tokens,
                       "l2": "weights (2.4 GB) larger than L2"},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": 0, "kind": "reference",
                             "sample": "the reference's own generator (CUDA build, one B200; it has no CPU path), prefill + decode seconds from its log; "
                                       f"whole run {time.perf_counter() - t_all:.0f} s incl. writing and loading the weights"},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "last_tokens": last}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + ["qwen3_0_6b_decode"], default=DEFAULT_WORKLOAD)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--precision", choices=["tf32", "3xtf32"], default="tf32",
                    help="3xtf32: every contraction splits its operands into TF32 high and low parts (near-fp32 results)")
    ap.add_argument("--rank-invariance", action="store_true",
                    help="after the timing, one step from identical weights on all ranks and on rank 0 alone: per-tensor "
                         "difference of the updated weights (needs room for the whole batch on rank 0)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        print(f"note: --warmup {args.warmup} < 3; timing rules ask for at least 3", file=sys.stderr)
    if args.workload == "qwen3_0_6b_decode":
        out = run_decode(args) if args.impl == "ours" else run_decode_reference(args)
    else:
        out = run_reference(args) if args.impl == "reference" else run_ours(args)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
