"""Times single ctdk kernels with CUDA events and prints achieved TFLOP/s or GB/s as JSON lines.

  python -m emberlm_b200.kernel_bench gemm --m 32736 --n 2560 --k 960 --tb 1
  python -m emberlm_b200.kernel_bench gemm-step --workload smollm2_360m   # every GEMM shape of a step
  python -m emberlm_b200.kernel_bench attn --b 32 --t 1023 --h 15 --hk 5 --d 64
  python -m emberlm_b200.kernel_bench adamw --n 361821120
  python -m emberlm_b200.kernel_bench rmsnorm --rows 32736 --hid 960
  python -m emberlm_b200.kernel_bench ce --rows 5376 --v 49152
  python -m emberlm_b200.kernel_bench qkrope --b 32 --t 1023 --h 15 --hk 5 --d 64 [--qknorm 1]

Inputs are larger than L2 or an L2-flushing write runs between timed iterations (--flush).
This is also the small case used for ncu captures of one kernel."""
from __future__ import annotations

import argparse
import json

import torch

from . import lib, ops
from .engine import PRESETS


def _time(fn, iters, warmup, flush):
    buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if buf is not None:
            buf.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def bench_gemm(M, N, K, ta, tb, iters, warmup, flush, epilogue=lib.EPI_STORE, precision=lib.GEMM_TF32):
    a = torch.randn((K, M) if ta else (M, K), device="cuda")
    b = torch.randn((N, K) if tb else (K, N), device="cuda")
    c = torch.zeros(M, N, device="cuda")
    aux = torch.zeros(M, N, device="cuda") if epilogue == lib.EPI_RESIDUAL else None
    ms = _time(lambda: ops.matmul(a, b, ta, tb, precision=precision, out=c, epilogue=epilogue, aux=aux),
               iters, warmup, flush)
    return dict(kernel="gemm", M=M, N=N, K=K, transa=int(ta), transb=int(tb), epilogue=epilogue, ms=ms,
                tflops=2.0 * M * N * K / ms / 1e9)


def step_gemm_shapes(cfg, tok):
    hid, I, D = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    H, Hk, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["vocab_size"]
    qkvn, hd = (H + 2 * Hk) * D, H * D
    fwd = [("qkv", tok, qkvn, hid), ("o", tok, hid, hd), ("gate_up", tok, 2 * I, hid), ("down", tok, hid, I)]
    out = []
    for name, m, n, k in fwd:
        out.append((name + ".fwd", m, n, k, False, True))    # Y = X W^T
        out.append((name + ".dx", m, k, n, False, False))    # dX = dY W
        out.append((name + ".dw", n, k, m, True, False))     # dW = dY^T X
    rows = min(tok, max(128, ((1 << 30) // (V * 4)) // 128 * 128))
    out += [("head.fwd", rows, V, hid, False, True), ("head.dx", rows, hid, V, False, False),
            ("head.dw", V, hid, rows, True, False)]
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "gemm-step", "attn", "adamw", "rmsnorm", "ce", "mlp", "qkrope"])
    ap.add_argument("--m", type=int, default=32736)
    ap.add_argument("--n", type=int, default=2560)
    ap.add_argument("--k", type=int, default=960)
    ap.add_argument("--ta", type=int, default=0)
    ap.add_argument("--tb", type=int, default=1)
    ap.add_argument("--epilogue", type=int, default=0)
    ap.add_argument("--workload", default="smollm2_360m")
    ap.add_argument("--tok", type=int, default=32736)
    ap.add_argument("--b", type=int, default=32)
    ap.add_argument("--t", type=int, default=1023)
    ap.add_argument("--h", type=int, default=15)
    ap.add_argument("--hk", type=int, default=5)
    ap.add_argument("--d", type=int, default=64)
    ap.add_argument("--rows", type=int, default=32736)
    ap.add_argument("--hid", type=int, default=960)
    ap.add_argument("--v", type=int, default=49152)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--flush", action="store_true")
    ap.add_argument("--qknorm", type=int, default=0)
    a = ap.parse_args()

    if a.kernel == "gemm":
        print(json.dumps(bench_gemm(a.m, a.n, a.k, bool(a.ta), bool(a.tb), a.iters, a.warmup, a.flush, a.epilogue)))
    elif a.kernel == "gemm-step":
        tot_ms = tot_fl = 0.0
        for name, m, n, k, ta, tb in step_gemm_shapes(PRESETS[a.workload], a.tok):
            r = bench_gemm(m, n, k, ta, tb, a.iters, a.warmup, a.flush)
            r["name"] = name
            tot_ms += r["ms"]
            tot_fl += 2.0 * m * n * k
            print(json.dumps(r))
        print(json.dumps(dict(kernel="gemm-step", layer_plus_head_ms=tot_ms, tflops=tot_fl / tot_ms / 1e9)))
    elif a.kernel == "mlp":
        # gate|up projection + SwiGLU and its backward through the down projection: fused GEMM
        # epilogues against GEMM + elementwise kernel (same results)
        M, I, K = a.tok, a.n, a.hid
        x, w = torch.randn(M, K, device="cuda"), torch.randn(2 * I, K, device="cuda") * 0.05
        dy, wd = torch.randn(M, K, device="cuda"), torch.randn(K, I, device="cuda") * 0.05
        gu = torch.randn(M, 2 * I, device="cuda")
        for name, fn, fl in (
                ("mlp_in fused", lambda: ops.mlp_in(x, w, I), 4.0 * M * I * K),
                ("mlp_in gemm + swiglu", lambda: ops.swiglu(ops.matmul(x, w, False, True)), 4.0 * M * I * K),
                ("mlp_in_backward fused", lambda: ops.mlp_in_backward(dy, wd, gu), 2.0 * M * I * K),
                ("mlp_in_backward gemm + swiglu_backward",
                 lambda: ops.swiglu_backward(gu, ops.matmul(dy, wd, False, False)), 2.0 * M * I * K)):
            ms = _time(fn, a.iters, a.warmup, a.flush)
            print(json.dumps({"kernel": name, "M": M, "I": I, "K": K, "ms": ms, "tflops": fl / ms / 1e9}))
    elif a.kernel == "attn":
        B, T, H, Hk, D = a.b, a.t, a.h, a.hk, a.d
        qkv = torch.randn(B * T, (H + 2 * Hk) * D, device="cuda")
        dout = torch.randn(B * T, H * D, device="cuda")
        out, lse = ops.attention(qkv, B, T, H, Hk, D)
        fl = 2.0 * B * H * T * T * D
        ms = _time(lambda: ops.attention(qkv, B, T, H, Hk, D), a.iters, a.warmup, a.flush)
        print(json.dumps(dict(kernel="attn_fwd", B=B, T=T, H=H, Hk=Hk, D=D, ms=ms, tflops=fl / ms / 1e9)))
        ms = _time(lambda: ops.attention_backward(qkv, out, dout, lse, B, T, H, Hk, D), a.iters, a.warmup, a.flush)
        print(json.dumps(dict(kernel="attn_bwd", B=B, T=T, H=H, Hk=Hk, D=D, ms=ms, tflops=2 * fl / ms / 1e9)))
    elif a.kernel == "adamw":
        n = a.n if a.n > 10_000_000 else 361821120
        p, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
        m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        ms = _time(lambda: ops.adamw_step(p, g, m, v, 1, 1e-4, 0.9, 0.999, 1e-8, 0.01), a.iters, a.warmup, a.flush)
        print(json.dumps(dict(kernel="adamw", n=n, ms=ms, gbs=28.0 * n / ms / 1e6)))
    elif a.kernel == "rmsnorm":
        x, w = torch.randn(a.rows, a.hid, device="cuda"), torch.ones(a.hid, device="cuda")
        dy = torch.randn(a.rows, a.hid, device="cuda")
        ms = _time(lambda: ops.rms_norm(x, w, 1e-5), a.iters, a.warmup, a.flush)
        print(json.dumps(dict(kernel="rmsnorm_fwd", rows=a.rows, H=a.hid, ms=ms, gbs=8.0 * x.numel() / ms / 1e6)))
        dx, dw = torch.empty_like(x), torch.empty_like(w)
        ms = _time(lambda: ops.rms_norm_backward(dy, x, w, 1e-5, dx=dx, dw=dw), a.iters, a.warmup, a.flush)
        print(json.dumps(dict(kernel="rmsnorm_bwd", rows=a.rows, H=a.hid, ms=ms, gbs=12.0 * x.numel() / ms / 1e6)))
    elif a.kernel == "qkrope":
        B, T, H, Hk, D = a.b, a.t, a.h, a.hk, a.d
        qkv = torch.randn(B * T, (H + 2 * Hk) * D, device="cuda")
        dqkv = torch.randn_like(qkv)
        table = ops.rope_table(T, D, 0, 100000.0)
        wq = torch.ones(D, device="cuda") if a.qknorm else None
        wk = torch.ones(D, device="cuda") if a.qknorm else None
        out, rq, rk = ops.qk_norm_rope(qkv, B, T, H, Hk, D, table, wq, wk)
        qk_elems = B * T * (H + Hk) * D
        fwd_bytes = 8.0 * (qk_elems + B * T * Hk * D)            # q, k read + written, v copied (out of place)
        ms = _time(lambda: ops.qk_norm_rope(qkv, B, T, H, Hk, D, table, wq, wk), a.iters, a.warmup, a.flush)
        print(json.dumps(dict(kernel="qk_norm_rope_fwd", B=B, T=T, H=H, Hk=Hk, D=D, qknorm=a.qknorm, ms=ms, gbs=fwd_bytes / ms / 1e6)))
        bwd_bytes = (12.0 if a.qknorm else 8.0) * qk_elems
        ms = _time(lambda: ops.qk_norm_rope_backward(dqkv, qkv, B, T, H, Hk, D, table, wq, wk, rq, rk), a.iters, a.warmup, a.flush)
        print(json.dumps(dict(kernel="qk_norm_rope_bwd", B=B, T=T, H=H, Hk=Hk, D=D, qknorm=a.qknorm, ms=ms, gbs=bwd_bytes / ms / 1e6)))
    elif a.kernel == "ce":
        z = torch.randn(a.rows, a.v, device="cuda")
        t = torch.randint(0, a.v, (a.rows,), device="cuda")
        mk = (torch.arange(a.rows, device="cuda") % 2).float()
        rw = mk / mk.sum()
        sums = torch.zeros(2, device="cuda")
        s = torch.cuda.current_stream().cuda_stream

        def run():
            lib.call("ctdk_ce_masked", z.data_ptr(), t.data_ptr(), mk.data_ptr(), rw.data_ptr(), sums.data_ptr(),
                     None, a.rows, a.v, 1, s)
        ms = _time(run, a.iters, a.warmup, a.flush)
        print(json.dumps(dict(kernel="ce_masked", rows=a.rows, V=a.v, ms=ms, gbs=8.0 * z.numel() / ms / 1e6)))


if __name__ == "__main__":
    main()
