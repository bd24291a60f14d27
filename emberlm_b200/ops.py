"""Host-side mirror of the reference's `ctd::ops` / `ctd::optim` free functions over torch CUDA
tensors (emberlm include/ctd/ops/*.h, include/ctd/optim.h). Same names, argument meaning and
error behaviour (a failed precondition raises, like the reference's std::runtime_error); every
function allocates its output with torch and calls the C-ABI kernel on torch's current stream.
Used by the parity tests and the benchmark; there is no CPU path."""
from __future__ import annotations

import ctypes as C

import torch

from . import lib
from .lib import RopeParams, AdamWParams


def _s() -> int:
    return torch.cuda.current_stream().cuda_stream


def _chk(t: torch.Tensor, name: str, dtype=torch.float32) -> torch.Tensor:
    if not t.is_cuda:
        raise RuntimeError(f"{name}: CUDA only")
    if t.dtype != dtype:
        raise RuntimeError(f"{name}: expected {dtype}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name}: contiguous only")
    return t


def _binary(fn, a, b, name):
    _chk(a, name), _chk(b, name)
    if a.shape != b.shape:
        raise RuntimeError(f"{name}: shape mismatch")
    out = torch.empty_like(a)
    lib.call(fn, a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _s())
    return out


def add(a, b): return _binary("ctdk_add", a, b, "add")
def sub(a, b): return _binary("ctdk_sub", a, b, "sub")
def mul(a, b): return _binary("ctdk_mul", a, b, "mul")


def scale(x, alpha):
    _chk(x, "scale")
    out = torch.empty_like(x)
    lib.call("ctdk_scale", x.data_ptr(), float(alpha), out.data_ptr(), x.numel(), _s())
    return out


mul_scalar = scale


def silu(x):
    _chk(x, "silu")
    out = torch.empty_like(x)
    lib.call("ctdk_silu", x.data_ptr(), out.data_ptr(), x.numel(), _s())
    return out


def silu_backward(x, g):
    _chk(x, "silu_backward"), _chk(g, "silu_backward")
    out = torch.empty_like(x)
    lib.call("ctdk_silu_bwd", x.data_ptr(), g.data_ptr(), out.data_ptr(), x.numel(), _s())
    return out


def mlp_in(x, w_gate_up, I, precision=lib.GEMM_TF32):
    """nn::MLP::forward up to the activation (include/ctd/nn/mlp.h:16-21) in one launch:
    x [M, K], w_gate_up [2I, K] (gate_proj rows then up_proj rows). Returns (gu [M, 2I] = gate | up,
    act [M, I] = silu(gate) * up)."""
    _chk(x, "mlp_in"), _chk(w_gate_up, "mlp_in")
    M, K = x.shape
    if tuple(w_gate_up.shape) != (2 * I, K):
        raise RuntimeError("mlp_in: weight must be [2I, K]")
    gu = torch.empty(M, 2 * I, device=x.device, dtype=x.dtype)
    act = torch.empty(M, I, device=x.device, dtype=x.dtype)
    lib.call("ctdk_gemm_swiglu", x.data_ptr(), w_gate_up.data_ptr(), gu.data_ptr(), act.data_ptr(), M, I, K,
             precision, _s())
    return gu, act


def mlp_in_backward(dy, w_down, gu, precision=lib.GEMM_TF32):
    """d(gate)|d(up) [M, 2I] from dy [M, hid], down_proj.weight [hid, I] and the saved gate|up [M, 2I]."""
    _chk(dy, "mlp_in_backward"), _chk(w_down, "mlp_in_backward"), _chk(gu, "mlp_in_backward")
    M, K = dy.shape
    I = w_down.shape[1]
    if w_down.shape[0] != K or tuple(gu.shape) != (M, 2 * I):
        raise RuntimeError("mlp_in_backward: shape mismatch")
    dgu = torch.empty_like(gu)
    scratch = torch.empty(M, I, device=dy.device, dtype=dy.dtype)
    lib.call("ctdk_gemm_swiglu_bwd", dy.data_ptr(), w_down.data_ptr(), gu.data_ptr(), dgu.data_ptr(),
             scratch.data_ptr(), M, I, K, precision, _s())
    return dgu


def oproj_backward(dy, w_o, attn_out, B, T, H, D, precision=lib.GEMM_TF32):
    """d(attention output) [B*T, H*D] = dy [B*T, hid] @ o_proj.weight [hid, H*D] and delta [B, H, T] =
    rowsum over each head of that product times the attention output (what the attention backward
    needs first), from one GEMM."""
    _chk(dy, "oproj_backward"), _chk(w_o, "oproj_backward"), _chk(attn_out, "oproj_backward")
    M, hid = dy.shape
    if M != B * T or tuple(w_o.shape) != (hid, H * D) or tuple(attn_out.shape) != (M, H * D):
        raise RuntimeError("oproj_backward: shape mismatch")
    dattn = torch.empty_like(attn_out)
    delta = torch.empty(B, H, T, device=dy.device, dtype=dy.dtype)
    lib.call("ctdk_gemm_dattn_delta", dy.data_ptr(), w_o.data_ptr(), attn_out.data_ptr(), dattn.data_ptr(),
             delta.data_ptr(), B, T, H, D, hid, precision, _s())
    return dattn, delta


def swiglu(gu):
    _chk(gu, "swiglu")
    rows, two_i = gu.shape
    out = torch.empty(rows, two_i // 2, device=gu.device, dtype=gu.dtype)
    lib.call("ctdk_swiglu_fwd", gu.data_ptr(), out.data_ptr(), rows, two_i // 2, _s())
    return out


def swiglu_backward(gu, dact):
    _chk(gu, "swiglu_backward"), _chk(dact, "swiglu_backward")
    rows, two_i = gu.shape
    out = torch.empty_like(gu)
    lib.call("ctdk_swiglu_bwd", gu.data_ptr(), dact.data_ptr(), out.data_ptr(), rows, two_i // 2, _s())
    return out


def matmul(a, b, transa=False, transb=False, precision=lib.GEMM_TF32, out=None, epilogue=lib.EPI_STORE,
           aux=None):
    _chk(a, "matmul"), _chk(b, "matmul")
    if a.dim() != 2 or b.dim() != 2:
        raise RuntimeError("matmul: expected 2D tensors")
    M, K = (a.shape[1], a.shape[0]) if transa else (a.shape[0], a.shape[1])
    Kb, N = (b.shape[1], b.shape[0]) if transb else (b.shape[0], b.shape[1])
    if K != Kb:
        raise RuntimeError("matmul: inner dims disagree")
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=a.dtype)
    if precision == lib.GEMM_3XTF32:
        # near-fp32 on the tensor cores: three passes over split operands, needs a workspace
        ws = torch.empty(lib.raw().ctdk_gemm_3xtf32_workspace_floats(M, N, K), device=a.device, dtype=a.dtype)
        lib.call("ctdk_gemm_ws", a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.shape[1], b.shape[1], N,
                 int(transa), int(transb), precision, epilogue, aux.data_ptr() if aux is not None else None,
                 ws.data_ptr(), ws.numel(), _s())
        return out
    lib.call("ctdk_gemm", a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.shape[1], b.shape[1], N,
             int(transa), int(transb), precision, epilogue, aux.data_ptr() if aux is not None else None, _s())
    return out


def bmm(a, b, transa=False, transb=False, precision=lib.GEMM_TF32):
    _chk(a, "bmm"), _chk(b, "bmm")
    if a.dim() != 3 or b.dim() != 3 or a.shape[0] != b.shape[0]:
        raise RuntimeError("bmm: expected 3D tensors with equal batch")
    M, K = (a.shape[2], a.shape[1]) if transa else (a.shape[1], a.shape[2])
    Kb, N = (b.shape[2], b.shape[1]) if transb else (b.shape[1], b.shape[2])
    if K != Kb:
        raise RuntimeError("bmm: inner dims disagree")
    out = torch.empty(a.shape[0], M, N, device=a.device, dtype=a.dtype)
    lib.call("ctdk_bmm", a.data_ptr(), b.data_ptr(), out.data_ptr(), a.shape[0], M, N, K, int(transa),
             int(transb), precision, _s())
    return out


def rms_norm(x, weight, eps, return_rstd=False):
    _chk(x, "rms_norm"), _chk(weight, "rms_norm")
    H = x.shape[-1]
    if weight.numel() != H:
        raise RuntimeError("rms_norm: weight size mismatch")
    rows = x.numel() // H
    y = torch.empty_like(x)
    rstd = torch.empty(rows, device=x.device, dtype=x.dtype) if return_rstd else None
    lib.call("ctdk_rmsnorm_fwd", x.data_ptr(), weight.data_ptr(), y.data_ptr(),
             rstd.data_ptr() if return_rstd else None, rows, H, float(eps), _s())
    return (y, rstd) if return_rstd else y


def rms_norm_backward(dy, x, w, eps, dx=None, dw=None, accumulate_dw=False, add_to_dx=False):
    _chk(dy, "rms_norm_backward"), _chk(x, "rms_norm_backward"), _chk(w, "rms_norm_backward")
    H = x.shape[-1]
    rows = x.numel() // H
    if dx is None:
        dx = torch.empty_like(x)
    if dw is None:
        dw = torch.empty_like(w)
    scratch = torch.empty(lib.raw().ctdk_rmsnorm_bwd_scratch_floats(H), device=x.device, dtype=x.dtype)
    lib.call("ctdk_rmsnorm_bwd", dy.data_ptr(), x.data_ptr(), w.data_ptr(), dx.data_ptr(), dw.data_ptr(),
             scratch.data_ptr(), rows, H, float(eps), int(accumulate_dw), int(add_to_dx), _s())
    return dx, dw


def rope_params(theta, factor=0.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_pos=8192):
    """RopeScaling of include/ctd/ops/rope.h:9-22 flattened for the kernels."""
    return RopeParams(theta, factor, original_max_pos / low_freq_factor, original_max_pos / high_freq_factor)


def rope(x, position_start, theta, scaling=None, sin_sign=1.0, out=None):
    """x: [B,T,H,D] contiguous. sin_sign=-1 gives rope_transpose (the backward)."""
    _chk(x, "rope")
    if x.dim() != 4 or x.shape[-1] % 2:
        raise RuntimeError("rope: expected [B,T,H,D] with even D")
    B, T, H, D = x.shape
    p = rope_params(theta, **(scaling or {}))
    out = torch.empty_like(x) if out is None else out
    lib.call("ctdk_rope", x.data_ptr(), out.data_ptr(), B, T, H, D, H * D, int(position_start), C.byref(p),
             float(sin_sign), _s())
    return out


def rope_table(T, D, position_start, theta, scaling=None, device="cuda"):
    p = rope_params(theta, **(scaling or {}))
    tab = torch.empty(T, D // 2, 2, device=device, dtype=torch.float32)
    lib.call("ctdk_rope_table", tab.data_ptr(), T, D, int(position_start), C.byref(p), _s())
    return tab


def qk_norm_rope(qkv, B, T, H, Hk, D, table, wq=None, wk=None, eps=1e-6):
    _chk(qkv, "qk_norm_rope")
    out = torch.empty_like(qkv)
    rq = torch.empty(B * T * H, device=qkv.device) if wq is not None else None
    rk = torch.empty(B * T * Hk, device=qkv.device) if wq is not None else None
    lib.call("ctdk_qk_norm_rope_fwd", qkv.data_ptr(), out.data_ptr(),
             wq.data_ptr() if wq is not None else None, wk.data_ptr() if wk is not None else None,
             rq.data_ptr() if rq is not None else None, rk.data_ptr() if rk is not None else None,
             table.data_ptr(), B, T, H, Hk, D, float(eps), _s())
    return out, rq, rk


def qk_norm_rope_backward(dqkv, qkv_pre, B, T, H, Hk, D, table, wq=None, wk=None, rq=None, rk=None):
    """In place on dqkv; returns (dqkv, dwq, dwk)."""
    dwq = torch.empty(D, device=dqkv.device) if wq is not None else None
    dwk = torch.empty(D, device=dqkv.device) if wq is not None else None
    scratch = torch.empty(lib.raw().ctdk_qk_norm_rope_bwd_scratch_floats(D), device=dqkv.device)
    lib.call("ctdk_qk_norm_rope_bwd", dqkv.data_ptr(), qkv_pre.data_ptr() if qkv_pre is not None else None,
             wq.data_ptr() if wq is not None else None, wk.data_ptr() if wk is not None else None,
             rq.data_ptr() if rq is not None else None, rk.data_ptr() if rk is not None else None,
             dwq.data_ptr() if dwq is not None else None, dwk.data_ptr() if dwk is not None else None,
             scratch.data_ptr(), table.data_ptr(), B, T, H, Hk, D, 0, _s())
    return dqkv, dwq, dwk


def embedding(ids, weight):
    _chk(ids, "embedding", torch.int64), _chk(weight, "embedding")
    V, H = weight.shape
    out = torch.empty(*ids.shape, H, device=weight.device, dtype=weight.dtype)
    lib.call("ctdk_embedding_fwd", ids.data_ptr(), weight.data_ptr(), out.data_ptr(), ids.numel(), H, V, _s())
    return out


def embedding_backward(ids, dy, vocab, out=None):
    _chk(ids, "embedding_backward", torch.int64), _chk(dy, "embedding_backward")
    H = dy.shape[-1]
    if out is None:
        out = torch.zeros(vocab, H, device=dy.device, dtype=dy.dtype)
    lib.call("ctdk_embedding_bwd", ids.data_ptr(), dy.data_ptr(), out.data_ptr(), ids.numel(), H, vocab, _s())
    return out


def cross_entropy_masked(logits, targets, loss_mask, dy=1.0, want_dlogits=True):
    """Returns (loss [1], dlogits or None, mask_sum). loss = sum(mask*(lse-z_t))/sum(mask), 0 when
    sum(mask) == 0; dlogits = dy/sum(mask) * mask * (softmax - onehot) (loss.cu:254-329,388-411).
    Like the reference's backward, asking for dlogits with sum(mask) == 0 raises."""
    _chk(logits, "cross_entropy_masked"), _chk(targets, "cross_entropy_masked", torch.int64)
    _chk(loss_mask, "cross_entropy_masked")
    if logits.dim() != 2 or targets.shape != (logits.shape[0],) or loss_mask.shape != targets.shape:
        raise RuntimeError("cross_entropy_masked: shape mismatch")
    n, V = logits.shape
    sums = torch.zeros(2, device=logits.device)
    work = logits.clone()
    ms = loss_mask.sum()
    if want_dlogits:
        if not float(ms) > 0:
            raise RuntimeError("cross_entropy_masked: sum(loss_mask) == 0 in backward")
        rw = (loss_mask * (dy / ms)).contiguous()
    else:
        rw = None
    lib.call("ctdk_ce_masked", work.data_ptr(), targets.data_ptr(), loss_mask.data_ptr(),
             rw.data_ptr() if rw is not None else None, sums.data_ptr(), None, n, V, int(want_dlogits), _s())
    loss = torch.where(sums[1] > 0, sums[0] / sums[1], torch.zeros_like(sums[0])).reshape(1)
    return loss, (work if want_dlogits else None), sums[1]


def attention(qkv, B, T, H, Hk, D, precision=lib.GEMM_TF32):
    _chk(qkv, "attention")
    out = torch.empty(B * T, H * D, device=qkv.device)
    lse = torch.empty(B, H, T, device=qkv.device)
    lib.call("ctdk_attn_fwd_p", qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), B, T, H, Hk, D, precision, _s())
    return out, lse


def attention_backward(qkv, out, dout, lse, B, T, H, Hk, D, precision=lib.GEMM_TF32, delta=None):
    """delta: rowsum(dout * out) per (batch, head, position) when oproj_backward has already formed it
    (out is then not read)."""
    dqkv = torch.empty_like(qkv)
    given = delta is not None
    delta = delta if given else torch.empty(B, H, T, device=qkv.device)
    lib.call("ctdk_attn_bwd_p", qkv.data_ptr(), 0 if given else out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
             delta.data_ptr(), dqkv.data_ptr(), B, T, H, Hk, D, precision, _s())
    return dqkv


def sumsq(g, out=None):
    out = torch.zeros(1, device=g.device) if out is None else out
    lib.call("ctdk_sumsq", g.data_ptr(), g.numel(), out.data_ptr(), _s())
    return out


def clip_grad_norm_(grads, max_norm, eps=1e-6):
    """optim::clip_grad_norm_ over a list of gradient tensors: returns (total_norm tensor,
    scale tensor); the scale is meant to be passed to adamw_step rather than applied in place."""
    acc = torch.zeros(3, device=grads[0].device)
    for g in grads:
        sumsq(g, acc)
    lib.call("ctdk_clip_scale", acc.data_ptr(), float(max_norm), float(eps), acc[1:].data_ptr(),
             acc[2:].data_ptr(), _s())
    return acc[2], acc[1]


def adamw_step(p, g, m, v, step, lr, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, grad_scale=None,
               seg_end=None, seg_wd=None):
    """In-place AdamW on flat tensors with the reference's float32 bias corrections
    (src/core/optim.cu:142-143)."""
    import numpy as np
    t = np.float32(step)
    bc1 = float(np.float32(1.0) - np.power(np.float32(beta1), t, dtype=np.float32))
    bc2 = float(np.float32(1.0) - np.power(np.float32(beta2), t, dtype=np.float32))
    hp = AdamWParams(lr, beta1, beta2, eps, weight_decay, bc1, bc2)
    nseg = 0 if seg_end is None else seg_end.numel()
    lib.call("ctdk_adamw", p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(), C.byref(hp),
             grad_scale.data_ptr() if grad_scale is not None else None,
             seg_end.data_ptr() if nseg else None, seg_wd.data_ptr() if nseg else None, nseg, _s())
