"""Size-independent properties at the benchmark's full shapes (SmolLM2-360M, 32 rows x 1023
positions), where the CPU oracle would take minutes: linearity of the GEMM, causality and
batch-independence of attention, the attention backward against a finite difference of the forward
along a random direction, AdamW / clip invariants on the full parameter count."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from emberlm_b200 import ops
    return ops


@pytest.mark.parametrize("ta,tb,M,N,Kd", [(False, True, 32736, 2560, 960), (False, False, 32736, 960, 5120),
                                          (True, False, 5120, 960, 32736)])
def test_gemm_linearity_and_exact_integers_full_size(K, ta, tb, M, N, Kd):
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randint(-2, 3, (Kd, M) if ta else (M, Kd), generator=g, device="cuda").float()
    b = torch.randint(-2, 3, (N, Kd) if tb else (Kd, N), generator=g, device="cuda").float()
    c = K.matmul(a, b, ta, tb)
    # exact: small integers are TF32-representable and sums stay below 2^24
    rows = torch.randint(0, M, (64,), generator=g, device="cuda")
    A = (a.t() if ta else a)[rows].double()
    Bm = (b.t() if tb else b).double()
    assert torch.equal(c[rows].double(), A @ Bm)
    # linearity: (2a) b == 2 (a b) exactly (powers of two)
    assert torch.equal(K.matmul(a * 2, b, ta, tb), c * 2)


def test_attention_causality_batch_independence_and_backward_fd(K):
    B, T, H, Hk, D = 32, 1023, 15, 5, 64
    g = torch.Generator(device="cuda").manual_seed(1)
    qkv = torch.randn(B * T, (H + 2 * Hk) * D, generator=g, device="cuda") * 0.5
    out, lse = K.attention(qkv, B, T, H, Hk, D)
    assert torch.isfinite(out).all() and torch.isfinite(lse).all()
    # determinism: the same launch twice gives the same bits (a missed wait shows up here first)
    out_b, lse_b = K.attention(qkv, B, T, H, Hk, D)
    assert torch.equal(out, out_b) and torch.equal(lse, lse_b)
    # causality: changing tokens >= 700 of every row leaves outputs of earlier positions unchanged
    q2 = qkv.clone().view(B, T, -1)
    q2[:, 700:] += 1.0
    out2, _ = K.attention(q2.view(B * T, -1).contiguous(), B, T, H, Hk, D)
    o1, o2 = out.view(B, T, -1), out2.view(B, T, -1)
    assert torch.equal(o1[:, :700], o2[:, :700]) and not torch.equal(o1[:, 700:], o2[:, 700:])
    # batch independence: row 5 alone gives the same result
    o5, _ = K.attention(qkv.view(B, T, -1)[5].contiguous(), 1, T, H, Hk, D)
    assert torch.equal(o5, o1[5])
    # backward: <dO, O(x + e v) - O(x - e v)> / 2e == <dx, v>. The direction is the gradient itself
    # (unit rms): along a random direction <dx, v> is a near-cancelling sum of the size of the
    # finite difference's own TF32 rounding noise, which made the comparison a coin toss.
    dout = torch.randn(B * T, H * D, generator=g, device="cuda")
    dqkv = K.attention_backward(qkv, out, dout, lse, B, T, H, Hk, D)
    assert torch.isfinite(dqkv).all()
    v = dqkv / dqkv.std()
    e = 1e-2
    op, _ = K.attention((qkv + e * v).contiguous(), B, T, H, Hk, D)
    om_, _ = K.attention((qkv - e * v).contiguous(), B, T, H, Hk, D)
    fd = float(((op - om_).double() * dout.double()).sum() / (2 * e))
    an = float((dqkv.double() * v.double()).sum())
    assert abs(fd - an) <= 1e-2 * abs(an), (fd, an)
    # the three parts of the gradient separately (a part that lost contributions would show here)
    for lo, hi in ((0, H * D), (H * D, (H + Hk) * D), ((H + Hk) * D, (H + 2 * Hk) * D)):
        vp = torch.zeros_like(v)
        vp[:, lo:hi] = v[:, lo:hi]
        op, _ = K.attention((qkv + e * vp).contiguous(), B, T, H, Hk, D)
        om_, _ = K.attention((qkv - e * vp).contiguous(), B, T, H, Hk, D)
        fd = float(((op - om_).double() * dout.double()).sum() / (2 * e))
        an = float((dqkv.double() * vp.double()).sum())
        assert abs(fd - an) <= 1e-2 * abs(an), (lo, fd, an)


def test_adamw_and_clip_invariants_full_parameter_count(K):
    n = 361821120
    g = torch.Generator(device="cuda").manual_seed(2)
    p = torch.randn(n, generator=g, device="cuda") * 0.02
    grad = torch.randn(n, generator=g, device="cuda") * 1e-3
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    p0 = p.clone()
    norm, scale = K.clip_grad_norm_([grad], 1.0)
    ref_norm = float(grad.double().norm())
    assert abs(float(norm) - ref_norm) <= 1e-4 * ref_norm
    assert abs(float(scale) - 1.0 / (ref_norm + 1e-6)) <= 1e-5
    K.adamw_step(p, grad, m, v, 1, 1e-4, 0.9, 0.999, 1e-8, 0.0, grad_scale=scale)
    # first step: |update| = lr * |g|/(|g| + eps) <= lr, sign opposite to the gradient
    d = p - p0
    assert float(d.abs().max()) <= 1.0001e-4
    big = grad.abs() > 1e-5
    assert bool((torch.sign(d[big]) == -torch.sign(grad[big])).all())
    assert torch.allclose(m, 0.1 * grad * scale, rtol=1e-5, atol=0) and bool((v >= 0).all())
