"""Parity of every ctdk kernel against the numpy oracle, through the C-ABI (ctypes), on a GPU.
Tolerances: exact-fp32 kernels 1e-5..1e-4 as the reference's own op tests
(tests/test_*.cpp there); TF32 tensor-core kernels relative to the largest reference entry."""
import math

import numpy as np
import pytest
import torch

from oracle import ops as oo

pytestmark = pytest.mark.gpu
F32 = np.float32


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def rnd(shape, seed, lo=-1.0, hi=1.0):
    return np.random.default_rng(seed).uniform(lo, hi, size=shape).astype(F32)


@pytest.fixture(scope="module")
def K():
    from emberlm_b200 import ops
    return ops


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    from emberlm_b200 import lib
    torch.cuda.synchronize()
    w = (lib.C.c_int * 4)()
    rc = lib.raw().ctdk_device_status(None, w)
    assert rc == 0, lib.last_error()


def relmax(got, ref, floor=1e-30):
    """max|got-ref| / max(max|ref|, floor); `floor` is the magnitude of the operands when the
    exact answer may be (near) zero."""
    return float(np.abs(got.astype(np.float64) - ref).max() / max(np.abs(ref).max(), floor))


# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [0, 1, 3, 1027, 1 << 20])
def test_elementwise(K, n):
    a, b = rnd((n,), 1), rnd((n,), 2)
    A, B = dev(a), dev(b)
    assert np.array_equal(host(K.add(A, B)), a + b)
    assert np.array_equal(host(K.sub(A, B)), a - b)
    assert np.array_equal(host(K.mul(A, B)), a * b)
    assert np.array_equal(host(K.scale(A, 0.37)), F32(0.37) * a)
    np.testing.assert_allclose(host(K.silu(A)), oo.silu(a, np.float64), atol=1e-5)
    np.testing.assert_allclose(host(K.silu_backward(A, B)), oo.silu_backward(a, b, np.float64), atol=1e-5)


def test_elementwise_unaligned_and_errors(K):
    a = dev(rnd((1030,), 3))
    got = K.add(a[1:1028].clone(), a[2:1029].clone())  # clones are aligned; views below are not
    assert np.array_equal(host(got), host(a[1:1028]) + host(a[2:1029]))
    from emberlm_b200 import lib
    out = torch.empty(1027, device="cuda")
    lib.call("ctdk_add", a[1:].data_ptr(), a[2:].data_ptr(), out.data_ptr(), 1027, None)
    assert np.array_equal(host(out), host(a[1:1028]) + host(a[2:1029]))
    with pytest.raises(RuntimeError):
        K.add(a[:4], a[:5])
    with pytest.raises(RuntimeError):
        K.add(a[:4].cpu(), a[:4].cpu())


def test_swiglu(K):
    rows, I = 37, 1536
    gu, d = rnd((rows, 2 * I), 4, -3, 3), rnd((rows, I), 5)
    g, u = gu[:, :I], gu[:, I:]
    np.testing.assert_allclose(host(K.swiglu(dev(gu))), oo.silu(g, np.float64) * u, atol=1e-5)
    dgu = host(K.swiglu_backward(dev(gu), dev(d)))
    np.testing.assert_allclose(dgu[:, :I], oo.silu_backward(g, (d * u).astype(F32), np.float64), atol=1e-5)
    np.testing.assert_allclose(dgu[:, I:], d * oo.silu(g, np.float64), atol=1e-5)


# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,H", [(1, 576), (5, 576), (1000, 960), (33, 1024), (17, 2048), (9, 4096),
                                    (64, 128), (7, 64), (3, 6), (4, 4100), (2, 8192)])
def test_rms_norm_forward_backward(K, rows, H):
    x, w, dy = rnd((rows, H), 6), rnd((H,), 7, 0.5, 1.5), rnd((rows, H), 8)
    y, rstd = K.rms_norm(dev(x), dev(w), 1e-5, return_rstd=True)
    ref = oo.rms_norm(x, w, 1e-5, np.float64)
    np.testing.assert_allclose(host(y), ref, atol=1e-4, rtol=1e-5)   # tests/test_norm.cpp: 1e-4
    xs = x.astype(np.float64)
    np.testing.assert_allclose(host(rstd), 1 / np.sqrt((xs * xs).mean(-1) + 1e-5), rtol=1e-5)
    dx, dw = K.rms_norm_backward(dev(dy), dev(x), dev(w), 1e-5)
    rdx, rdw = oo.rms_norm_backward(dy, x, w, 1e-5, np.float64)
    np.testing.assert_allclose(host(dx), rdx, atol=1e-4, rtol=1e-4)
    np.testing.assert_allclose(host(dw), rdw, atol=1e-4 * math.sqrt(rows), rtol=1e-4)


def test_rms_norm_backward_accumulates(K):
    rows, H = 300, 960
    x, w, dy = rnd((rows, H), 9), rnd((H,), 10, 0.5, 1.5), rnd((rows, H), 11)
    base_dx, base_dw = rnd((rows, H), 12), rnd((H,), 13)
    dx, dw = dev(base_dx), dev(base_dw)
    K.rms_norm_backward(dev(dy), dev(x), dev(w), 1e-5, dx=dx, dw=dw, accumulate_dw=True, add_to_dx=True)
    rdx, rdw = oo.rms_norm_backward(dy, x, w, 1e-5, np.float64)
    np.testing.assert_allclose(host(dx), base_dx + rdx, atol=1e-4)
    np.testing.assert_allclose(host(dw), base_dw + rdw, atol=2e-3)


def test_rms_norm_empty_and_errors(K):
    y = K.rms_norm(torch.empty(0, 64, device="cuda"), torch.ones(64, device="cuda"), 1e-5)
    assert y.shape == (0, 64)
    with pytest.raises(RuntimeError):
        K.rms_norm(torch.ones(2, 64, device="cuda"), torch.ones(32, device="cuda"), 1e-5)


# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("pos,theta,scaling", [(0, 100000.0, None), (7, 10000.0, None),
                                               (0, 500000.0, dict(factor=32.0, original_max_pos=8192)),
                                               (4000, 1000000.0, None)])
def test_rope(K, pos, theta, scaling):
    x = rnd((2, 9, 3, 64), 14)
    kw = {}
    if scaling:
        kw = dict(scaling_factor=scaling["factor"], low_freq_wavelen=8192.0, high_freq_wavelen=2048.0)
    np.testing.assert_allclose(host(K.rope(dev(x), pos, theta, scaling)), oo.rope(x, pos, theta, 1.0, **kw),
                               atol=1e-4)                                  # tests/test_rope.cpp: 1e-4
    np.testing.assert_allclose(host(K.rope(dev(x), pos, theta, scaling, sin_sign=-1.0)),
                               oo.rope(x, pos, theta, -1.0, **kw), atol=1e-4)
    c, s = oo.rope_cos_sin(9, 64, pos, theta, **kw)
    tab = host(K.rope_table(9, 64, pos, theta, scaling))
    np.testing.assert_allclose(tab[..., 0], c, atol=2e-4 if pos else 1e-5)
    np.testing.assert_allclose(tab[..., 1], s, atol=2e-4 if pos else 1e-5)


@pytest.mark.parametrize("D,norm", [(64, False), (64, True), (128, True), (128, False)])
def test_qk_norm_rope_forward_backward(K, D, norm):
    B, T, H, Hk = 2, 11, 4, 2
    HT = H + 2 * Hk
    qkv, dq = rnd((B * T, HT * D), 15), rnd((B * T, HT * D), 16)
    wq, wk = rnd((D,), 17, 0.5, 1.5), rnd((D,), 18, 0.5, 1.5)
    theta, eps = 1e6, 1e-6
    tab = K.rope_table(T, D, 0, theta)
    out, rq, rk = K.qk_norm_rope(dev(qkv), B, T, H, Hk, D, tab, dev(wq) if norm else None,
                                 dev(wk) if norm else None, eps)
    x4 = qkv.reshape(B, T, HT, D)
    q, k, v = x4[:, :, :H], x4[:, :, H:H + Hk], x4[:, :, H + Hk:]
    qn = oo.rms_norm(q, wq, eps, np.float64) if norm else q
    kn = oo.rms_norm(k, wk, eps, np.float64) if norm else k
    ref = np.concatenate([oo.rope(qn, 0, theta), oo.rope(kn, 0, theta), v], axis=2).reshape(B * T, -1)
    np.testing.assert_allclose(host(out), ref, atol=2e-4)
    g4 = dq.reshape(B, T, HT, D)
    gq, gk = oo.rope(g4[:, :, :H], 0, theta, -1.0), oo.rope(g4[:, :, H:H + Hk], 0, theta, -1.0)
    if norm:
        gq, rdwq = oo.rms_norm_backward(gq, q, wq, eps, np.float64)
        gk, rdwk = oo.rms_norm_backward(gk, k, wk, eps, np.float64)
    rref = np.concatenate([gq, gk, g4[:, :, H + Hk:]], axis=2).reshape(B * T, -1)
    d, dwq, dwk = K.qk_norm_rope_backward(dev(dq), dev(qkv), B, T, H, Hk, D, tab, dev(wq) if norm else None,
                                          dev(wk) if norm else None, rq, rk)
    np.testing.assert_allclose(host(d), rref, atol=5e-4)
    if norm:
        np.testing.assert_allclose(host(dwq), rdwq, atol=2e-3)
        np.testing.assert_allclose(host(dwk), rdwk, atol=2e-3)


# ---------------------------------------------------------------------------------------
def ints(shape, seed, lim=3):
    return np.random.default_rng(seed).integers(-lim, lim + 1, size=shape).astype(F32)


GEMM_SHAPES = [(128, 256, 32), (128, 128, 64), (2044, 576, 576), (300, 960, 1536), (1, 192, 576),
               (257, 1600, 960), (130, 64, 96), (64, 8, 8), (515, 320, 100), (200, 1000, 36),
               (192, 576, 3000), (576, 200, 2044), (960, 960, 8192),   # few tiles, long K: split-K
               (2048, 512, 256), (4093, 1600, 960), (1300, 5120, 96)]  # large outputs: paired-CTA kernel


@pytest.mark.parametrize("M,N,K_", GEMM_SHAPES)
@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
def test_gemm_exact_on_small_integers(K, M, N, K_, ta, tb):
    """Inputs representable in TF32 and sums below 2^24: any tile/layout/descriptor mistake
    shows as a wrong integer, independent of rounding."""
    a = ints((K_, M) if ta else (M, K_), 20)
    b = ints((N, K_) if tb else (K_, N), 21)
    ref = (a.T if ta else a).astype(np.float64) @ (b.T if tb else b).astype(np.float64)
    got = host(K.matmul(dev(a), dev(b), ta, tb))
    assert np.array_equal(got, ref.astype(F32))


@pytest.mark.parametrize("M,N,K_", [(2044, 576, 576), (300, 2560, 960), (960, 2560, 2047)])
@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False)])
def test_gemm_tf32_accuracy(K, M, N, K_, ta, tb):
    a = rnd((K_, M) if ta else (M, K_), 22)
    b = rnd((N, K_) if tb else (K_, N), 23)
    ref = (a.T if ta else a).astype(np.float64) @ (b.T if tb else b).astype(np.float64)
    got = host(K.matmul(dev(a), dev(b), ta, tb))
    assert relmax(got, ref) < 3e-3          # TF32 inputs (10-bit mantissa), fp32 accumulate


def test_gemm_epilogues_and_fallbacks(K):
    from emberlm_b200 import lib
    a, b = ints((200, 96), 24), ints((320, 96), 25)
    base = ints((200, 320), 26)
    ref = a.astype(np.float64) @ b.T
    c = dev(base.copy())
    K.matmul(dev(a), dev(b), False, True, out=c, epilogue=lib.EPI_ACCUMULATE)
    assert np.array_equal(host(c), (ref + base).astype(F32))
    c2 = K.matmul(dev(a), dev(b), False, True, epilogue=lib.EPI_RESIDUAL, aux=dev(base))
    assert np.array_equal(host(c2), (ref + base).astype(F32))
    # split-K shapes (few output tiles, long K) with every epilogue
    a5, b5, base5 = ints((4000, 192), 40), ints((4000, 320), 41), ints((192, 320), 42)
    ref5 = a5.T.astype(np.float64) @ b5
    assert np.array_equal(host(K.matmul(dev(a5), dev(b5), True, False)), ref5.astype(F32))
    c5 = dev(base5.copy())
    K.matmul(dev(a5), dev(b5), True, False, out=c5, epilogue=lib.EPI_ACCUMULATE)
    assert np.array_equal(host(c5), (ref5 + base5).astype(F32))
    c6 = K.matmul(dev(a5), dev(b5), True, False, epilogue=lib.EPI_RESIDUAL, aux=dev(base5))
    assert np.array_equal(host(c6), (ref5 + base5).astype(F32))
    # paired-CTA kernel: few tiles with long K (split-K) and a partly empty last round, every epilogue
    for (m7, n7, k7, ta7, tb7) in [(512, 512, 4096, True, False), (4092, 960, 960, False, True), (4092, 1600, 960, False, False)]:
        a7 = ints((k7, m7) if ta7 else (m7, k7), 43)
        b7 = ints((n7, k7) if tb7 else (k7, n7), 44)
        base7 = ints((m7, n7), 45)
        ref7 = (a7.T if ta7 else a7).astype(np.float64) @ (b7.T if tb7 else b7).astype(np.float64)
        assert np.array_equal(host(K.matmul(dev(a7), dev(b7), ta7, tb7)), ref7.astype(F32))
        c7 = dev(base7.copy())
        K.matmul(dev(a7), dev(b7), ta7, tb7, out=c7, epilogue=lib.EPI_ACCUMULATE)
        assert np.array_equal(host(c7), (ref7 + base7).astype(F32))
        c8 = K.matmul(dev(a7), dev(b7), ta7, tb7, epilogue=lib.EPI_RESIDUAL, aux=dev(base7))
        assert np.array_equal(host(c8), (ref7 + base7).astype(F32))
    # SIMT path: odd leading dimensions, exact fp32 (tests/test_matmul.cpp tolerance 1e-4)
    a3, b3 = rnd((5, 7), 27), rnd((7, 6), 28)
    np.testing.assert_allclose(host(K.matmul(dev(a3), dev(b3))), a3 @ b3, atol=1e-5)
    a4, b4 = rnd((200, 96), 29), rnd((320, 96), 30)
    got = host(K.matmul(dev(a4), dev(b4), False, True, precision=lib.GEMM_FP32_SIMT))
    np.testing.assert_allclose(got, a4.astype(np.float64) @ b4.T, atol=2e-5)
    got = host(K.matmul(dev(a4), dev(b4), False, True, precision=lib.GEMM_3XTF32))
    np.testing.assert_allclose(got, a4.astype(np.float64) @ b4.T, atol=2e-5)
    with pytest.raises(RuntimeError):
        K.matmul(dev(a3), dev(a3))
    # K == 0 and empty outputs
    z = K.matmul(torch.empty(4, 0, device="cuda"), torch.empty(0, 8, device="cuda"))
    assert z.shape == (4, 8) and float(z.abs().sum()) == 0.0


def test_bmm(K):
    a, b = ints((3, 40, 64), 31), ints((3, 72, 64), 32)
    got = host(K.bmm(dev(a), dev(b), False, True))
    assert np.array_equal(got, np.matmul(a.astype(np.float64), np.swapaxes(b, 1, 2)).astype(F32))


# ---------------------------------------------------------------------------------------
def split_qkv(qkv, B, T, H, Hk, D):
    x4 = qkv.reshape(B, T, H + 2 * Hk, D)
    return (np.ascontiguousarray(x4[:, :, :H]), np.ascontiguousarray(x4[:, :, H:H + Hk]),
            np.ascontiguousarray(x4[:, :, H + Hk:]))


@pytest.mark.parametrize("B,T,H,Hk,D", [(1, 1, 2, 1, 64), (2, 63, 4, 2, 64), (1, 64, 3, 1, 64),
                                        (2, 65, 3, 3, 64), (1, 200, 4, 2, 128), (2, 130, 2, 1, 128),
                                        (1, 257, 9, 3, 64)])
def test_attention_forward_backward(K, B, T, H, Hk, D):
    qkv = rnd((B * T, (H + 2 * Hk) * D), 33, -1.5, 1.5)
    dout = rnd((B * T, H * D), 34)
    q, k, v = split_qkv(qkv, B, T, H, Hk, D)
    ref, probs = oo.attention_train(q, k, v, H // Hk, np.float64)
    out, lse = K.attention(dev(qkv), B, T, H, Hk, D)
    assert relmax(host(out), ref.reshape(B * T, H * D)) < 4e-3
    rdq, rdk, rdv = oo.attention_train_backward(dout.reshape(B, T, H * D), q, k, v, probs, H // Hk, np.float64)
    rref = np.concatenate([rdq, rdk, rdv], axis=2).reshape(B * T, -1)
    dqkv = host(K.attention_backward(dev(qkv), out, dev(dout), lse, B, T, H, Hk, D))
    HD, KD = H * D, Hk * D
    # T == 1 has dq = dk = 0 exactly; the floor keeps the TF32 rounding of dP there in scale
    assert relmax(dqkv[:, :HD], rref[:, :HD], 0.1) < 6e-3
    assert relmax(dqkv[:, HD:HD + KD], rref[:, HD:HD + KD], 0.1) < 8e-3
    assert relmax(dqkv[:, HD + KD:], rref[:, HD + KD:], 0.1) < 6e-3


def test_attention_is_causal(K):
    """Changing a later token must not change earlier outputs (tests/test_mask.cpp's triangle)."""
    B, T, H, Hk, D = 1, 100, 2, 1, 64
    qkv = rnd((B * T, (H + 2 * Hk) * D), 35)
    o1, _ = K.attention(dev(qkv), B, T, H, Hk, D)
    qkv2 = qkv.copy()
    qkv2[70:] += 1.0
    o2, _ = K.attention(dev(qkv2), B, T, H, Hk, D)
    assert torch.equal(o1[:70], o2[:70]) and not torch.equal(o1[70:], o2[70:])


# ---------------------------------------------------------------------------------------
def test_embedding(K):
    V, H = 50, 96
    W = rnd((V, H), 36)
    ids = np.array([[1, 3, 1, 49], [0, 3, 3, 7]], dtype=np.int64)
    assert np.array_equal(host(K.embedding(dev(ids), dev(W))), W[ids])    # tests/test_embedding.cpp: exact
    dy = rnd((2, 4, H), 37)
    np.testing.assert_allclose(host(K.embedding_backward(dev(ids), dev(dy), V)),
                               oo.embedding_backward(ids, dy, V, np.float64), atol=1e-6)
    base = dev(rnd((V, H), 38))
    want = host(base) + oo.embedding_backward(ids, dy, V, np.float64)
    np.testing.assert_allclose(host(K.embedding_backward(dev(ids), dev(dy), V, out=base)), want, atol=1e-6)


@pytest.mark.parametrize("n,V", [(5, 7), (64, 49152), (33, 1001), (3, 151936)])
def test_cross_entropy_masked(K, n, V):
    z = rnd((n, V), 39, -4, 4)
    t = np.random.default_rng(40).integers(0, V, size=n).astype(np.int64)
    mk = (np.arange(n) % 3 != 1).astype(F32)
    loss, dl, ms = K.cross_entropy_masked(dev(z), dev(t), dev(mk), dy=0.25)
    rl, rp, rms = oo.cross_entropy_masked(z, t, mk, np.float64)
    assert abs(float(loss) - float(rl)) < 1e-5 * max(1.0, abs(float(rl)))
    assert float(ms) == float(rms)
    ref = oo.cross_entropy_masked_backward(oo.cross_entropy_masked(z, t, mk, np.float64)[1], t, mk, rms, 0.25)
    got = host(dl)
    np.testing.assert_allclose(got, ref, atol=1e-6)
    assert (got[mk == 0] == 0).all()          # masked rows: exactly zero (test_autograd.cpp:467-474)


def test_cross_entropy_masked_identities_and_zero_sum(K):
    z, t = rnd((5, 7), 11), np.array([0, 3, 6, 2, 1], dtype=np.int64)
    l1, _, _ = K.cross_entropy_masked(dev(z), dev(t), dev(np.ones(5, F32)), want_dlogits=False)
    zz = z.astype(np.float64)
    assert abs(float(l1) - float(np.mean(np.log(np.exp(zz).sum(-1)) - zz[np.arange(5), t]))) < 1e-6
    l0, _, _ = K.cross_entropy_masked(dev(z), dev(t), dev(np.zeros(5, F32)), want_dlogits=False)
    assert float(l0) == 0.0
    with pytest.raises(RuntimeError):
        K.cross_entropy_masked(dev(z), dev(t), dev(np.zeros(5, F32)))


@pytest.mark.parametrize("M,I,K", [(256, 128, 64), (1000, 256, 960), (4092, 2560, 960), (300, 96, 64), (100, 128, 32)])
def test_fused_mlp_input_projection(M, I, K):
    """gate|up GEMM with the SwiGLU activation in its epilogue against the two separate launches:
    the accumulation order per element is the same, so the results are bit-identical; shapes the
    fused kernel does not take (I % 128 != 0, M < 256) go through the same two launches."""
    from emberlm_b200 import ops
    x, w = dev(rnd((M, K), 61)), dev(rnd((2 * I, K), 62, -0.2, 0.2))
    gu, act = ops.mlp_in(x, w, I)
    gu_ref = ops.matmul(x, w, False, True)
    act_ref = ops.swiglu(gu_ref)
    assert torch.equal(gu, gu_ref) and torch.equal(act, act_ref)
    g64 = host(x).astype(np.float64) @ host(w).astype(np.float64).T
    want = g64[:, :I] / (1.0 + np.exp(-g64[:, :I])) * g64[:, I:]
    assert np.abs(host(act) - want).max() <= 2e-2 * max(np.abs(want).max(), 1e-6)   # TF32 inputs


@pytest.mark.parametrize("M,I,K", [(256, 256, 64), (1000, 320, 960), (4092, 2560, 960), (300, 96, 64), (100, 256, 32)])
def test_fused_mlp_input_backward(M, I, K):
    """down_proj dX GEMM with the SwiGLU backward in its epilogue against GEMM + swiglu_backward:
    same accumulation order and the same formulas, so bit-identical."""
    from emberlm_b200 import ops
    dy, wd = dev(rnd((M, K), 63)), dev(rnd((K, I), 64, -0.2, 0.2))
    gu = dev(rnd((M, 2 * I), 65, -3, 3))
    got = ops.mlp_in_backward(dy, wd, gu)
    dact = ops.matmul(dy, wd, False, False)
    want = ops.swiglu_backward(gu, dact)
    assert torch.equal(got, want)


@pytest.mark.parametrize("n,H", [(0, 64), (1, 4), (257, 960), (4099, 576)])
def test_row_gather_scatter_and_ce_input_gather(n, H):
    from emberlm_b200 import lib
    rows = 2 * n + 3
    rng = np.random.default_rng(41)
    idx = np.sort(rng.choice(rows, size=n, replace=False)).astype(np.int32)
    src = rnd((rows, H), 42)
    d_src, d_idx = dev(src), dev(idx)
    out = torch.full((max(n, 1), H), -7.0, device="cuda")
    lib.call("ctdk_gather_rows", d_src.data_ptr(), d_idx.data_ptr(), out.data_ptr(), n, H, None)
    assert np.array_equal(host(out)[:n], src[idx])
    back = torch.zeros(rows, H, device="cuda")
    lib.call("ctdk_scatter_rows", out.data_ptr(), d_idx.data_ptr(), back.data_ptr(), n, H, None)
    want = np.zeros_like(src)
    want[idx] = src[idx]
    assert np.array_equal(host(back), want)
    t = rng.integers(0, 1000, size=rows).astype(np.int64)
    m, w = rnd(rows, 43), rnd(rows, 44)
    to = torch.zeros(max(n, 1), dtype=torch.int64, device="cuda")
    mo, wo = torch.zeros(max(n, 1), device="cuda"), torch.zeros(max(n, 1), device="cuda")
    d_t, d_m, d_w = dev(t), dev(m), dev(w)
    lib.call("ctdk_gather_ce_inputs", d_t.data_ptr(), d_m.data_ptr(), d_w.data_ptr(), d_idx.data_ptr(),
             to.data_ptr(), mo.data_ptr(), wo.data_ptr(), n, None)
    assert np.array_equal(host(to)[:n], t[idx]) and np.array_equal(host(mo)[:n], m[idx])
    assert np.array_equal(host(wo)[:n], w[idx])


# ---------------------------------------------------------------------------------------
def test_adamw_closed_form_and_weight_decay(K):
    from tests import ref_cases as rc
    p, g = dev(np.array([1.0], F32)), dev(np.array([0.1], F32))
    m, v = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    e1, e2 = rc.adamw_closed_form_two_steps()
    K.adamw_step(p, g, m, v, 1, 0.01, 0.9, 0.999, 1e-8, 0.0)
    assert abs(float(p) - e1) < 1e-5
    K.adamw_step(p, g, m, v, 2, 0.01, 0.9, 0.999, 1e-8, 0.0)
    assert abs(float(p) - e2) < 1e-5
    p2 = dev(np.array([1.0], F32))
    K.adamw_step(p2, torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda"),
                 1, 0.01, 0.9, 0.999, 1e-8, 0.1)
    assert abs(float(p2) - (1.0 - 0.01 * 0.1)) < 1e-6


@pytest.mark.parametrize("n", [4, 1000, 1 << 20, (1 << 20) + 3])
def test_adamw_matches_oracle_with_segments_and_scale(K, n):
    p0, g, m0, v0 = rnd((n,), 41), rnd((n,), 42), rnd((n,), 43, 0, 0.1), rnd((n,), 44, 0, 0.1)
    n4 = n // 4 * 4
    cut = max(4, (n4 // 3) // 4 * 4)
    seg_end = torch.tensor([cut, n], dtype=torch.int64, device="cuda")
    seg_wd = torch.tensor([0.1, 0.0], device="cuda")
    scale = torch.tensor([0.5], device="cuda")
    p, m, v = dev(p0), dev(m0), dev(v0)
    K.adamw_step(p, dev(g), m, v, 3, 1e-3, 0.9, 0.95, 1e-8, 0.0, grad_scale=scale, seg_end=seg_end, seg_wd=seg_wd)
    gs = (g * F32(0.5)).astype(F32)
    ra, ma, va = oo.adamw_step(p0[:cut], gs[:cut], m0[:cut], v0[:cut], 3, 1e-3, 0.9, 0.95, 1e-8, 0.1)
    rb, mb, vb = oo.adamw_step(p0[cut:], gs[cut:], m0[cut:], v0[cut:], 3, 1e-3, 0.9, 0.95, 1e-8, 0.0)
    np.testing.assert_allclose(host(p), np.concatenate([ra, rb]), atol=1e-6, rtol=1e-6)
    np.testing.assert_allclose(host(m), np.concatenate([ma, mb]), atol=1e-7, rtol=1e-6)
    np.testing.assert_allclose(host(v), np.concatenate([va, vb]), atol=1e-7, rtol=1e-6)


def test_clip_grad_norm(K):
    gs = [torch.ones(2, 2, device="cuda"), torch.ones(3, 3, device="cuda"), torch.ones(4, 4, device="cuda")]
    norm, scale = K.clip_grad_norm_(gs, 1.0)
    assert abs(float(norm) - math.sqrt(29.0)) < 1e-4
    assert abs(float(scale) * math.sqrt(29.0) - 1.0) < 1e-4
    norm, scale = K.clip_grad_norm_([torch.full((2, 2), 0.1, device="cuda")], 1.0)
    assert abs(float(norm) - 0.2) < 1e-5 and float(scale) == 1.0
    big = dev(rnd((3_000_001,), 45))
    assert abs(float(K.sumsq(big)) / float((host(big).astype(np.float64) ** 2).sum()) - 1) < 1e-5


@pytest.mark.parametrize("B,T,H,Hk,D,hid", [(2, 256, 15, 5, 64, 960), (1, 384, 16, 8, 128, 1024), (3, 100, 4, 2, 64, 256),
                                            (1, 64, 4, 4, 64, 128)])
def test_oproj_backward_with_delta(K, B, T, H, Hk, D, hid):
    """The o-proj dX GEMM that also forms delta: d(attention output) equal to the plain GEMM (which may
    cut K in two for few-tile shapes, so equal to fp32 summation order, not bit for bit),
    delta equal to rowsum(dattn * out) (fp64) to fp32 rounding, and the attention backward fed with it
    equal to the one that computes delta itself. The last two shapes take the unfused path (fewer
    than 256 rows)."""
    ops = K
    g = torch.Generator(device="cuda").manual_seed(B * 1000 + T)
    M = B * T
    dy = torch.randn(M, hid, device="cuda", generator=g)
    w = torch.randn(hid, H * D, device="cuda", generator=g) * 0.05
    qkv = torch.randn(M, (H + 2 * Hk) * D, device="cuda", generator=g)
    out, lse = ops.attention(qkv, B, T, H, Hk, D)
    dattn, delta = ops.oproj_backward(dy, w, out, B, T, H, D)
    ref = ops.matmul(dy, w, False, False)
    assert float((dattn - ref).abs().max()) <= 2e-6 * float(ref.abs().max())
    want = (ref.double() * out.double()).view(B, T, H, D).sum(-1).permute(0, 2, 1)
    scale = float(want.abs().max())
    assert float((delta.double() - want).abs().max()) <= 2e-6 * scale + 1e-6
    a = ops.attention_backward(qkv, out, dattn, lse, B, T, H, Hk, D)
    b = ops.attention_backward(qkv, out, dattn, lse, B, T, H, Hk, D, delta=delta)
    assert float((a - b).abs().max()) <= 1e-5 * float(a.abs().max())
