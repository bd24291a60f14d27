"""Pins the numpy oracle (CPU only): against the CPU reference functions and known-answer tests
the reference's own test-suite carries, and against an independent fp64 torch-autograd statement
of the model for the hand-written backward."""
import math

import numpy as np
import pytest

from oracle import model as om
from oracle import ops as oo
from tests import ref_cases as rc
from tests import torch_ref

F32 = np.float32


def rnd(shape, seed, lo=-1.0, hi=1.0):
    return np.random.default_rng(seed).uniform(lo, hi, size=shape).astype(F32)


# --- CPU reference functions embedded in the reference's tests ------------------------------
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_matmul_matches_mm_cpu(ta, tb):
    M, K, N = 5, 7, 6  # tests/test_bmm.cpp shapes are of this order; tolerance 1e-4 as there
    a = rnd((K, M) if ta else (M, K), 1)
    b = rnd((N, K) if tb else (K, N), 2)
    np.testing.assert_allclose(oo.matmul(a, b, ta, tb), rc.mm_cpu(a, b, M, K, N, ta, tb), atol=1e-4)


def test_bmm_matches_mm_cpu_per_batch():
    a, b = rnd((3, 4, 5), 3), rnd((3, 6, 5), 4)
    got = oo.bmm(a, b, False, True)
    for i in range(3):
        np.testing.assert_allclose(got[i], rc.mm_cpu(a[i], b[i], 4, 5, 6, False, True), atol=1e-4)


def test_rms_norm_matches_cpu():
    x, w = rnd((5, 576), 5), rnd((576,), 6, 0.5, 1.5)  # tests/test_norm.cpp:26-49: H=576, 1e-4
    np.testing.assert_allclose(oo.rms_norm(x, w, 1e-5), rc.rms_norm_cpu(x, w, 1e-5), atol=1e-4)


def test_softmax_matches_cpu_and_extremes():
    x = rnd((4, 33), 7, -5, 5)
    np.testing.assert_allclose(oo.softmax(x), rc.softmax_cpu(x), atol=1e-5)
    y = oo.softmax(np.array([[1000.0, 1001.0, 999.0]], dtype=F32))  # tests/test_softmax.cpp:54-65
    assert abs(float(y.sum()) - 1.0) < 1e-5 and y[0, 1] > y[0, 0] > y[0, 2]


@pytest.mark.parametrize("pos", [0, 7])
def test_rope_matches_cpu(pos):
    x = rnd((2, 5, 3, 64), 8)  # tests/test_rope.cpp: theta 1e5, D=64, offset case, 1e-4
    np.testing.assert_allclose(oo.rope(x, pos, 100000.0), rc.rope_cpu(x, pos, 100000.0), atol=1e-4)


def test_rope_backward_is_transpose():
    x, g = rnd((1, 6, 2, 64), 9), rnd((1, 6, 2, 64), 10)
    lhs = float((oo.rope(x, 3, 1e4).astype(np.float64) * g).sum())
    rhs = float((x.astype(np.float64) * oo.rope(g, 3, 1e4, sin_sign=-1.0)).sum())
    assert abs(lhs - rhs) < 1e-3


def test_llama3_rope_scaling_branches():
    f0 = oo.rope_freqs(64, 500000.0)
    f = oo.rope_freqs(64, 500000.0, scaling_factor=32.0, low_freq_wavelen=8192.0, high_freq_wavelen=2048.0)
    wl = 6.2831853 / f0
    assert np.allclose(f[wl <= 2048.0], f0[wl <= 2048.0])            # high frequency: unchanged
    assert np.allclose(f[wl > 8192.0], f0[wl > 8192.0] / 32.0)        # low frequency: / factor
    mid = (wl > 2048.0) & (wl <= 8192.0)
    assert mid.any() and np.all(f[mid] < f0[mid]) and np.all(f[mid] > f0[mid] / 32.0)


def test_causal_mask_patterns():
    s = np.zeros((1, 3, 3), dtype=F32)  # tests/test_mask.cpp:11-41
    m = oo.apply_causal_mask(s, 0)
    assert (m[0] == np.array([[0, -oo.FLT_MAX, -oo.FLT_MAX], [0, 0, -oo.FLT_MAX], [0, 0, 0]], dtype=F32)).all()
    d = oo.apply_causal_mask(np.zeros((1, 1, 5), dtype=F32), 4)  # decode: all keys kept
    assert (d == 0).all()


def test_silu_and_backward():
    x, g = rnd((64,), 11, -4, 4), rnd((64,), 12)
    np.testing.assert_allclose(oo.silu(x), x / (1 + np.exp(-x)), atol=1e-6)
    e = 1e-3
    fd = (oo.silu((x + e).astype(F32), np.float64).astype(np.float64) -
          oo.silu((x - e).astype(F32), np.float64)) / (2 * e)
    np.testing.assert_allclose(oo.silu_backward(x, g), g * fd, atol=2e-3)


def test_embedding_backward_repeated_ids():
    ids = np.array([[1, 3, 1]], dtype=np.int64)
    dy = rnd((1, 3, 4), 13)
    dW = oo.embedding_backward(ids, dy, 5)
    np.testing.assert_allclose(dW[1], dy[0, 0] + dy[0, 2], atol=1e-6)
    np.testing.assert_allclose(dW[3], dy[0, 1], atol=1e-6)
    assert (dW[[0, 2, 4]] == 0).all()


# --- masked CE identities (tests/test_autograd.cpp:397-498) ----------------------------------
def test_ce_masked_all_ones_equals_unmasked():
    z, t = rnd((5, 7), 11), np.array([0, 3, 6, 2, 1])
    l1, _, _ = oo.cross_entropy_masked(z, t, np.ones(5, F32))
    zz = z.astype(np.float64)
    l2 = float(np.mean(np.log(np.exp(zz).sum(-1)) - zz[np.arange(5), t]))
    assert abs(float(l1) - l2) < 1e-6


def test_ce_masked_half_equals_subset():
    z, t = rnd((5, 7), 17), np.array([1, 4, 0, 6, 3])
    mk = np.array([1, 0, 1, 0, 1], dtype=F32)
    l1, _, _ = oo.cross_entropy_masked(z, t, mk)
    l2, _, _ = oo.cross_entropy(z[[0, 2, 4]], t[[0, 2, 4]])
    assert abs(float(l1) - float(l2)) < 1e-5


def test_ce_masked_backward_fd_and_exact_zero_rows():
    z, t = rnd((4, 5), 23), np.array([2, 0, 4, 1])
    mk = np.array([1, 0, 1, 1], dtype=F32)
    _, p, ms = oo.cross_entropy_masked(z, t, mk)
    g = oo.cross_entropy_masked_backward(p, t, mk, ms)
    assert (g[1] == 0).all()
    e = 1e-3
    for i in range(4):
        for j in range(5):
            zp, zm = z.copy(), z.copy()
            zp[i, j] += e
            zm[i, j] -= e
            fd = (float(oo.cross_entropy_masked(zp, t, mk, np.float64)[0]) -
                  float(oo.cross_entropy_masked(zm, t, mk, np.float64)[0])) / (2 * e)
            assert abs(fd - g[i, j]) < 1e-3


def test_ce_masked_zero_sum():
    z, t = rnd((3, 4), 31), np.zeros(3, dtype=np.int64)
    l, p, ms = oo.cross_entropy_masked(z, t, np.zeros(3, F32))
    assert float(l) == 0.0
    with pytest.raises(RuntimeError):
        oo.cross_entropy_masked_backward(p, t, np.zeros(3, F32), ms)


# --- optimizer known answers (tests/test_autograd.cpp:530-597, 649-685) ----------------------
def test_adamw_closed_form_two_steps():
    p, m, v = np.array([1.0], F32), np.zeros(1, F32), np.zeros(1, F32)
    g = np.array([0.1], F32)
    e1, e2 = rc.adamw_closed_form_two_steps()
    p, m, v = oo.adamw_step(p, g, m, v, 1, 0.01, 0.9, 0.999, 1e-8, 0.0)
    assert abs(float(p[0]) - e1) < 1e-5
    p, m, v = oo.adamw_step(p, g, m, v, 2, 0.01, 0.9, 0.999, 1e-8, 0.0)
    assert abs(float(p[0]) - e2) < 1e-5


def test_adamw_decoupled_weight_decay_zero_grad():
    p, m, v = oo.adamw_step(np.array([1.0], F32), np.zeros(1, F32), np.zeros(1, F32), np.zeros(1, F32),
                            1, 0.01, 0.9, 0.999, 1e-8, 0.1)
    assert abs(float(p[0]) - (1.0 - 0.01 * 0.1)) < 1e-6


def test_clip_scales_to_max_and_noop_under_max():
    gs = [np.ones((2, 2), F32), np.ones((3, 3), F32), np.ones((4, 4), F32)]
    norm, out = oo.clip_grad_norm(gs, 1.0)
    assert abs(float(norm) - math.sqrt(29.0)) < 1e-4
    assert abs(math.sqrt(sum(float((o * o).sum()) for o in out)) - 1.0) < 1e-4
    g = [np.full((2, 2), 0.1, F32)]
    norm, out = oo.clip_grad_norm(g, 1.0)
    assert abs(float(norm) - 0.2) < 1e-5 and (out[0] == g[0]).all()


def test_lr_schedule_constant_when_warmup0_ratio1():
    assert all(float(oo.lr_at_step(s, 1e-4, 0, 13, 1.0)) == float(F32(1e-4)) for s in range(1, 14))
    assert float(oo.lr_at_step(5, 3e-4, 10, 100, 0.1)) == pytest.approx(1.5e-4)


# --- the model backward vs independent fp64 autograd ------------------------------------------
def tiny_cfg(**kw):
    base = dict(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                num_attention_heads=2, num_key_value_heads=1, head_dim=64, rms_norm_eps=1e-5,
                rope_theta=10000.0)
    base.update(kw)
    return om.LlamaConfig(**base)


@pytest.mark.parametrize("kw", [dict(), dict(qk_norm=True, rms_norm_eps=1e-6),
                                dict(rope_scaling_factor=32.0, rope_theta=500000.0,
                                     rope_scaling_original_max_pos=16)])
def test_oracle_model_backward_matches_fp64_autograd(kw):
    cfg = tiny_cfg(**kw)
    params = om.init_params(cfg, seed=5, std=0.05)
    for k in params:  # move norm weights off 1.0 so their gradients are exercised
        if params[k].ndim == 1:
            params[k] = (params[k] + rnd(params[k].shape, 99, -0.2, 0.2)).astype(F32)
    tok, msk = om.synth_batch(cfg.vocab_size, 3, 20, seed=3)
    msk[:, 5:12] = 1
    ids, tgt, m = om.make_batch(tok, msk, [0, 2])
    loss, ms, grads = om.forward_backward(params, cfg, ids, tgt, m, dy=0.5, acc=np.float64)
    ref_loss, ref_grads = torch_ref.loss_and_grads(params, cfg, ids, tgt, m, dy=0.5)
    assert abs(float(loss) - ref_loss) < 1e-5 * abs(ref_loss)
    assert float(ms) == float(m.sum())
    for k, g in grads.items():
        ref = ref_grads[k]
        err = np.abs(g - ref).max() / max(np.abs(ref).max(), 1e-12)
        assert err < 1e-4, (k, err)


def test_oracle_f32_close_to_f64():
    cfg = tiny_cfg()
    params = om.init_params(cfg, seed=6, std=0.05)
    tok, msk = om.synth_batch(cfg.vocab_size, 2, 24, seed=4)
    ids, tgt, m = om.make_batch(tok, msk, [0, 1])
    l32, _, g32 = om.forward_backward(params, cfg, ids, tgt, m)
    l64, _, g64 = om.forward_backward(params, cfg, ids, tgt, m, acc=np.float64)
    assert abs(float(l32) - float(l64)) < 1e-5 * abs(float(l64))
    for k in g32:
        assert np.abs(g32[k] - g64[k]).max() <= 2e-4 * max(np.abs(g64[k]).max(), 1e-12), k


def test_micro_batch_weighting_equals_reference_loop():
    """Summed gradient with per-row weights mask/(A*sum(mask_micro)) equals accumulating
    d(loss_i/A) over micro-batches (tools/ctd_train/main.cpp:346-361)."""
    cfg = tiny_cfg(num_hidden_layers=1)
    params = om.init_params(cfg, seed=7, std=0.05)
    tok, msk = om.synth_batch(cfg.vocab_size, 4, 24, seed=5)
    mbs = [om.make_batch(tok, msk, [0, 1]), om.make_batch(tok, msk, [2, 3])]
    total = None
    for ids, tgt, m in mbs:
        _, _, g = om.forward_backward(params, cfg, ids, tgt, m, dy=0.5, acc=np.float64)
        total = g if total is None else {k: total[k] + g[k] for k in g}
    # one fused pass: emulate by weighting rows — use the fp64 autograd statement with weights
    import torch
    P = {k: torch.from_numpy(v).double().requires_grad_(True) for k, v in params.items()}
    loss = sum(0.5 * torch_ref.loss_fn(P, cfg, torch.from_numpy(i), torch.from_numpy(t),
                                       torch.from_numpy(m).double()) for i, t, m in mbs)
    loss.backward()
    for k in total:
        ref = P[k].grad.numpy()
        assert np.abs(total[k] - ref).max() <= 1e-4 * max(np.abs(ref).max(), 1e-12), k


def test_train_step_updates_and_state():
    cfg = tiny_cfg(num_hidden_layers=1)
    params = om.init_params(cfg, seed=8, std=0.05)
    before = {k: v.copy() for k, v in params.items()}
    tok, msk = om.synth_batch(cfg.vocab_size, 2, 20, seed=6)
    opt = om.AdamWState()
    loss, norm, pre = om.train_step(params, cfg, [om.make_batch(tok, msk, [0, 1])], opt, 1e-3, 0.9, 0.999,
                                    1e-8, 0.01, clip=1.0)
    assert opt.step == 1 and loss > 0 and norm > 0
    # first AdamW step moves every element with a non-zero gradient by about lr (sign-like update)
    k = "model.layers.0.mlp.down_proj.weight"
    moved = np.abs(params[k] - before[k])
    assert moved.max() < 1.2e-3 and np.median(moved[pre[k] != 0]) > 0.5e-3
