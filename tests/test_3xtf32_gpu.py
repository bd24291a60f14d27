"""The optional 3xTF32 mode: every contraction (GEMMs and attention) splits its operands into
TF32 high and low parts. Stated tolerance for this mode: per-tensor gradient and updated-weight
error <= 1e-4 (max|a-b|/max|b|), loss rel <= 1e-3."""
import numpy as np
import pytest
import torch

from oracle import model as om
from oracle import ops as oo

pytestmark = pytest.mark.gpu
F32 = np.float32


def relmax(got, ref):
    return float(np.abs(got.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


@pytest.mark.parametrize("ta,tb,M,N,K", [(False, True, 2044, 576, 576), (False, False, 300, 2560, 960),
                                         (True, False, 960, 320, 4000), (False, True, 4093, 1600, 960)])
def test_gemm_3xtf32_is_near_fp32(ta, tb, M, N, K):
    from emberlm_b200 import lib, ops
    rng = np.random.default_rng(1)
    a = rng.uniform(-1, 1, (K, M) if ta else (M, K)).astype(F32)
    b = rng.uniform(-1, 1, (N, K) if tb else (K, N)).astype(F32)
    ref = (a.T if ta else a).astype(np.float64) @ (b.T if tb else b).astype(np.float64)
    A, B = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    e3 = relmax(ops.matmul(A, B, ta, tb, precision=lib.GEMM_3XTF32).cpu().numpy(), ref)
    e1 = relmax(ops.matmul(A, B, ta, tb).cpu().numpy(), ref)
    assert e3 < 5e-6 and e3 < e1 / 20, (e3, e1)
    # accumulate epilogue in the split mode
    base = torch.from_numpy(rng.uniform(-1, 1, (M, N)).astype(F32)).cuda()
    c = base.clone()
    ops.matmul(A, B, ta, tb, precision=lib.GEMM_3XTF32, out=c, epilogue=lib.EPI_ACCUMULATE)
    assert relmax(c.cpu().numpy(), ref + base.cpu().numpy()) < 5e-6


@pytest.mark.parametrize("B,T,H,Hk,D", [(2, 130, 4, 2, 64), (1, 200, 2, 1, 128)])
def test_attention_3xtf32_is_near_fp32(B, T, H, Hk, D):
    from emberlm_b200 import lib, ops
    rng = np.random.default_rng(2)
    qkv = rng.uniform(-1.5, 1.5, (B * T, (H + 2 * Hk) * D)).astype(F32)
    dout = rng.uniform(-1, 1, (B * T, H * D)).astype(F32)
    x4 = qkv.reshape(B, T, H + 2 * Hk, D)
    q, k, v = (np.ascontiguousarray(x4[:, :, :H]), np.ascontiguousarray(x4[:, :, H:H + Hk]),
               np.ascontiguousarray(x4[:, :, H + Hk:]))
    ref, probs = oo.attention_train(q, k, v, H // Hk, np.float64)
    rdq, rdk, rdv = oo.attention_train_backward(dout.reshape(B, T, H * D), q, k, v, probs, H // Hk, np.float64)
    rref = np.concatenate([rdq, rdk, rdv], axis=2).reshape(B * T, -1)
    Q, DO = torch.from_numpy(qkv).cuda(), torch.from_numpy(dout).cuda()
    out, lse = ops.attention(Q, B, T, H, Hk, D, precision=lib.GEMM_3XTF32)
    assert relmax(out.cpu().numpy(), ref.reshape(B * T, H * D)) < 2e-5
    dqkv = ops.attention_backward(Q, out, DO, lse, B, T, H, Hk, D, precision=lib.GEMM_3XTF32)
    assert relmax(dqkv.cpu().numpy(), rref) < 5e-5


@pytest.mark.parametrize("kw", [dict(), dict(qk_norm=True, rms_norm_eps=1e-6, head_dim=128, hidden_size=128)])
def test_engine_3xtf32_matches_oracle_to_1e4(kw):
    from emberlm_b200 import engine as E, lib
    base = dict(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2,
                num_key_value_heads=1, head_dim=64, rms_norm_eps=1e-5, rope_theta=10000.0)
    base.update(kw)
    ocfg, ecfg = om.LlamaConfig(**base), E.make_config(**base, precision=lib.GEMM_3XTF32)
    params = om.init_params(ocfg, seed=5, std=0.05)
    tok, msk = om.synth_batch(ocfg.vocab_size, 3, 131, seed=3)
    ids, tgt, m = om.make_batch(tok, msk, [0, 1, 2])
    loss, ms, ref = om.forward_backward(params, ocfg, ids, tgt, m, acc=np.float64)
    eng = E.TrainEngine(ecfg, 3, 130)
    eng.load_parameters(params)
    d_m = torch.from_numpy(m).cuda()
    eng.loss_sums.zero_()
    eng.forward_backward(torch.from_numpy(ids).cuda(), torch.from_numpy(tgt).cuda(), d_m, E.row_weights(d_m, 3, 1))
    torch.cuda.synchronize()
    ls = eng.loss_sums.tolist()
    assert abs(ls[0] / ls[1] - float(loss)) <= 1e-5 * float(loss)
    for k, g in eng.named_grads().items():
        assert relmax(g.cpu().numpy(), ref[k]) <= 1e-4, k
