"""KV-cache greedy decoding against the numpy oracle (full-prefix recomputation), through the
C-ABI: prefill logits, token-by-token agreement, cache consistency (prefill + steps == longer
prefill), limits and errors."""
import numpy as np
import pytest
import torch

from oracle import model as om

pytestmark = pytest.mark.gpu
F32 = np.float32

CASES = [
    dict(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
         num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-5, rope_theta=10000.0),
    dict(vocab_size=384, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
         num_key_value_heads=1, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0, qk_norm=True),
]


def build(kw, seed):
    from emberlm_b200 import engine as E
    ocfg, ecfg = om.LlamaConfig(**kw), E.make_config(**kw)
    params = om.init_params(ocfg, seed=seed, std=0.08)
    rng = np.random.default_rng(seed + 1)
    for k in params:
        if params[k].ndim == 1:
            params[k] = (params[k] + rng.uniform(-0.2, 0.2, params[k].shape)).astype(F32)
    return ocfg, ecfg, params


@pytest.mark.parametrize("kw", CASES)
def test_greedy_decode_matches_oracle(kw):
    from emberlm_b200 import engine as E
    ocfg, ecfg, params = build(kw, 41)
    prompt = np.random.default_rng(5).integers(0, ocfg.vocab_size, size=19)
    dec = E.Decoder(ecfg, max_seq_len=64)
    dec.load_parameters(params)
    got = dec.generate(prompt, 12).cpu().tolist()
    want, margins = om.greedy_generate(params, ocfg, prompt, 12, acc=np.float64)
    # tokens must agree wherever the oracle's top-2 logit margin is larger than TF32 noise; after a
    # (legitimate) near-tie divergence the continuations differ, so stop comparing there
    for i, (g, w, m) in enumerate(zip(got, want, margins)):
        if g != w:
            assert m < 2e-3, (i, g, w, m)
            break
    assert len(got) == 12
    # logits of the last processed position against the oracle on the same prefix
    prefix = np.concatenate([prompt, np.array(got[:-1], dtype=np.int64)])
    ref = om.forward_logits(params, ocfg, prefix[None, :], acc=np.float64)[0, -1]
    z = dec.last_logits().cpu().numpy()
    assert np.abs(z - ref).max() <= 5e-3 * max(np.abs(ref).max(), 1.0)


def test_cached_steps_equal_longer_prefill():
    from emberlm_b200 import engine as E
    ocfg, ecfg, params = build(CASES[0], 43)
    prompt = np.random.default_rng(6).integers(0, ocfg.vocab_size, size=33)
    dec = E.Decoder(ecfg, max_seq_len=80)
    dec.load_parameters(params)
    toks = dec.generate(prompt, 9).cpu().numpy()
    z_cached = dec.last_logits().cpu().numpy().copy()
    longer = np.concatenate([prompt, toks[:-1]])
    dec2 = E.Decoder(ecfg, max_seq_len=80, params=dec.params)
    dec2.generate(longer, 1)
    z_prefill = dec2.last_logits().cpu().numpy()
    # tests/test_integration_kvcache.cpp: prefill + decode == full forward within 5e-4 (fp32 there;
    # TF32 projections in the prefill here)
    assert np.abs(z_cached - z_prefill).max() <= 5e-3 * max(np.abs(z_prefill).max(), 1.0)


def test_decode_limits_and_errors():
    from emberlm_b200 import engine as E
    ocfg, ecfg, params = build(CASES[0], 45)
    dec = E.Decoder(ecfg, max_seq_len=24)
    dec.load_parameters(params)
    assert dec.generate(np.arange(20), 100).numel() == 5      # stops at max_seq_len: 24 - 20 cache positions + the token that needs none
    with pytest.raises(RuntimeError):
        dec.generate([], 4)
    with pytest.raises(RuntimeError):
        dec.generate(np.arange(24), 1)                        # prompt must leave room for one token
