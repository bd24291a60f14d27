"""Seeded inputs of the golden cases: the reference's outputs for them are stored in
tests/golden/ref_step_<name>.npz (made by tests/golden/make_golden.py on a B200)."""
import numpy as np

from oracle import model as om

F32 = np.float32
STEPS = 2
HP = dict(lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, clip=1.0)

CASES = {
    # name: (config kwargs, docs, seq_len, micro-batch rows, grad-accum)
    "tiny_gqa": (dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-5,
                      rope_theta=10000.0), 8, 48, 2, 2),
    "tiny_qknorm": (dict(vocab_size=384, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                         num_attention_heads=2, num_key_value_heads=1, head_dim=128, rms_norm_eps=1e-6,
                         rope_theta=1000000.0, qk_norm=True), 4, 40, 2, 1),
    "tiny_llama3rope": (dict(vocab_size=256, hidden_size=128, intermediate_size=384, num_hidden_layers=1,
                             num_attention_heads=2, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-5,
                             rope_theta=500000.0, rope_scaling_factor=32.0, rope_scaling_original_max_pos=32),
                        4, 72, 2, 1),
}


def build_case(name):
    kw, docs, S, b, A = CASES[name]
    cfg = om.LlamaConfig(**kw)
    params = om.init_params(cfg, seed=21, std=0.05)
    rng = np.random.default_rng(22)
    for k in params:
        if params[k].ndim == 1:
            params[k] = (params[k] + rng.uniform(-0.2, 0.2, params[k].shape)).astype(F32)
    tok, msk = om.synth_batch(cfg.vocab_size, docs, S, seed=23)
    return cfg, params, tok, msk, b, A


def micro_batches(tok, msk, b, A, step):
    """Rows of step `step`, micro-batch j = docs [(step*A+j)*b, +b) modulo the document count, as
    oracle/ref_harness.cpp takes them."""
    docs = tok.shape[0]
    out = []
    for j in range(A):
        idx = [((step * A + j) * b + r) % docs for r in range(b)]
        out.append(om.make_batch(tok, msk, idx))
    return out
