"""CPU oracle of the decoder training step (forward, backward, clip, AdamW) — TEST
INFRASTRUCTURE ONLY; see oracle/ops.py for who may import it.

Wiring follows the reference (KyleCr4ne/emberlm):
  block      include/ctd/nn/transformer_block.h:28-35
  attention  include/ctd/nn/attention.h:100-143 (QK-Norm before RoPE: 115-121)
  mlp        include/ctd/nn/mlp.h:16-21
  model      include/ctd/nn/model.h:170-206 (tied LM head: 180-182)
  parameters src/nn/model.cpp:63-100 (order and decay / no-decay split)
  step       tools/ctd_train/main.cpp:346-373 (micro-batches, 1/A loss scaling, clip, AdamW)
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from . import ops

F32 = np.float32


@dataclass
class LlamaConfig:
    """Field names as include/ctd/nn/model.h:19-37."""
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int = 8192
    rms_norm_eps: float = 1e-5
    rope_theta: float = 100000.0
    tie_word_embeddings: bool = True
    qk_norm: bool = False
    rope_scaling_factor: float = 0.0
    rope_scaling_low_freq_factor: float = 1.0
    rope_scaling_high_freq_factor: float = 4.0
    rope_scaling_original_max_pos: int = 8192

    def rope_kwargs(self):
        return dict(scaling_factor=self.rope_scaling_factor,
                    low_freq_wavelen=self.rope_scaling_original_max_pos / self.rope_scaling_low_freq_factor,
                    high_freq_wavelen=self.rope_scaling_original_max_pos / self.rope_scaling_high_freq_factor)


# The five presets of include/ctd/nn/model.h:39-124.
PRESETS = {
    "smollm2_135m": LlamaConfig(49152, 576, 1536, 30, 9, 3, 64, 8192, 1e-5, 100000.0),
    "smollm2_360m": LlamaConfig(49152, 960, 2560, 32, 15, 5, 64, 8192, 1e-5, 100000.0),
    "qwen3_0_6b": LlamaConfig(151936, 1024, 3072, 28, 16, 8, 128, 40960, 1e-6, 1000000.0, True, True),
    "qwen3_1_7b": LlamaConfig(151936, 2048, 6144, 28, 16, 8, 128, 40960, 1e-6, 1000000.0, True, True),
    "llama3_2_1b": LlamaConfig(128256, 2048, 8192, 16, 32, 8, 64, 131072, 1e-5, 500000.0, True, False,
                               32.0, 1.0, 4.0, 8192),
}


def param_specs(cfg: LlamaConfig):
    """[(name, shape, decay)] in Model::collect_parameters order (src/nn/model.cpp:78-98)."""
    hid, I, D = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    H, Hk = cfg.num_attention_heads, cfg.num_key_value_heads
    out = [("model.embed_tokens.weight", (cfg.vocab_size, hid), True)]
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        out.append((p + "input_layernorm.weight", (hid,), False))
        out.append((p + "self_attn.q_proj.weight", (H * D, hid), True))
        out.append((p + "self_attn.k_proj.weight", (Hk * D, hid), True))
        out.append((p + "self_attn.v_proj.weight", (Hk * D, hid), True))
        out.append((p + "self_attn.o_proj.weight", (hid, H * D), True))
        if cfg.qk_norm:
            out.append((p + "self_attn.q_norm.weight", (D,), False))
            out.append((p + "self_attn.k_norm.weight", (D,), False))
        out.append((p + "post_attention_layernorm.weight", (hid,), False))
        out.append((p + "mlp.gate_proj.weight", (I, hid), True))
        out.append((p + "mlp.up_proj.weight", (I, hid), True))
        out.append((p + "mlp.down_proj.weight", (hid, I), True))
    out.append(("model.norm.weight", (hid,), False))
    return out


def init_params(cfg: LlamaConfig, seed: int = 1234, std: float = 0.02):
    """Synthetic weights: N(0, std) for embedding and linear weights, 1.0 for every norm weight."""
    rng = np.random.default_rng(seed)
    params = {}
    for name, shape, decay in param_specs(cfg):
        if decay:
            params[name] = (rng.standard_normal(shape, dtype=F32) * F32(std)).astype(F32)
        else:
            params[name] = np.ones(shape, dtype=F32)
    return params


def synth_batch(vocab, n_docs, seq_len, seed=4321):
    """Synthetic token rows and loss masks in the reference's bin format (int32 tokens, int8
    0/1 masks; mask[0]=0, alternating spans of 16..128 positions, assistant spans = 1)."""
    rng = np.random.default_rng(seed)
    tok = rng.integers(0, vocab, size=(n_docs, seq_len), dtype=np.int32)
    msk = np.zeros((n_docs, seq_len), dtype=np.int8)
    for d in range(n_docs):
        pos, val = 1, 0
        while pos < seq_len:
            ln = int(rng.integers(16, 129))
            msk[d, pos:pos + ln] = val
            pos += ln
            val ^= 1
        if msk[d].sum() == 0:
            msk[d, -1] = 1
    return tok, msk


def make_batch(tok, msk, doc_indices):
    """make_batch of tools/ctd_train/main.cpp:145-174: inputs tok[:-1], targets tok[1:], mask[1:]."""
    rows = tok[doc_indices]
    ids = rows[:, :-1].astype(np.int64)
    tgt = rows[:, 1:].astype(np.int64)
    m = msk[doc_indices][:, 1:].astype(F32)
    return ids, tgt, m


# ---------------------------------------------------------------------------------------
def forward_backward(params, cfg: LlamaConfig, ids, targets, mask, dy=1.0, acc=F32, want_grads=True):
    """Model::forward_train_masked (model.h:196-206) and the reverse pass the autograd tape
    would run (src/core/autograd.cu:158-237). Returns (loss, mask_sum, grads-by-name)."""
    B, T = ids.shape
    hid, D = cfg.hidden_size, cfg.head_dim
    H, Hk = cfg.num_attention_heads, cfg.num_key_value_heads
    G = H // Hk
    eps = cfg.rms_norm_eps
    rk = cfg.rope_kwargs()
    E = params["model.embed_tokens.weight"]
    h = ops.embedding(ids, E)  # [B,T,hid]
    caches = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        c = {"x": h}
        h1 = ops.rms_norm(h, params[p + "input_layernorm.weight"], eps, acc)
        x2 = h1.reshape(B * T, hid)
        q = ops.matmul(x2, params[p + "self_attn.q_proj.weight"], False, True, acc).reshape(B, T, H, D)
        k = ops.matmul(x2, params[p + "self_attn.k_proj.weight"], False, True, acc).reshape(B, T, Hk, D)
        v = ops.matmul(x2, params[p + "self_attn.v_proj.weight"], False, True, acc).reshape(B, T, Hk, D)
        c.update(h1=h1, q_pre=q, k_pre=k)
        if cfg.qk_norm:
            q = ops.rms_norm(q, params[p + "self_attn.q_norm.weight"], eps, acc)
            k = ops.rms_norm(k, params[p + "self_attn.k_norm.weight"], eps, acc)
        q = ops.rope(q, 0, cfg.rope_theta, 1.0, **rk)
        k = ops.rope(k, 0, cfg.rope_theta, 1.0, **rk)
        attn, probs = ops.attention_train(q, k, v, G, acc)
        c.update(q=q, k=k, v=v, probs=probs, attn=attn)
        a = ops.matmul(attn.reshape(B * T, H * D), params[p + "self_attn.o_proj.weight"], False, True, acc)
        hm = ops.add(h, a.reshape(B, T, hid))
        h2 = ops.rms_norm(hm, params[p + "post_attention_layernorm.weight"], eps, acc)
        y2 = h2.reshape(B * T, hid)
        g = ops.matmul(y2, params[p + "mlp.gate_proj.weight"], False, True, acc)
        u = ops.matmul(y2, params[p + "mlp.up_proj.weight"], False, True, acc)
        sg = ops.silu(g, acc)
        act = ops.mul(sg, u)
        m = ops.matmul(act, params[p + "mlp.down_proj.weight"], False, True, acc)
        c.update(hm=hm, h2=h2, g=g, u=u, sg=sg, act=act)
        h = ops.add(hm, m.reshape(B, T, hid))
        caches.append(c)
    hf = ops.rms_norm(h, params["model.norm.weight"], eps, acc)
    logits = ops.matmul(hf.reshape(B * T, hid), E, False, True, acc)
    loss, probs, mask_sum = ops.cross_entropy_masked(logits, targets.reshape(-1), mask.reshape(-1), acc)
    if not want_grads:
        return loss, mask_sum, None

    grads = {}
    dlogits = ops.cross_entropy_masked_backward(probs, targets.reshape(-1), mask.reshape(-1), mask_sum, dy)
    dhf, dE = ops.matmul_backward(dlogits, hf.reshape(B * T, hid), E, False, True, acc)
    grads["model.embed_tokens.weight"] = dE
    dh, dwn = ops.rms_norm_backward(dhf.reshape(B, T, hid), h, params["model.norm.weight"], eps, acc)
    grads["model.norm.weight"] = dwn
    for i in reversed(range(cfg.num_hidden_layers)):
        p = f"model.layers.{i}."
        c = caches[i]
        dm = dh.reshape(B * T, hid)
        dact, dWd = ops.matmul_backward(dm, c["act"], params[p + "mlp.down_proj.weight"], False, True, acc)
        grads[p + "mlp.down_proj.weight"] = dWd
        dsg = ops.mul(dact, c["u"])
        du = ops.mul(dact, c["sg"])
        dg = ops.silu_backward(c["g"], dsg, acc)
        y2 = c["h2"].reshape(B * T, hid)
        dy2_g, dWg = ops.matmul_backward(dg, y2, params[p + "mlp.gate_proj.weight"], False, True, acc)
        dy2_u, dWu = ops.matmul_backward(du, y2, params[p + "mlp.up_proj.weight"], False, True, acc)
        grads[p + "mlp.gate_proj.weight"] = dWg
        grads[p + "mlp.up_proj.weight"] = dWu
        dh2 = ops.add(dy2_g, dy2_u).reshape(B, T, hid)
        dhm_n, dwp = ops.rms_norm_backward(dh2, c["hm"], params[p + "post_attention_layernorm.weight"], eps, acc)
        grads[p + "post_attention_layernorm.weight"] = dwp
        dhm = ops.add(dh, dhm_n)
        dattn, dWo = ops.matmul_backward(dhm.reshape(B * T, hid), c["attn"].reshape(B * T, H * D),
                                         params[p + "self_attn.o_proj.weight"], False, True, acc)
        grads[p + "self_attn.o_proj.weight"] = dWo
        dq, dk, dv = ops.attention_train_backward(dattn.reshape(B, T, H * D), c["q"], c["k"], c["v"],
                                                  c["probs"], G, acc)
        dq = ops.rope(dq, 0, cfg.rope_theta, -1.0, **rk)
        dk = ops.rope(dk, 0, cfg.rope_theta, -1.0, **rk)
        if cfg.qk_norm:
            dq, dwq = ops.rms_norm_backward(dq, c["q_pre"], params[p + "self_attn.q_norm.weight"], eps, acc)
            dk, dwk = ops.rms_norm_backward(dk, c["k_pre"], params[p + "self_attn.k_norm.weight"], eps, acc)
            grads[p + "self_attn.q_norm.weight"] = dwq
            grads[p + "self_attn.k_norm.weight"] = dwk
        x2 = c["h1"].reshape(B * T, hid)
        dx_q, dWq = ops.matmul_backward(dq.reshape(B * T, H * D), x2, params[p + "self_attn.q_proj.weight"], False, True, acc)
        dx_k, dWk = ops.matmul_backward(dk.reshape(B * T, Hk * D), x2, params[p + "self_attn.k_proj.weight"], False, True, acc)
        dx_v, dWv = ops.matmul_backward(dv.reshape(B * T, Hk * D), x2, params[p + "self_attn.v_proj.weight"], False, True, acc)
        grads[p + "self_attn.q_proj.weight"] = dWq
        grads[p + "self_attn.k_proj.weight"] = dWk
        grads[p + "self_attn.v_proj.weight"] = dWv
        dh1 = (dx_q + dx_k + dx_v).astype(F32).reshape(B, T, hid)
        dx_n, dwi = ops.rms_norm_backward(dh1, c["x"], params[p + "input_layernorm.weight"], eps, acc)
        grads[p + "input_layernorm.weight"] = dwi
        dh = ops.add(dhm, dx_n)
    # tied embedding: LM-head gradient plus the scatter-add (include/ctd/nn/model.h:171,181)
    grads["model.embed_tokens.weight"] = ops.add(grads["model.embed_tokens.weight"],
                                                 ops.embedding_backward(ids, dh, cfg.vocab_size, acc))
    return loss, mask_sum, grads


@dataclass
class AdamWState:
    step: int = 0
    m: dict = field(default_factory=dict)
    v: dict = field(default_factory=dict)


def train_step(params, cfg, micro_batches, opt: AdamWState, lr, beta1, beta2, eps, weight_decay,
               clip=1.0, acc=F32):
    """One optimizer step of tools/ctd_train/main.cpp:346-373. micro_batches is a list of
    (ids, targets, mask); returns (logged_loss, grad_norm, grads_before_clip). params and opt are
    updated in place."""
    A = len(micro_batches)
    grads = None
    acc_loss, acc_active = 0.0, 0.0
    for ids, tgt, mask in micro_batches:
        sm = float(mask.sum())
        if sm <= 0:
            continue  # main.cpp:357
        loss, _, g = forward_backward(params, cfg, ids, tgt, mask, dy=1.0 / A, acc=acc)
        acc_loss += float(loss) * sm
        acc_active += sm
        if grads is None:
            grads = g
        else:
            for k in grads:
                grads[k] = ops.add(grads[k], g[k])
    specs = param_specs(cfg)
    names = [n for n, _, _ in specs]
    pre_clip = {n: grads[n].copy() for n in names}
    norm, clipped = ops.clip_grad_norm([grads[n] for n in names], clip, 1e-6, acc)
    opt.step += 1
    for (n, _, decay), g in zip(specs, clipped):
        if n not in opt.m:
            opt.m[n] = np.zeros_like(params[n])
            opt.v[n] = np.zeros_like(params[n])
        params[n], opt.m[n], opt.v[n] = ops.adamw_step(params[n], g, opt.m[n], opt.v[n], opt.step, lr,
                                                       beta1, beta2, eps, weight_decay if decay else 0.0)
    logged = acc_loss / acc_active if acc_active > 0 else 0.0
    return logged, float(norm), pre_clip


def forward_logits(params, cfg: LlamaConfig, ids, acc=F32):
    """Model::forward without a cache (include/ctd/nn/model.h:155-167): logits [B, T, V]. With a
    causal mask this equals the cached inference path position by position (the reference tests
    that in tests/test_integration_kvcache.cpp)."""
    B, T = ids.shape
    hid, D = cfg.hidden_size, cfg.head_dim
    H, Hk = cfg.num_attention_heads, cfg.num_key_value_heads
    eps, rk = cfg.rms_norm_eps, cfg.rope_kwargs()
    E = params["model.embed_tokens.weight"]
    h = ops.embedding(ids, E)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        x2 = ops.rms_norm(h, params[p + "input_layernorm.weight"], eps, acc).reshape(B * T, hid)
        q = ops.matmul(x2, params[p + "self_attn.q_proj.weight"], False, True, acc).reshape(B, T, H, D)
        k = ops.matmul(x2, params[p + "self_attn.k_proj.weight"], False, True, acc).reshape(B, T, Hk, D)
        v = ops.matmul(x2, params[p + "self_attn.v_proj.weight"], False, True, acc).reshape(B, T, Hk, D)
        if cfg.qk_norm:
            q = ops.rms_norm(q, params[p + "self_attn.q_norm.weight"], eps, acc)
            k = ops.rms_norm(k, params[p + "self_attn.k_norm.weight"], eps, acc)
        q, k = ops.rope(q, 0, cfg.rope_theta, 1.0, **rk), ops.rope(k, 0, cfg.rope_theta, 1.0, **rk)
        attn, _ = ops.attention_train(q, k, v, H // Hk, acc)
        a = ops.matmul(attn.reshape(B * T, H * D), params[p + "self_attn.o_proj.weight"], False, True, acc)
        hm = ops.add(h, a.reshape(B, T, hid))
        y2 = ops.rms_norm(hm, params[p + "post_attention_layernorm.weight"], eps, acc).reshape(B * T, hid)
        g = ops.matmul(y2, params[p + "mlp.gate_proj.weight"], False, True, acc)
        u = ops.matmul(y2, params[p + "mlp.up_proj.weight"], False, True, acc)
        m = ops.matmul(ops.mul(ops.silu(g, acc), u), params[p + "mlp.down_proj.weight"], False, True, acc)
        h = ops.add(hm, m.reshape(B, T, hid))
    hf = ops.rms_norm(h, params["model.norm.weight"], eps, acc)
    return ops.matmul(hf.reshape(B * T, hid), E, False, True, acc).reshape(B, T, -1)


def greedy_generate(params, cfg: LlamaConfig, prompt, max_new_tokens, acc=F32):
    """Greedy decoding as tools/ctd_generate/main.cpp:110-184 with temperature <= 0 and no EOS:
    argmax = first index of the maximum (src/core/sampling.cpp:13-20). Recomputes the full prefix
    each step (no cache), which gives the same logits."""
    ids = list(int(t) for t in prompt)
    out, margins = [], []
    for _ in range(max_new_tokens):
        z = forward_logits(params, cfg, np.array([ids], dtype=np.int64), acc)[0, -1]
        t = int(np.argmax(z))
        top2 = np.partition(z, -2)[-2:]
        margins.append(float(top2[1] - top2[0]))
        out.append(t)
        ids.append(t)
    return out, margins
