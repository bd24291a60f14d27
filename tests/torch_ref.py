"""Independent double-precision statement of the decoder in torch (CPU autograd), used only to
cross-check the hand-written backward of the numpy oracle. Wiring as the reference:
include/ctd/nn/{attention,mlp,transformer_block,model}.h."""
import math

import numpy as np
import torch

from oracle import ops as oops


def rms(x, w, eps):
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rope(x, cos, sin):
    D = x.shape[-1]
    a, b = x[..., : D // 2], x[..., D // 2:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def loss_fn(params, cfg, ids, targets, mask):
    B, T = ids.shape
    hid, D = cfg.hidden_size, cfg.head_dim
    H, Hk = cfg.num_attention_heads, cfg.num_key_value_heads
    G = H // Hk
    eps = cfg.rms_norm_eps
    c, s = oops.rope_cos_sin(T, D, 0, cfg.rope_theta, **cfg.rope_kwargs())
    cos, sin = torch.from_numpy(c).double(), torch.from_numpy(s).double()
    E = params["model.embed_tokens.weight"]
    h = E[ids]
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        h1 = rms(h, params[p + "input_layernorm.weight"], eps)
        q = (h1 @ params[p + "self_attn.q_proj.weight"].T).view(B, T, H, D)
        k = (h1 @ params[p + "self_attn.k_proj.weight"].T).view(B, T, Hk, D)
        v = (h1 @ params[p + "self_attn.v_proj.weight"].T).view(B, T, Hk, D)
        if cfg.qk_norm:
            q = rms(q, params[p + "self_attn.q_norm.weight"], eps)
            k = rms(k, params[p + "self_attn.k_norm.weight"], eps)
        q, k = rope(q, cos, sin), rope(k, cos, sin)
        k = k.repeat_interleave(G, dim=2)
        v = v.repeat_interleave(G, dim=2)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        sc = (q @ k.transpose(-1, -2)) / math.sqrt(D)
        causal = torch.triu(torch.ones(T, T, dtype=torch.bool), 1)
        sc = sc.masked_fill(causal, -torch.finfo(torch.float32).max)
        a = (torch.softmax(sc, -1) @ v).transpose(1, 2).reshape(B, T, H * D)
        hm = h + a @ params[p + "self_attn.o_proj.weight"].T
        h2 = rms(hm, params[p + "post_attention_layernorm.weight"], eps)
        g = h2 @ params[p + "mlp.gate_proj.weight"].T
        u = h2 @ params[p + "mlp.up_proj.weight"].T
        h = hm + (torch.nn.functional.silu(g) * u) @ params[p + "mlp.down_proj.weight"].T
    hf = rms(h, params["model.norm.weight"], eps)
    logits = (hf @ E.T).view(B * T, -1)
    lse = torch.logsumexp(logits, -1)
    zt = logits[torch.arange(B * T), targets.reshape(-1)]
    m = mask.reshape(-1)
    return (m * (lse - zt)).sum() / m.sum()


def loss_and_grads(params_np, cfg, ids, targets, mask, dy=1.0):
    params = {k: torch.from_numpy(v).double().requires_grad_(True) for k, v in params_np.items()}
    loss = loss_fn(params, cfg, torch.from_numpy(ids), torch.from_numpy(targets), torch.from_numpy(mask).double())
    (loss * dy).backward()
    return float(loss), {k: v.grad.numpy() for k, v in params.items()}
