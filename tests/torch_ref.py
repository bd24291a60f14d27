"""Independent double-precision statement of the decoder in torch autograd: on the CPU it
cross-checks the hand-written backward of the numpy oracle; on a GPU (loss_and_grads_device) it
is the fp64 arbiter of the full-size comparisons, where the reference's own CUDA build is not
reproducible from run to run. Wiring as the reference:
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


def _layer(h, cfg, cos, sin, w_in, wq, wk, wv, wo, wqn, wkn, w_post, wg, wu, wd):
    B, T, _ = h.shape
    D, H, Hk = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    G, eps = H // Hk, cfg.rms_norm_eps
    h1 = rms(h, w_in, eps)
    q = (h1 @ wq.T).view(B, T, H, D)
    k = (h1 @ wk.T).view(B, T, Hk, D)
    v = (h1 @ wv.T).view(B, T, Hk, D)
    if cfg.qk_norm:
        q = rms(q, wqn, eps)
        k = rms(k, wkn, eps)
    q, k = rope(q, cos, sin), rope(k, cos, sin)
    k = k.repeat_interleave(G, dim=2)
    v = v.repeat_interleave(G, dim=2)
    q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    sc = (q @ k.transpose(-1, -2)) / math.sqrt(D)
    causal = torch.triu(torch.ones(T, T, dtype=torch.bool, device=h.device), 1)
    sc = sc.masked_fill(causal, -torch.finfo(torch.float32).max)
    a = (torch.softmax(sc, -1) @ v).transpose(1, 2).reshape(B, T, H * D)
    hm = h + a @ wo.T
    h2 = rms(hm, w_post, eps)
    return hm + (torch.nn.functional.silu(h2 @ wg.T) * (h2 @ wu.T)) @ wd.T


def loss_fn(params, cfg, ids, targets, mask, checkpoint_layers=False):
    """Mask-weighted mean loss of one micro-batch. checkpoint_layers: keep only layer inputs and
    recompute inside the backward (torch.utils.checkpoint), for the full-size shapes."""
    B, T = ids.shape
    E = params["model.embed_tokens.weight"]
    c, s = oops.rope_cos_sin(T, cfg.head_dim, 0, cfg.rope_theta, **cfg.rope_kwargs())
    cos, sin = torch.from_numpy(c).double().to(E.device), torch.from_numpy(s).double().to(E.device)
    h = E[ids]
    one = torch.ones((), dtype=E.dtype, device=E.device)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        w = [params[p + n] for n in ("input_layernorm.weight", "self_attn.q_proj.weight", "self_attn.k_proj.weight",
                                     "self_attn.v_proj.weight", "self_attn.o_proj.weight")]
        w += [params[p + "self_attn.q_norm.weight"], params[p + "self_attn.k_norm.weight"]] if cfg.qk_norm else [one, one]
        w += [params[p + n] for n in ("post_attention_layernorm.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight",
                                      "mlp.down_proj.weight")]
        if checkpoint_layers:
            from torch.utils.checkpoint import checkpoint
            h = checkpoint(lambda x, *ws: _layer(x, cfg, cos, sin, *ws), h, *w, use_reentrant=False)
        else:
            h = _layer(h, cfg, cos, sin, *w)
    hf = rms(h, params["model.norm.weight"], cfg.rms_norm_eps)
    logits = (hf @ E.T).view(B * T, -1)
    lse = torch.logsumexp(logits, -1)
    zt = logits[torch.arange(B * T, device=E.device), targets.reshape(-1)]
    m = mask.reshape(-1)
    return (m * (lse - zt)).sum() / m.sum()


def loss_and_grads_device(params_np, cfg, micro_batches, device="cuda"):
    """fp64 loss and gradients of a whole step on `device`: micro_batches is a list of
    (ids, targets, mask) numpy triples; each is normalised by its own mask sum and weighted
    1/len(micro_batches) (tools/ctd_train/main.cpp:346-361). Returns (logged loss = mask-weighted
    mean, {name: fp64 gradient tensor on the device})."""
    params = {k: torch.from_numpy(v).to(device).double().requires_grad_(True) for k, v in params_np.items()}
    A = len(micro_batches)
    num = den = 0.0
    for ids, tgt, m in micro_batches:
        d_m = torch.from_numpy(m).to(device).double()
        if float(d_m.sum()) <= 0:
            continue
        loss = loss_fn(params, cfg, torch.from_numpy(ids).to(device), torch.from_numpy(tgt).to(device), d_m,
                       checkpoint_layers=True)
        (loss / A).backward()
        num += float(loss) * float(d_m.sum())
        den += float(d_m.sum())
    return num / den, {k: v.grad for k, v in params.items()}


def loss_and_grads(params_np, cfg, ids, targets, mask, dy=1.0):
    params = {k: torch.from_numpy(v).double().requires_grad_(True) for k, v in params_np.items()}
    loss = loss_fn(params, cfg, torch.from_numpy(ids), torch.from_numpy(targets), torch.from_numpy(mask).double())
    (loss * dy).backward()
    return float(loss), {k: v.grad.numpy() for k, v in params.items()}
