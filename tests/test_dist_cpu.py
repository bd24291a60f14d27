"""Data-parallel host logic on CPU with gloo, world_size 2: micro-batch dealing, per-row loss
weights, ZeRO-1 shard ownership and the per-shard weight-decay segments. The numpy oracle does
the arithmetic (no GPU); the result of the two-rank step must equal the single-process step of
tools/ctd_train/main.cpp:346-373 as restated in oracle.model.train_step."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import model as om
from oracle import ops as oo

HP = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.1, clip=0.5)
KW = dict(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2,
          num_key_value_heads=1, head_dim=64, rms_norm_eps=1e-5, rope_theta=10000.0)
A, MB, S = 4, 2, 24


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _flatten(layout, tensors, total):
    flat = np.zeros(total, np.float32)
    for n, o, k in zip(layout.names, layout.offsets, layout.numels):
        flat[o:o + k] = tensors[n].reshape(-1)
    return flat


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from emberlm_b200 import engine as E
    ocfg, ecfg = om.LlamaConfig(**KW), E.make_config(**KW)
    layout = E.model_layout(ecfg)
    total = E.padded_total(layout.total, world)
    params = om.init_params(ocfg, seed=3, std=0.05)
    tok, msk = om.synth_batch(ocfg.vocab_size, A * MB, S, seed=4)
    # this rank's micro-batches, fused into one pass with per-row weights
    mine = E.deal_micro_batches(A, world, rank)
    rows = [r for j in mine for r in range(j * MB, (j + 1) * MB)]
    ids, tgt, m = om.make_batch(tok, msk, rows)
    w = E.row_weights(torch.from_numpy(m), MB, A).numpy()
    grads = None
    for j in range(len(mine)):  # the oracle has no per-row weights: weight = dy/sum(mask) per micro-batch
        sl = slice(j * MB, (j + 1) * MB)
        _, _, g = om.forward_backward(params, ocfg, ids[sl], tgt[sl], m[sl], dy=1.0 / A, acc=np.float64)
        grads = g if grads is None else {k: grads[k] + g[k] for k in g}
        # the weights the engine would get are exactly dy/sum(mask) on the masked positions
        assert np.allclose(w[sl][m[sl] > 0], (1.0 / A) / m[sl].sum())
    gflat = torch.from_numpy(_flatten(layout, grads, total))
    dist.all_reduce(gflat)                       # gloo has no reduce_scatter: sum, then keep own slices
    # ownership as in TrainEngine: rank r owns slice r of every bucket (one layer per bucket here)
    buckets = E.make_buckets(layout, total, world, ocfg.num_hidden_layers, layers_per_bucket=1)
    mine_sl = [E.bucket_slice(lo, hi, world, rank) for lo, hi, _ in buckets]
    ss = torch.tensor([sum(float((gflat[a:b].numpy().astype(np.float64) ** 2).sum()) for a, b in mine_sl)],
                      dtype=torch.float64)
    dist.all_reduce(ss)
    norm = np.float32(np.sqrt(ss.item()))
    scale = np.float32(HP["clip"]) / (norm + np.float32(1e-6)) if norm > HP["clip"] else np.float32(1.0)
    pflat = _flatten(layout, params, total)
    full = np.zeros(total, np.float32)
    for (lo, hi, _), (a, b) in zip(buckets, mine_sl):
        gshard = gflat[a:b].numpy()
        ends, wds = E.build_segments(layout, HP["weight_decay"], a, b)
        new = pflat[a:b].copy()
        start = 0
        for end, wd in zip(ends, wds):
            p, _, _ = oo.adamw_step(pflat[a + start:a + end], (gshard[start:end] * scale).astype(np.float32),
                                    np.zeros(end - start, np.float32), np.zeros(end - start, np.float32), 1,
                                    HP["lr"], HP["beta1"], HP["beta2"], HP["eps"], wd)
            new[start:end] = p
            start = end
        gathered = [torch.zeros(b - a) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(new))
        full[lo:hi] = np.concatenate([g.numpy() for g in gathered])
    if rank == 0:
        np.save(out, full)
        np.save(out + ".norm.npy", np.array([norm]))
    dist.destroy_process_group()


def test_two_rank_zero1_step_equals_single_process_step(tmp_path):
    from emberlm_b200 import engine as E
    out = str(tmp_path / "params.npy")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = np.load(out)
    ocfg, ecfg = om.LlamaConfig(**KW), E.make_config(**KW)
    layout = E.model_layout(ecfg)
    params = om.init_params(ocfg, seed=3, std=0.05)
    tok, msk = om.synth_batch(ocfg.vocab_size, A * MB, S, seed=4)
    mbs = [om.make_batch(tok, msk, list(range(j * MB, (j + 1) * MB))) for j in range(A)]
    _, norm, _ = om.train_step(params, ocfg, mbs, om.AdamWState(), HP["lr"], HP["beta1"], HP["beta2"], HP["eps"],
                               HP["weight_decay"], HP["clip"], acc=np.float64)
    assert abs(float(np.load(out + ".norm.npy")[0]) - norm) <= 1e-5 * norm
    for n, o, k in zip(layout.names, layout.offsets, layout.numels):
        ref = params[n].reshape(-1)
        assert np.abs(got[o:o + k] - ref).max() <= 2e-5 * max(np.abs(ref).max(), 1e-12), n


def test_shard_segments_cover_every_tensor_once():
    from emberlm_b200 import engine as E
    cfg = E.make_config(**E.PRESETS["qwen3_0_6b"])
    layout = E.model_layout(cfg)
    for world in (1, 2, 4, 8):
        total = E.padded_total(layout.total, world)
        assert total % (64 * world) == 0 and total >= layout.total
        wd = np.full(total, -1, np.int8)   # per element: -1 unowned, 1 decayed, 0 not decayed
        for r in range(world):
            lo, hi = E.shard_bounds(total, world, r)
            ends, wds = E.build_segments(layout, 0.01, lo, hi)
            assert ends[-1] == hi - lo and all(e % 4 == 0 for e in ends) and ends == sorted(ends)
            start = 0
            for e, w in zip(ends, wds):
                wd[lo + start:lo + e] = 1 if w > 0 else 0
                start = e
        assert (wd >= 0).all()
        for o, k, d in zip(layout.offsets, layout.numels, layout.decay):
            assert (wd[o:o + k] == (1 if d else 0)).all()


def test_buckets_partition_the_arena_and_know_when_they_are_complete():
    from emberlm_b200 import engine as E
    for preset in ("smollm2_360m", "qwen3_0_6b"):
        cfg = E.make_config(**E.PRESETS[preset])
        layout = E.model_layout(cfg)
        L = cfg.num_hidden_layers
        for world in (2, 4, 8):
            total = E.padded_total(layout.total, world)
            buckets = E.make_buckets(layout, total, world, L)
            assert buckets[0][0] == 0 and buckets[-1][1] == total
            assert all(x[1] == y[0] for x, y in zip(buckets[:-1], buckets[1:]))
            assert all((hi - lo) % (64 * world) == 0 and hi > lo for lo, hi, _ in buckets)
            # the embedding bucket is complete last (-1), later buckets earlier and earlier
            assert buckets[0][2] == -1 and [b[2] for b in buckets] == sorted(b[2] for b in buckets)
            # a bucket is complete once the lowest-numbered tensor it touches is
            for lo, hi, ready in buckets:
                touching = [E.tensor_layer(n, L) for n, o, k in zip(layout.names, layout.offsets, layout.numels)
                            if o < hi and o + k > lo]
                assert ready == min(touching)
            # slices of all ranks tile every bucket; per-slice decay segments match the tensors
            wd = np.full(total, -1, np.int8)
            owned = 0
            for r in range(world):
                for lo, hi, _ in buckets:
                    a, b = E.bucket_slice(lo, hi, world, r)
                    owned += b - a
                    ends, wds = E.build_segments(layout, 0.01, a, b)
                    assert ends[-1] == b - a
                    start = 0
                    for e, w in zip(ends, wds):
                        assert (wd[a + start:a + e] == -1).all()
                        wd[a + start:a + e] = 1 if w > 0 else 0
                        start = e
            assert owned == total and (wd >= 0).all()
            for o, k, d in zip(layout.offsets, layout.numels, layout.decay):
                assert (wd[o:o + k] == (1 if d else 0)).all()
    assert E.tensor_layer("model.layers.17.mlp.up_proj.weight", 32) == 17
    assert E.tensor_layer("model.norm.weight", 32) == 32 and E.tensor_layer("model.embed_tokens.weight", 32) == -1


def test_dealing_and_row_weights():
    from emberlm_b200 import engine as E
    assert E.deal_micro_batches(8, 4, 1) == [1, 5]
    assert sorted(sum((E.deal_micro_batches(8, 8, r) for r in range(8)), [])) == list(range(8))
    with pytest.raises(ValueError):
        E.deal_micro_batches(8, 3, 0)
    m = torch.tensor([[0, 1, 1, 0], [0, 0, 1, 0], [0, 0, 0, 0], [0, 0, 0, 0]], dtype=torch.float32)
    w = E.row_weights(m, 2, 4)                    # micro-batch 0: 3 ones; micro-batch 1: empty mask
    assert torch.allclose(w[:2][m[:2] > 0], torch.tensor(1.0 / (4 * 3)))
    assert float(w[2:].abs().sum()) == 0.0 and float(w[:2][m[:2] == 0].abs().sum()) == 0.0


def test_library_plan_equals_the_python_statement():
    """ctdk_dp_buckets / ctdk_dp_segments (the C++ trainer's plan, host only) against the Python
    statement of the same rules above, for the five presets, 1-8 ranks and three bucket sizes."""
    from emberlm_b200 import engine as E
    for name in E.PRESETS:
        cfg = E.make_config(**E.PRESETS[name])
        lay = E.model_layout(cfg)
        for world in (1, 2, 4, 8):
            total = E.padded_total(lay.total, world)
            assert total == E.lib.raw().ctdk_dp_arena_floats(cfg, world)
            for per in (0, 1, 4):
                py = E.make_buckets(lay, total, world, cfg.num_hidden_layers, per)
                for rank in range(world):
                    cc = E.dp_plan(cfg, world, rank, per)
                    assert len(cc) == len(py)
                    pos = 0
                    for c, (lo, hi, ready) in zip(cc, py):
                        a, b = E.bucket_slice(lo, hi, world, rank)
                        assert (c["lo"], c["hi"], c["ready"], c["a"], c["b"], c["state"]) == (lo, hi, ready, a, b, pos)
                        pos += b - a
                        e1, w1 = E.build_segments(lay, 0.01, a, b)
                        e2, w2 = E.dp_segments(cfg, 0.01, a, b)
                        assert e1 == e2 and np.allclose(w1, w2, atol=1e-9)
                    assert pos == total // world
