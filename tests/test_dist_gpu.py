"""Two-GPU data-parallel step (NCCL reduce-scatter -> shard AdamW -> all-gather) against the
one-GPU step on the same rows: the result must not depend on the number of ranks beyond
summation order. Needs two visible GPUs; skipped otherwise."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

KW = dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
          num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-5, rope_theta=10000.0)
HP = dict(lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, clip=1.0)
A, MB, S, STEPS = 4, 2, 65, 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(rank, world, port, out):
    import torch.distributed as dist
    from emberlm_b200 import engine as E
    from oracle import model as om
    torch.cuda.set_device(rank)
    group = None
    if world > 1:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
        group = dist.group.WORLD
    ocfg, ecfg = om.LlamaConfig(**KW), E.make_config(**KW)
    params = om.init_params(ocfg, seed=31, std=0.05)
    mine = E.deal_micro_batches(A, world, rank)
    eng = E.TrainEngine(ecfg, len(mine) * MB, S - 1, device=f"cuda:{rank}", group=group, **HP)
    eng.load_parameters(params)
    losses = []
    for step in range(STEPS):
        tok, msk = om.synth_batch(ocfg.vocab_size, A * MB, S, seed=40 + step)
        rows = [r for j in mine for r in range(j * MB, (j + 1) * MB)]
        ids, tgt, m = om.make_batch(tok, msk, rows)
        d_m = torch.from_numpy(m).cuda()
        eng.train_step(torch.from_numpy(ids).cuda(), torch.from_numpy(tgt).cuda(), d_m, E.row_weights(d_m, MB, A))
        losses.append(eng.read_metrics())
    if world > 1:
        eng.wait_parameters()      # the last step's all-gathers are still in flight on NCCL's stream
    if rank == 0:
        np.savez(out, loss=np.array([x["loss"] for x in losses]), norm=np.array([x["grad_norm"] for x in losses]),
                 params=eng.params[:eng.layout.total].cpu().numpy())
    if world > 1:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_step_equals_one_gpu_step(tmp_path):
    import torch.multiprocessing as mp
    one, two = str(tmp_path / "one.npz"), str(tmp_path / "two.npz")
    mp.spawn(_run, args=(1, 0, one), nprocs=1, join=True)
    mp.spawn(_run, args=(2, _free_port(), two), nprocs=2, join=True)
    a, b = np.load(one), np.load(two)
    np.testing.assert_allclose(b["loss"], a["loss"], rtol=1e-5)
    np.testing.assert_allclose(b["norm"], a["norm"], rtol=1e-4)
    # AdamW's early steps are sign-like, so summation-order noise on near-zero gradients can move
    # single elements by up to 2*lr; bound the error relative to the largest weight
    assert np.abs(b["params"] - a["params"]).max() <= 3 * HP["lr"]
    assert np.mean(np.abs(b["params"] - a["params"]) > 1e-6) < 1e-3
