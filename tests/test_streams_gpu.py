"""Stream ordering inside the step engine and the attention backward:
  - the weight-gradient GEMMs run on a side stream by default; with CTDK_ENGINE_SIDE_STREAM=0
    everything stays on the caller's stream. Both schedules must give the same gradients, with
    and without accumulation and checkpointing, at a size whose kernels take long enough to
    overlap. "The same" is measured against what one schedule does from run to run: GEMMs split
    into more than two k-ranges add their parts at L2 in arrival order, so two runs of ONE
    schedule already differ in the last bits of the head's d(hidden), which TF32 rounding then
    amplifies down the layers; a missed wait would show up far above that;
  - the layer callback contract: when cb(l) fires, everything that writes layer l's gradients is
    ordered before the caller's stream, so a copy issued on a second stream behind an event
    recorded there must see the final values;
  - two ctdk_attn_bwd calls at head size 64 on different streams of one device (the dK/dV kernel
    claims work items from a global counter: each call has its own)."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

KW = dict(vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=4, num_attention_heads=8,
          num_key_value_heads=4, head_dim=64, rms_norm_eps=1e-5, rope_theta=10000.0)

_CHILD = r"""
import sys, numpy as np, torch
sys.path.insert(0, sys.argv[1])
from emberlm_b200 import engine as E
from oracle import model as om
kw = dict(vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=4, num_attention_heads=8,
          num_key_value_heads=4, head_dim=64, rms_norm_eps=1e-5, rope_theta=10000.0)
ckpt, accumulate, out = int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
cfg = om.LlamaConfig(**kw)
params = om.init_params(cfg, seed=3, std=0.05)
tok, msk = om.synth_batch(cfg.vocab_size, 8, 513, seed=4)
ids, tgt, m = om.make_batch(tok, msk, list(range(8)))
eng = E.TrainEngine(E.make_config(**kw, gradient_checkpointing=bool(ckpt)), 8, 512)
eng.load_parameters(params)
d = [torch.from_numpy(a).cuda() for a in (ids, tgt, m)]
w = E.row_weights(d[2], 4, 2)
eng.loss_sums.zero_()
if accumulate:
    eng.forward_backward(d[0][:4].contiguous(), d[1][:4].contiguous(), d[2][:4].contiguous(), w[:4].contiguous())
    eng.forward_backward(d[0][4:].contiguous(), d[1][4:].contiguous(), d[2][4:].contiguous(), w[4:].contiguous(), accumulate=True)
else:
    eng.forward_backward(*d, w)
torch.cuda.synchronize()
E.check_device_status()
g = eng.named_grads()
np.savez(out, **{k: v.cpu().numpy() for k, v in g.items() if k != "model.embed_tokens.weight"})
"""


@pytest.mark.parametrize("ckpt,accumulate", [(0, 0), (1, 0), (0, 1), (1, 1)])
def test_side_stream_schedule_is_bit_identical_to_one_stream(tmp_path, ckpt, accumulate):
    outs = []
    for i, side in enumerate(("0", "0", "1")):      # one stream twice (the run-to-run floor), then the side stream
        out = tmp_path / f"g{i}.npz"
        env = dict(os.environ, CTDK_ENGINE_SIDE_STREAM=side)
        r = subprocess.run([sys.executable, "-c", _CHILD, str(ROOT), str(ckpt), str(accumulate), str(out)], env=env,
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        outs.append(np.load(out))

    def err(a, b):
        return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))

    # (the tied embedding's gradient takes float atomics from the scatter-add: left out above)
    floor = max(err(outs[1][k], outs[0][k]) for k in outs[0].files)
    worst = max((err(outs[2][k], outs[0][k]), k) for k in outs[0].files)
    print(f"run-to-run {floor:.2e}, side stream vs one stream {worst[0]:.2e} ({worst[1]})")
    assert worst[0] <= max(4 * floor, 1e-6), (worst, floor)


def test_layer_callback_sees_final_gradients():
    from emberlm_b200 import engine as E
    from oracle import model as om
    cfg = om.LlamaConfig(**KW)
    params = om.init_params(cfg, seed=3, std=0.05)
    tok, msk = om.synth_batch(cfg.vocab_size, 8, 513, seed=4)
    ids, tgt, m = om.make_batch(tok, msk, list(range(8)))
    eng = E.TrainEngine(E.make_config(**KW), 8, 512)
    eng.load_parameters(params)
    lay = eng.layout
    L = KW["num_hidden_layers"]
    copies, order = {}, []
    second = torch.cuda.Stream()
    main = torch.cuda.current_stream()

    def on_layer(layer):
        order.append(layer)
        ev = torch.cuda.Event()
        ev.record(main)
        second.wait_event(ev)
        with torch.cuda.stream(second):
            for n, o, k in zip(lay.names, lay.offsets, lay.numels):
                if E.tensor_layer(n, L) == layer:
                    copies[n] = eng.grads[o:o + k].clone()

    eng.set_layer_callback(on_layer)
    d = [torch.from_numpy(a).cuda() for a in (ids, tgt, m)]
    eng.grads.fill_(float("nan"))       # anything copied too early is NaN
    eng.loss_sums.zero_()
    eng.forward_backward(*d, E.row_weights(d[2], 8, 1))
    torch.cuda.synchronize()
    assert order == [L] + list(range(L - 1, -1, -1)) + [-1]
    final = eng.named_grads()
    assert set(copies) == set(final)
    for n, c in copies.items():
        assert torch.equal(c, final[n].reshape(-1)), n


def test_attention_backward_on_two_streams():
    from emberlm_b200 import ops
    B, T, H, Hk, D = 4, 700, 8, 4, 64
    gen = torch.Generator(device="cuda").manual_seed(1)
    ins = []
    for _ in range(2):
        qkv = torch.randn(B * T, (H + 2 * Hk) * D, device="cuda", generator=gen)
        dout = torch.randn(B * T, H * D, device="cuda", generator=gen)
        out, lse = ops.attention(qkv, B, T, H, Hk, D)
        ins.append((qkv, out, dout, lse))
    want = [ops.attention_backward(*x, B, T, H, Hk, D) for x in ins]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for rep in range(3):
        got = []
        for s, x in zip(streams, ins):
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                got.append(ops.attention_backward(*x, B, T, H, Hk, D))
        torch.cuda.synchronize()
        for g, w in zip(got, want):
            assert torch.equal(g, w), rep
    from emberlm_b200 import engine as E
    E.check_device_status()
