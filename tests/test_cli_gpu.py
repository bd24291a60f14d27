"""ctd_train end to end on a GPU: SmolLM2-135M with random weights, two optimizer steps from bins
with a single training document (so the reference's random document picks are all the same row),
against the Python-driven engine on the same rows; then resume for one more step."""
import json
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from emberlm_b200 import build, safetensors_io

pytestmark = pytest.mark.gpu
EXE = Path(build.HERE) / "ctd_train"
S, B, A = 65, 2, 2
HP = dict(lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)


def test_two_steps_match_the_engine_then_resume(tmp_path):
    from emberlm_b200 import engine as E
    build.build()
    cfg = E.make_config(**E.PRESETS["smollm2_135m"])
    eng = E.TrainEngine(cfg, A * B, S - 1, clip=1.0, **HP)
    eng.init_parameters(seed=5)
    names = list(eng.named_parameters().items())
    w0 = tmp_path / "init.safetensors"
    safetensors_io.save_safetensors([(n, v.cpu().numpy()) for n, v in names], w0)
    rng = np.random.default_rng(9)
    tok = rng.integers(0, cfg.vocab_size, size=(1, S), dtype=np.int32)
    msk = np.zeros((1, S), np.int8)
    msk[0, 20:50] = 1
    data = tmp_path / "data"
    data.mkdir()
    for name, arr in (("train.bin", tok), ("train_mask.bin", msk), ("val.bin", np.repeat(tok, 3, 0)),
                      ("val_mask.bin", np.repeat(msk, 3, 0))):
        arr.tofile(data / name)
    run_dir = tmp_path / "run"
    run_dir.mkdir()
    conf = dict(init_weights=str(w0), data_dir=str(data), seq_len=S, batch_size=B, grad_accum_steps=A, total_steps=2,
                warmup_steps=0, min_lr_ratio=1.0, clip_grad_norm=1.0, val_every=2, save_every=0, log_every=1, seed=42, **HP)
    (run_dir / "config.json").write_text(json.dumps(conf))
    r = subprocess.run([str(EXE), "--config", str(run_dir / "config.json")], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "[ctd_train] arch: hidden=576 layers=30 heads=9" in r.stderr and "done. final" in r.stderr
    events = [json.loads(l) for l in (run_dir / "loss.jsonl").read_text().splitlines()]
    train = [e for e in events if e["phase"] == "train"]
    val = [e for e in events if e["phase"] == "val"]
    assert [e["step"] for e in train] == [1, 2] and [e["step"] for e in val] == [2]
    assert set(train[0]) == {"step", "phase", "loss", "lr", "grad_norm", "tokens_per_sec", "wall_s"}
    assert all(abs(e["lr"] - 1e-4) < 1e-10 for e in train)

    # the same two steps through the Python driver: every row is document 0
    ids = torch.from_numpy(np.repeat(tok[:, :-1], A * B, 0).astype(np.int64)).cuda()
    tgt = torch.from_numpy(np.repeat(tok[:, 1:], A * B, 0).astype(np.int64)).cuda()
    m = torch.from_numpy(np.repeat(msk[:, 1:], A * B, 0).astype(np.float32)).cuda()
    w = E.row_weights(m, B, A)
    for k in range(2):
        eng.train_step(ids, tgt, m, w)
        met = eng.read_metrics()
        assert abs(train[k]["loss"] - met["loss"]) <= 1e-5 * abs(met["loss"])
        assert abs(train[k]["grad_norm"] - met["grad_norm"]) <= 5e-4 * met["grad_norm"]   # two runs differ by the order of the split-K adds
    # validation after step 2 = forward loss with the updated weights on the same document
    eng.loss_sums.zero_()
    eng.forward_loss(ids[:3], tgt[:3], m[:3])
    ls = eng.loss_sums.tolist()
    assert abs(val[0]["loss"] - ls[0] / ls[1]) <= 1e-5 * abs(ls[0] / ls[1])

    final = safetensors_io.load_safetensors(run_dir / "final.safetensors")
    for n, v in eng.named_parameters().items():
        ref = v.cpu().numpy()
        assert final[n].shape == ref.shape
        # AdamW's first steps are sign-like: an element whose gradient is atomics-order noise can move by
        # up to 2*lr per step in either run, so bound the error by that and require it to be rare
        d = np.abs(final[n] - ref)
        assert d.max() <= 4.5e-4 and np.mean(d > 2e-5) < (0.15 if "k_proj" in n or "q_proj" in n else 3e-2) and np.median(d) < 1e-6, n
    opt = safetensors_io.load_safetensors(str(run_dir / "final.safetensors") + ".opt.safetensors")
    assert float(opt["optimizer.step"][0]) == 2.0
    assert set(opt) == {"optimizer.step"} | {f"optimizer.{k}.{n}" for k in "mv" for n, _ in names}
    n0 = "model.layers.3.mlp.down_proj.weight"
    st = eng.layout.names.index(n0)
    o, k = eng.layout.offsets[st], eng.layout.numels[st]
    assert np.abs(opt["optimizer.m." + n0].reshape(-1) - eng.m[o:o + k].cpu().numpy()).max() <= 1e-6

    # resume: one more step, log appended, step counter continues
    conf.update(resume_from=str(run_dir / "final.safetensors"), total_steps=3, val_every=0)
    (run_dir / "config.json").write_text(json.dumps(conf))
    r = subprocess.run([str(EXE), "--config", str(run_dir / "config.json")], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "resumed at step 2" in r.stderr
    events = [json.loads(l) for l in (run_dir / "loss.jsonl").read_text().splitlines()]
    assert [e["step"] for e in events if e["phase"] == "train"] == [1, 2, 3]
    eng.train_step(ids, tgt, m, w)
    met = eng.read_metrics()
    assert abs(events[-1]["loss"] - met["loss"]) <= 1e-4 * abs(met["loss"])
    opt = safetensors_io.load_safetensors(str(run_dir / "final.safetensors") + ".opt.safetensors")
    assert float(opt["optimizer.step"][0]) == 3.0


def test_generate_matches_the_python_decoder(tmp_path):
    """ctd_generate on SmolLM2-135M with random weights: greedy tokens equal Decoder.generate; a
    sampled request with top_k = 1 (only the maximum survives) goes through the one-token-at-a-time
    path and must produce the same ids; eos and the thinking budget end / steer the stream."""
    from emberlm_b200 import engine as E
    build.build()
    gen = Path(build.HERE) / "ctd_generate"
    cfg = E.make_config(**E.PRESETS["smollm2_135m"])
    eng = E.TrainEngine(cfg, 1, 8, train=False)
    eng.init_parameters(seed=11)
    w0 = tmp_path / "m.safetensors"
    safetensors_io.save_safetensors([(n, v.cpu().numpy()) for n, v in eng.named_parameters().items()], w0)
    prompt = [5, 17, 300, 4242, 9, 77, 12345]
    dec = E.Decoder(cfg, 64, params=eng.params[:eng.layout.total])
    want = dec.generate(prompt, 24).cpu().tolist()

    def ask(**req):
        r = subprocess.run([str(gen), "--model", str(w0)], input=json.dumps(dict(input_ids=prompt, max_seq_len=64, **req)),
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-1500:]
        lines = [json.loads(l) for l in r.stdout.strip().splitlines()]
        return [l["token"] for l in lines[:-1]], lines[-1]

    toks, done = ask(max_new_tokens=24, temperature=0.0)
    assert toks == want and done == {"done": True, "reason": "max_tokens", "generated_tokens": 24}
    toks, done = ask(max_new_tokens=24, temperature=0.7, top_k=1, seed=3)
    assert toks == want and done["reason"] == "max_tokens"
    toks, done = ask(max_new_tokens=24, temperature=0.0, eos_ids=[want[5]])
    stop = want.index(want[5])
    assert toks == want[:stop + 1] and done["reason"] == "eos" and done["generated_tokens"] == stop + 1
    toks, done = ask(max_new_tokens=200, temperature=0.0)            # the cache (64 positions) ends the run
    assert done["reason"] == "max_seq_len" and toks[:24] == want and len(toks) == 64 - len(prompt) + 1
    # thinking budget (main.cpp:139-170): tokens after the open marker are counted (the count restarts
    # whenever the marker shows up again); once it reaches the budget the close marker is forced
    budget, close = 3, [7, 8]
    toks, done = ask(max_new_tokens=16, temperature=0.0, thinking_token_budget=budget, think_open_ids=[want[0]],
                     think_close_ids=close)
    count, forced_at = 0, None
    for i, t in enumerate(want):
        count = 0 if t == want[0] else count + 1
        if count >= budget:
            forced_at = i + 1
            break
    assert forced_at is not None and forced_at + 2 <= 16
    assert toks[:forced_at] == want[:forced_at] and toks[forced_at:forced_at + 2] == close
