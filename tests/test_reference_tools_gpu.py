"""The reference's two command-line tools in three builds, on the same files:
  ref_*   the reference's tool source + the reference's own library (oracle/_ref, unmodified sources)
  api_*   the SAME tool source compiled against this repository's include/ctd headers and libctdk.so
  ours    this repository's own tools (emberlm_b200/ctd_train, ctd_generate)
All are built ahead of time (oracle/Makefile, emberlm_b200/build.py). Checked here: the three
trainers log the same losses / gradient norms / validation loss on the same config and bins and
end with the same weights within the TF32 tolerance; a run directory written by one resumes under
another (weights, optimizer.m / optimizer.v by name, optimizer.step); the three generators emit
the same seeded token stream for the same request."""
import json
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from emberlm_b200 import build, safetensors_io

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "oracle" / "_ref"
TRAINERS = {"ref": REF / "ref_ctd_train", "api": REF / "api_ctd_train", "ours": Path(build.HERE) / "ctd_train"}
GENERATORS = {"ref": REF / "ref_ctd_generate", "api": REF / "api_ctd_generate", "ours": Path(build.HERE) / "ctd_generate"}
needs_tools = pytest.mark.skipif(not all(p.exists() for p in list(TRAINERS.values()) + list(GENERATORS.values())),
                                 reason="oracle/_ref tools not built (make -C oracle where the reference sources are)")
S, B, A = 65, 2, 2
HP = dict(lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)


@pytest.fixture(scope="module")
def workspace(tmp_path_factory):
    """SmolLM2-135M-shaped random weights (the tools detect the architecture from the embedding's
    shape) and small bins."""
    from emberlm_b200 import engine as E
    root = tmp_path_factory.mktemp("tools")
    cfg = E.make_config(**E.PRESETS["smollm2_135m"])
    eng = E.TrainEngine(cfg, 1, 8, train=False)
    eng.init_parameters(seed=5)
    names = [(n, v.cpu().numpy()) for n, v in eng.named_parameters().items()]
    w0 = root / "init.safetensors"
    safetensors_io.save_safetensors(names, w0)
    del eng
    torch.cuda.empty_cache()
    rng = np.random.default_rng(9)
    docs = 6
    tok = rng.integers(0, cfg.vocab_size, size=(docs, S), dtype=np.int32)
    msk = np.zeros((docs, S), np.int8)
    for d in range(docs):
        msk[d, 10 + d:40 + d] = 1
    data = root / "data"
    data.mkdir()
    for name, arr in (("train.bin", tok), ("train_mask.bin", msk), ("val.bin", tok[:3]), ("val_mask.bin", msk[:3])):
        arr.tofile(data / name)
    return root, w0, data, [n for n, _ in names]


def run_trainer(which, run_dir, **conf):
    run_dir.mkdir(parents=True, exist_ok=True)
    (run_dir / "config.json").write_text(json.dumps(conf))
    r = subprocess.run([str(TRAINERS[which]), "--config", str(run_dir / "config.json")], capture_output=True, text=True, timeout=1200)
    assert r.returncode == 0, f"{which}: {r.stderr[-2000:]}"
    events = [json.loads(l) for l in (run_dir / "loss.jsonl").read_text().splitlines()]
    return events, r.stderr


def base_conf(w0, data, **kw):
    conf = dict(init_weights=str(w0), data_dir=str(data), seq_len=S, batch_size=B, grad_accum_steps=A, total_steps=2,
                warmup_steps=0, min_lr_ratio=1.0, clip_grad_norm=1.0, val_every=2, save_every=0, log_every=1, seed=42, **HP)
    conf.update(kw)
    return conf


@needs_tools
def test_three_trainers_agree_and_checkpoints_interchange(workspace):
    root, w0, data, names = workspace
    ev, finals = {}, {}
    for which in TRAINERS:
        ev[which], err = run_trainer(which, root / f"run_{which}", **base_conf(w0, data))
        assert "arch: hidden=576 layers=30 heads=9" in err
        finals[which] = safetensors_io.load_safetensors(root / f"run_{which}" / "final.safetensors")
    train = {k: [e for e in v if e["phase"] == "train"] for k, v in ev.items()}
    val = {k: [e for e in v if e["phase"] == "val"] for k, v in ev.items()}
    for which in ("api", "ours"):
        assert [e["step"] for e in train[which]] == [1, 2] and [e["step"] for e in val[which]] == [2]
        assert set(train[which][0]) == set(train["ref"][0])          # the same loss.jsonl keys
        for a, b in zip(train[which], train["ref"]):
            assert abs(a["loss"] - b["loss"]) <= 1e-3 * abs(b["loss"]), (which, a, b)
            assert abs(a["grad_norm"] - b["grad_norm"]) <= 1e-2 * b["grad_norm"], (which, a, b)
            assert abs(a["lr"] - b["lr"]) < 1e-12
        assert abs(val[which][0]["loss"] - val["ref"][0]["loss"]) <= 1e-3 * abs(val["ref"][0]["loss"])
        assert set(finals[which]) == set(finals["ref"]) == set(names)
        for n in names:
            d = np.abs(finals[which][n] - finals["ref"][n]).max() / max(np.abs(finals["ref"][n]).max(), 1e-30)
            assert d <= 1e-2, (which, n, d)
    opt = {k: safetensors_io.load_safetensors(str(root / f"run_{k}" / "final.safetensors") + ".opt.safetensors") for k in TRAINERS}
    for which in ("api", "ours"):
        assert set(opt[which]) == set(opt["ref"])
        assert float(opt[which]["optimizer.step"][0]) == 2.0
        for key in ("optimizer.m.model.layers.3.mlp.down_proj.weight", "optimizer.v.model.norm.weight"):
            d = np.abs(opt[which][key] - opt["ref"][key]).max() / max(np.abs(opt["ref"][key]).max(), 1e-30)
            assert d <= 2e-2, (which, key, d)

    # every writer's run directory resumes under every other reader: one more step, counter continues
    step3 = {}
    for writer in TRAINERS:
        for reader in TRAINERS:
            if writer == reader and writer != "ref":
                continue
            src = root / f"run_{writer}"
            dst = root / f"resume_{writer}_to_{reader}"
            dst.mkdir()
            for f in ("final.safetensors", "final.safetensors.opt.safetensors"):
                (dst / f).write_bytes((src / f).read_bytes())
            events, err = run_trainer(reader, dst, **base_conf(w0, data, resume_from=str(dst / "final.safetensors"), total_steps=3,
                                                               val_every=0))
            assert "resumed at step 2" in err, (writer, reader, err[-500:])
            last = [e for e in events if e["phase"] == "train"][-1]
            assert last["step"] == 3
            step3[(writer, reader)] = last["loss"]
            o = safetensors_io.load_safetensors(str(dst / "final.safetensors") + ".opt.safetensors")
            assert float(o["optimizer.step"][0]) == 3.0
    want = step3[("ref", "ref")]
    for k, v in step3.items():
        assert abs(v - want) <= 1e-3 * abs(want), (k, v, want)


@needs_tools
def test_three_generators_emit_the_same_seeded_stream(workspace):
    root, w0, data, names = workspace
    prompt = [5, 17, 300, 4242, 9, 77, 12345]
    # Low temperatures: with the plain random weights the logits of 49 152 tokens differ by a standard
    # deviation of 0.5, i.e. at temperature 1 the distribution is flat and every draw sits within
    # rounding of an inverse-CDF boundary one time in five; at 0.2 - 0.3 a few hundred tokens carry
    # the mass.
    def ask(which, model=w0, **req):
        # exact fp32 products everywhere, as in the reference: this repo's generator by default, the
        # reference's source on this repo's headers through CTD_MATMUL_PRECISION
        r = subprocess.run([str(GENERATORS[which]), "--model", str(model)], input=json.dumps(dict(input_ids=prompt, max_seq_len=64, **req)),
                           capture_output=True, text=True, timeout=900, env=dict(os.environ, CTD_MATMUL_PRECISION="fp32"))
        assert r.returncode == 0, f"{which}: {r.stderr[-1500:]}"
        lines = [json.loads(l) for l in r.stdout.strip().splitlines()]
        return [l["token"] for l in lines[:-1]], lines[-1]

    # Sampled requests draw the same tokens from the same seed when sampler, draw order and logits
    # agree. What is left between the builds is fp32 rounding (different summation orders, this repo's
    # libm-accurate RoPE table against the reference's fast-math one): a draw that falls within it of
    # an inverse-CDF boundary lands on the neighbouring surviving id, and from there on the streams
    # condition on different tokens. So: identical up to the first difference; a first difference in
    # at most one of the three requests per build; and for the pure-temperature request, where every id
    # survives, that difference is a neighbouring id.
    differing = {w: 0 for w in ("api", "ours")}
    for req in (dict(temperature=0.25, seed=7), dict(temperature=0.2, top_p=0.9, seed=11), dict(temperature=0.3, top_k=50, seed=3)):
        got = {w: ask(w, max_new_tokens=16, **req) for w in GENERATORS}
        assert got["ref"][1] == {"done": True, "reason": "max_tokens", "generated_tokens": 16}
        print(req, {w: got[w][0] for w in got})
        for w in ("api", "ours"):
            assert got[w][1] == got["ref"][1], (w, req)
            a, b = got[w][0], got["ref"][0]
            first = next((i for i in range(len(b)) if a[i] != b[i]), None)
            if first is not None:
                differing[w] += 1
                if "top_k" not in req and "top_p" not in req:
                    assert abs(a[first] - b[first]) <= 3, (w, req, first, a, b)
    assert max(differing.values()) <= 1, differing
    # the TF32 prompt pass of this repo's generator is an option, not the default: it runs and answers
    r = subprocess.run([str(GENERATORS["ours"]), "--model", str(w0), "--precision", "tf32"],
                       input=json.dumps(dict(input_ids=prompt, max_seq_len=64, max_new_tokens=4, temperature=0.0)), capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0 and json.loads(r.stdout.strip().splitlines()[-1])["generated_tokens"] == 4
    # protocol corners on every build: empty prompt, the cache limit
    for w in GENERATORS:
        r = subprocess.run([str(GENERATORS[w]), "--model", str(w0)], input=json.dumps(dict(input_ids=[])), capture_output=True, text=True,
                           timeout=900)
        assert json.loads(r.stdout.strip().splitlines()[-1]) == {"done": True, "reason": "empty_prompt"}, w
        toks, done = ask(w, max_new_tokens=200, temperature=0.0)
        assert done["reason"] == "max_seq_len" and len(toks) == 64 - len(prompt) + 1, w   # the last token needs no cache position
