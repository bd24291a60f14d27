"""ctd_train command line, host-side behaviour that needs no GPU: usage and error exits
(tools/ctd_train/main.cpp:33-43, 431-434: usage -> exit 2, any error -> "[ctd_train] error: ..."
and exit 1), the config reader and the safetensors header reader."""
import json
import subprocess
from pathlib import Path

import numpy as np
import pytest

from emberlm_b200 import build, safetensors_io

EXE = Path(build.HERE) / "ctd_train"


@pytest.fixture(scope="module", autouse=True)
def _built():
    build.build()
    assert EXE.exists()


def run(*args):
    return subprocess.run([str(EXE), *args], capture_output=True, text=True, timeout=120)


def test_usage_and_missing_config():
    r = run()
    assert r.returncode == 2 and "usage:" in r.stderr and "--config" in r.stderr
    r = run("--config", "/nonexistent/dir/config.json")
    assert r.returncode == 1 and "[ctd_train] error: cannot open config" in r.stderr


def test_config_errors(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text("{ not json")
    r = run("--config", str(cfg))
    assert r.returncode == 1 and "[ctd_train] error: json:" in r.stderr
    cfg.write_text(json.dumps({"data_dir": "x"}))
    r = run("--config", str(cfg))
    assert r.returncode == 1 and "init_weights" in r.stderr          # required key (main.cpp:79)
    cfg.write_text(json.dumps({"init_weights": str(tmp_path / "missing.safetensors"), "data_dir": "x"}))
    r = run("--config", str(cfg))
    assert r.returncode == 1 and "cannot open" in r.stderr and "missing.safetensors" in r.stderr
    cfg.write_text(json.dumps({"init_weights": "w", "data_dir": "x", "precision": "fp8"}))
    r = run("--config", str(cfg))
    assert r.returncode == 1 and "precision" in r.stderr


def test_weights_header_is_parsed_and_unknown_architecture_rejected(tmp_path):
    w = tmp_path / "w.safetensors"
    safetensors_io.save_safetensors([("model.embed_tokens.weight", np.zeros((10, 7), np.float32)),
                                     ("other", np.ones((3,), np.float32))], w)
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps({"init_weights": str(w), "data_dir": str(tmp_path), "run_name": "r"}))
    r = run("--config", str(cfg))
    # same message as autodetect_config (include/ctd/nn/model.h:138-140)
    assert r.returncode == 1 and "autodetect_config: unsupported hidden_size=7 vocab_size=10" in r.stderr
    assert "[ctd_train] run=r" in r.stderr and "loading init weights" in r.stderr
    w2 = tmp_path / "w2.safetensors"
    safetensors_io.save_safetensors([("something.else", np.zeros((2, 2), np.float32))], w2)
    cfg.write_text(json.dumps({"init_weights": str(w2), "data_dir": str(tmp_path)}))
    r = run("--config", str(cfg))
    assert r.returncode == 1 and "model.embed_tokens.weight" in r.stderr
    w3 = tmp_path / "w3.safetensors"
    w3.write_bytes(b"\x10\x00\x00")
    cfg.write_text(json.dumps({"init_weights": str(w3), "data_dir": str(tmp_path)}))
    r = run("--config", str(cfg))
    assert r.returncode == 1 and "short read" in r.stderr


GEN = Path(build.HERE) / "ctd_generate"


def run_gen(request, *args):
    return subprocess.run([str(GEN), *args], input=request, capture_output=True, text=True, timeout=120)


def test_generate_usage_and_errors(tmp_path):
    """tools/ctd_generate/main.cpp:33-44, 186-191: usage -> exit 2; any error -> stderr message, a
    {"done": true, "reason": "error"} line on stdout and exit 1."""
    assert GEN.exists()
    r = run_gen('{"input_ids": [1]}')
    assert r.returncode == 2 and "usage:" in r.stderr and "--model" in r.stderr
    r = run_gen("not json", "--model", "x")
    assert r.returncode == 1 and "[ctd_generate] error: json:" in r.stderr
    last = json.loads(r.stdout.strip().splitlines()[-1])
    assert last["done"] is True and last["reason"] == "error" and "json" in last["error"]
    r = run_gen('{"max_new_tokens": 4}', "--model", "x")
    assert r.returncode == 1 and "input_ids" in r.stderr
    r = run_gen('{"input_ids": [1, 2]}', "--model", str(tmp_path / "missing.safetensors"))
    assert r.returncode == 1 and "cannot open" in r.stderr
    w = tmp_path / "w.safetensors"
    safetensors_io.save_safetensors([("model.embed_tokens.weight", np.zeros((10, 7), np.float32))], w)
    r = run_gen('{"input_ids": [1, 2]}', "--model", str(w))
    assert r.returncode == 1 and "autodetect_config: unsupported hidden_size=7 vocab_size=10" in r.stderr
