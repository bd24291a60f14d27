"""Runs the reference's own CUDA build of the training step (oracle/_ref/ref_harness, built by
oracle/Makefile from the unmodified reference sources) on the same bytes the ctdk engine gets.
TEST / BENCH INFRASTRUCTURE ONLY. Needs a GPU; the binary is prebuilt where the reference
sources are available and travels with the repository snapshot."""
from __future__ import annotations

import json
import subprocess
import tempfile
from dataclasses import asdict
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
BINARY = HERE / "_ref" / "ref_harness"


def available() -> bool:
    return BINARY.exists()


def run_reference(cfg, params: dict, tok: np.ndarray, msk: np.ndarray, batch_size: int, accum: int,
                  steps: int = 1, warmup: int = 0, lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8,
                  weight_decay=0.01, clip=1.0, gradient_checkpointing=False, want_grads=True,
                  want_params=True, timeout=1800):
    """cfg: oracle.model.LlamaConfig; params: {name: fp32 array}; tok int32 / msk int8 [docs, S].
    Returns dict(loss=[...], grad_norm=[...], step_ms=[...], grads={...} | None, params={...} | None)."""
    from safetensors.numpy import load_file, save_file
    if not available():
        raise RuntimeError(f"{BINARY} is missing: run `make -C oracle` where the reference sources are")
    with tempfile.TemporaryDirectory(prefix="ref_harness_") as d:
        d = Path(d)
        save_file({k: np.ascontiguousarray(v, dtype=np.float32) for k, v in params.items()}, str(d / "w.safetensors"))
        np.ascontiguousarray(tok, dtype=np.int32).tofile(d / "tokens.bin")
        np.ascontiguousarray(msk, dtype=np.int8).tofile(d / "mask.bin")
        spec = dict(weights=str(d / "w.safetensors"), tokens=str(d / "tokens.bin"), mask=str(d / "mask.bin"),
                    seq_len=int(tok.shape[1]), batch_size=batch_size, grad_accum_steps=accum, steps=steps,
                    warmup=warmup, lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay,
                    clip=clip, gradient_checkpointing=bool(gradient_checkpointing),
                    dump_grads=str(d / "grads.safetensors") if want_grads else "",
                    dump_params=str(d / "params.safetensors") if want_params else "",
                    config=asdict(cfg))
        (d / "spec.json").write_text(json.dumps(spec))
        r = subprocess.run([str(BINARY), str(d / "spec.json")], capture_output=True, text=True, timeout=timeout)
        if r.returncode != 0:
            raise RuntimeError(f"ref_harness failed ({r.returncode}): {r.stderr[-2000:]}")
        out = json.loads(r.stdout.strip().splitlines()[-1])
        out["grads"] = load_file(str(d / "grads.safetensors")) if want_grads else None
        out["params"] = load_file(str(d / "params.safetensors")) if want_params else None
        return out
