"""Generates tests/golden/ref_step_*.npz by running the reference's own CUDA build of the
training step (oracle/_ref/ref_harness, built from the unmodified reference sources by
oracle/Makefile) on a GPU. Run on a B200 box:  python tests/golden/make_golden.py <out_dir>
The inputs are regenerated from seeds by tests/golden_cases.py, so the fixtures hold only the
reference's outputs: loss and gradient norm per step, the gradients of the first step (before
clipping) and the parameters after the last step."""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import ref_run  # noqa: E402
from tests.golden_cases import CASES, HP, STEPS, build_case  # noqa: E402


def main(out_dir):
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    for name in CASES:
        cfg, params, tok, msk, b, A = build_case(name)
        r = ref_run.run_reference(cfg, params, tok, msk, b, A, steps=STEPS, warmup=0, **HP)
        arrays = {"loss": np.array(r["loss"], np.float32), "grad_norm": np.array(r["grad_norm"], np.float32)}
        for k, v in r["grads"].items():
            arrays["grad/" + k] = v
        for k, v in r["params"].items():
            arrays["param/" + k] = v
        np.savez_compressed(out / f"ref_step_{name}.npz", **arrays)
        print(name, r["loss"], r["grad_norm"])


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else str(Path(__file__).parent))
