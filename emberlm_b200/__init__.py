"""emberlm_b200 — B200-native kernels for emberlm's decoder training step.

The product is `libctdk.so` (hand-written sm_100a CUDA behind the C-ABI declared in
`include/ctdk.h`). This package only loads it and offers thin host-side helpers that
mirror the reference's `ctd::ops` / `ctd::optim` interface for tests and the benchmark.
There is no CPU fallback: importing `emberlm_b200.lib` fails loudly when the library has
not been built (`python -m emberlm_b200.build`).
"""

__all__ = ["build", "lib", "ops"]
