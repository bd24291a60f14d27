"""Reader / writer for the reference's safetensors files (weights `*.safetensors` and optimizer
state `*.opt.safetensors`), byte-compatible with emberlm's src/core/safetensors.cpp:

  8-byte little-endian header length | JSON header | raw little-endian tensor data
  header: {"name": {"dtype": "F32", "shape": [...], "data_offsets": [begin, end]}, ...}
  The reference emits header keys in alphabetical order (an ordered JSON object,
  safetensors.cpp:100-115) while data offsets follow the caller's tensor order, and pads the
  header with spaces to a multiple of 8 bytes (safetensors.cpp:118-119). It reads F32 / I64 /
  I32 and ignores "__metadata__" (safetensors.cpp:55-66); it writes F32 only.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np

_DTYPES = {"F32": np.float32, "I64": np.int64, "I32": np.int32}
_NAMES = {np.dtype(np.float32): "F32"}


def save_safetensors(named_tensors, path) -> None:
    """named_tensors: iterable of (name, array-like fp32). Order is preserved in the data section."""
    items = [(n, np.ascontiguousarray(a)) for n, a in named_tensors]
    header, running = {}, 0
    for name, a in items:
        if a.dtype != np.float32:
            raise RuntimeError(f"save_safetensors: only fp32 supported, got {name}")
        header[name] = {"dtype": "F32", "shape": list(a.shape), "data_offsets": [running, running + a.nbytes]}
        running += a.nbytes
    text = json.dumps(header, sort_keys=True, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for _, a in items:
            f.write(a.tobytes())


def load_safetensors(path) -> dict:
    """Returns {name: numpy array}; raises RuntimeError on the conditions the reference throws on."""
    data = Path(path).read_bytes()
    if len(data) < 8:
        raise RuntimeError("safetensors: short read on header length")
    (hlen,) = struct.unpack("<Q", data[:8])
    if 8 + hlen > len(data):
        raise RuntimeError("safetensors: short read on header")
    header = json.loads(data[8:8 + hlen])
    origin = 8 + hlen
    out = {}
    for name, spec in header.items():
        if name == "__metadata__":
            continue
        dt = spec["dtype"]
        if dt not in _DTYPES:
            raise RuntimeError(f"safetensors: {name} has dtype {dt} which is not supported on the read path")
        b, e = spec["data_offsets"]
        arr = np.frombuffer(data, dtype=_DTYPES[dt], count=(e - b) // np.dtype(_DTYPES[dt]).itemsize,
                            offset=origin + b)
        shape = tuple(spec["shape"])
        if arr.size != int(np.prod(shape, dtype=np.int64)):
            raise RuntimeError(f"safetensors: size mismatch for {name}")
        out[name] = arr.reshape(shape).copy()
    return out
