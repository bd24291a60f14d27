"""ctypes binding of libctdk.so. Signatures follow include/ctdk.h one to one."""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libctdk.so"
HEADER = HERE.parent / "include" / "ctdk.h"

CTDK_OK, CTDK_EINVAL, CTDK_ELAUNCH, CTDK_ETIMEOUT, CTDK_ENOMEM = 0, -1, -2, -3, -4
GEMM_TF32, GEMM_3XTF32, GEMM_FP32_SIMT = 0, 1, 2
EPI_STORE, EPI_ACCUMULATE, EPI_RESIDUAL = 0, 1, 2


class CtdkError(RuntimeError):
    """Raised for any non-zero status, like the reference's std::runtime_error."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"ctdk error {code}: {msg}")
        self.code = code


class RopeParams(C.Structure):
    _fields_ = [("theta", C.c_float), ("scaling_factor", C.c_float),
                ("low_freq_wavelen", C.c_float), ("high_freq_wavelen", C.c_float)]


class AdamWParams(C.Structure):
    _fields_ = [("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float),
                ("eps", C.c_float), ("wd", C.c_float), ("bc1", C.c_float), ("bc2", C.c_float)]


def declared_symbols() -> list[str]:
    """Every function name include/ctdk.h declares."""
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(ctdk_[a-z0-9_]+)\s*\(", text)))


def load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m emberlm_b200.build` "
            "(there is no CPU fallback)")
    return C.CDLL(str(LIB_PATH))


_lib = load()

_p, _i, _l, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float
_SIGS = {
    "ctdk_reserve_sms": [_i],
    "ctdk_gemm": [_p, _p, _p, _l, _l, _l, _l, _l, _l, _i, _i, _i, _i, _p, _p],
    "ctdk_gemm_ws": [_p, _p, _p, _l, _l, _l, _l, _l, _l, _i, _i, _i, _i, _p, _p, _l, _p],
    "ctdk_attn_fwd_p": [_p, _p, _p, _l, _l, _i, _i, _i, _i, _p],
    "ctdk_attn_bwd_p": [_p, _p, _p, _p, _p, _p, _l, _l, _i, _i, _i, _i, _p],
    "ctdk_gemm_swiglu": [_p, _p, _p, _p, _l, _l, _l, _i, _p],
    "ctdk_gemm_swiglu_bwd": [_p, _p, _p, _p, _p, _l, _l, _l, _i, _p],
    "ctdk_gemm_dattn_delta": [_p, _p, _p, _p, _p, _l, _l, _i, _i, _l, _i, _p],
    "ctdk_bmm": [_p, _p, _p, _l, _l, _l, _l, _i, _i, _i, _p],
    "ctdk_rmsnorm_fwd": [_p, _p, _p, _p, _l, _i, _f, _p],
    "ctdk_rmsnorm_bwd": [_p, _p, _p, _p, _p, _p, _l, _i, _f, _i, _i, _p],
    "ctdk_rmsnorm_bwd_static": [_p, _p, _p, _p, _p, _l, _i, _f, _i, _i, _p],
    "ctdk_rope": [_p, _p, _l, _l, _i, _i, _l, _i, C.POINTER(RopeParams), _f, _p],
    "ctdk_rope_table": [_p, _l, _i, _i, C.POINTER(RopeParams), _p],
    "ctdk_qk_norm_rope_fwd": [_p, _p, _p, _p, _p, _p, _p, _l, _l, _i, _i, _i, _f, _p],
    "ctdk_qk_norm_rope_bwd": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _l, _l, _i, _i, _i, _i, _p],
    "ctdk_add": [_p, _p, _p, _l, _p],
    "ctdk_sub": [_p, _p, _p, _l, _p],
    "ctdk_mul": [_p, _p, _p, _l, _p],
    "ctdk_scale": [_p, _f, _p, _l, _p],
    "ctdk_silu": [_p, _p, _l, _p],
    "ctdk_silu_bwd": [_p, _p, _p, _l, _p],
    "ctdk_swiglu_fwd": [_p, _p, _l, _i, _p],
    "ctdk_swiglu_bwd": [_p, _p, _p, _l, _i, _p],
    "ctdk_embedding_fwd": [_p, _p, _p, _l, _i, _l, _p],
    "ctdk_embedding_bwd": [_p, _p, _p, _l, _i, _l, _p],
    "ctdk_ce_masked": [_p, _p, _p, _p, _p, _p, _l, _l, _i, _p],
    "ctdk_gather_rows": [_p, _p, _p, _l, _i, _p],
    "ctdk_scatter_rows": [_p, _p, _p, _l, _i, _p],
    "ctdk_gather_ce_inputs": [_p, _p, _p, _p, _p, _p, _p, _l, _p],
    "ctdk_attn_fwd": [_p, _p, _p, _l, _l, _i, _i, _i, _p],
    "ctdk_attn_bwd": [_p, _p, _p, _p, _p, _p, _l, _l, _i, _i, _i, _p],
    "ctdk_sumsq": [_p, _l, _p, _p],
    "ctdk_clip_scale": [_p, _f, _f, _p, _p, _p],
    "ctdk_adamw": [_p, _p, _p, _p, _l, C.POINTER(AdamWParams), _p, _p, _p, _i, _p],
    "ctdk_device_status": [_p, C.POINTER(C.c_int)],
    "ctdk_softmax_fwd": [_p, _p, _l, _l, _p],
    "ctdk_softmax_bwd": [_p, _p, _p, _l, _l, _p],
    "ctdk_permute": [_p, _p, _i, C.POINTER(C.c_int64), C.POINTER(C.c_int), _p],
    "ctdk_repeat_kv": [_p, _p, _l, _i, _i, _i, _p],
    "ctdk_repeat_kv_sum": [_p, _p, _l, _i, _i, _i, _p],
    "ctdk_causal_mask": [_p, _p, _l, _l, _l, _i, _f, _p],
    "ctdk_mse_fwd": [_p, _p, _l, _p, _p],
    "ctdk_mse_bwd": [_p, _p, _p, _p, _l, _p],
    "ctdk_kv_write": [_p, _p, _l, _l, _i, _i, _l, _l, _p],
    "ctdk_kv_read_expanded": [_p, _p, _l, _i, _i, _l, _i, _l, _p],
    "ctdk_loss_ratio": [_p, _p, _p],
    "ctdk_sample": [_p, _l, _l, _f, _i, _f, _p, _p, _p, _p],
    "ctdk_ce_row_weight": [_p, _p, _p, _l, _p, _p],
}
for _name, _args in _SIGS.items():
    _fn = getattr(_lib, _name)
    _fn.argtypes = _args
    _fn.restype = C.c_int
_lib.ctdk_last_error.restype = C.c_char_p
_lib.ctdk_last_error.argtypes = []
_lib.ctdk_sm_count.restype = C.c_int
_lib.ctdk_launch_count.restype = C.c_longlong
_lib.ctdk_launch_count.argtypes = []
_lib.ctdk_prof_enable.restype = C.c_int
_lib.ctdk_prof_enable.argtypes = [C.c_int]
_lib.ctdk_prof_collect.restype = C.c_int
_lib.ctdk_prof_collect.argtypes = [C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double),
                                   C.POINTER(C.c_longlong)]
_lib.ctdk_sample_workspace_bytes.restype = C.c_int64
_lib.ctdk_sample_workspace_bytes.argtypes = [C.c_int64, C.c_int64]
_lib.ctdk_rmsnorm_bwd_scratch_floats.restype = C.c_int64
_lib.ctdk_rmsnorm_bwd_scratch_floats.argtypes = [C.c_int]
_lib.ctdk_gemm_3xtf32_workspace_floats.restype = C.c_int64
_lib.ctdk_gemm_3xtf32_workspace_floats.argtypes = [C.c_int64, C.c_int64, C.c_int64]
_lib.ctdk_qk_norm_rope_bwd_scratch_floats.restype = C.c_int64
_lib.ctdk_qk_norm_rope_bwd_scratch_floats.argtypes = [C.c_int]


def raw() -> C.CDLL:
    return _lib


def last_error() -> str:
    return _lib.ctdk_last_error().decode()


def check(rc: int) -> None:
    if rc != 0:
        raise CtdkError(rc, last_error())


def call(name: str, *args) -> None:
    """Calls a status-returning entry point and raises CtdkError on failure."""
    check(getattr(_lib, name)(*args))
