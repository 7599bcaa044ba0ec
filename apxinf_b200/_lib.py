"""ctypes binding of libpi05_b200.so (the C ABI in include/pi05_b200.h).

The library is the product: if it is missing or cannot be loaded this module
raises — there is no CPU or PyTorch fallback for any operator.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
# PI05_LIB_PATH: another build of the library (A/B measurements of two builds on one machine)
import os as _os
LIB_PATH = Path(_os.environ["PI05_LIB_PATH"]) if _os.environ.get("PI05_LIB_PATH") else _PKG / "libpi05_b200.so"

OP_BF16, OP_E4M3, OP_S8 = 0, 1, 2
OUT_BF16, OUT_E4M3, OUT_F32, OUT_S32 = 0, 1, 2, 3
(EPI_STORE, EPI_BIAS_GELU, EPI_BIAS_SILU, EPI_BIAS_RESIDUAL, EPI_BIAS_POS,
 EPI_GATE_RESIDUAL, EPI_GEGLU, EPI_ROPE, EPI_EULER) = range(9)
PRO_NONE, PRO_ADA_NORM, PRO_QUANTIZE, PRO_RMS_NORM = range(4)
OUT_S8 = 4

STATUS_NAMES = {
    0: "PI05_OK",
    -1: "PI05_ERR_INVALID_VALUE",
    -2: "PI05_ERR_UNSUPPORTED",
    -3: "PI05_ERR_DRIVER",
    -4: "PI05_ERR_CUDA",
    -5: "PI05_ERR_DEVICE_TIMEOUT",
    -6: "PI05_ERR_NOT_BUILT",
    -7: "PI05_ERR_SCRATCH_LIMIT",
}


class Pi05Error(RuntimeError):
    def __init__(self, code: int, where: str, detail: str = ""):
        self.code = code
        name = STATUS_NAMES.get(code, str(code))
        super().__init__(f"{where}: {name}" + (f" ({detail})" if detail else ""))


class GemmArgs(C.Structure):
    _fields_ = [
        ("op", C.c_int32), ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
        ("nb0", C.c_int32), ("nb1", C.c_int32),
        ("a", C.c_void_p), ("lda", C.c_int64), ("a_sb0", C.c_int64), ("a_sb1", C.c_int64),
        ("b", C.c_void_p), ("ldb", C.c_int64), ("b_sb0", C.c_int64), ("b_sb1", C.c_int64),
        ("b_mn_major", C.c_int32),
        ("out", C.c_void_p), ("ldc", C.c_int64), ("out_sb0", C.c_int64), ("out_sb1", C.c_int64),
        ("out_type", C.c_int32), ("mode", C.c_int32),
        ("residual", C.c_void_p), ("bias", C.c_void_p),
        ("col_scale", C.c_void_p), ("row_scale", C.c_void_p),
        ("pos", C.c_void_p), ("pos_rows", C.c_int32), ("pos_ld", C.c_int64),
        ("gate", C.c_void_p),
        ("alpha", C.c_float), ("out_inv_scale", C.c_float),
        ("status", C.c_void_p),
        ("force_swap", C.c_int32), ("force_block_n", C.c_int32),
        ("partials", C.c_void_p), ("partials_bytes", C.c_uint64),
        ("tile_counters", C.c_void_p), ("max_tiles", C.c_int32), ("force_split_k", C.c_int32),
        ("b_blocked", C.c_int32),
        ("force_skinny", C.c_int32), ("prologue", C.c_int32), ("style", C.c_void_p),
        ("eps", C.c_float), ("a_inv_scale", C.c_float), ("a_dynamic_rows", C.c_int32),
        ("rope_q_out", C.c_void_p), ("rope_k_cache", C.c_void_p), ("rope_v_cache", C.c_void_p),
        ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p),
        ("rope_tokens", C.c_int32), ("rope_q_heads", C.c_int32), ("rope_head_dim", C.c_int32),
        ("rope_position_offset", C.c_int32), ("rope_cache_rows", C.c_int32), ("dt", C.c_float),
        ("k_slices", C.c_int32),
    ]


_lib = None


def lib() -> C.CDLL:
    """Load the shared library once; fail loudly when it is absent."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise Pi05Error(-6, "load libpi05_b200.so",
                            f"{LIB_PATH} not built; run `python -m apxinf_b200.build`")
        handle = C.CDLL(str(LIB_PATH))
        handle.pi05_last_cuda_error.restype = C.c_char_p
        handle.pi05_version.restype = C.c_char_p
        handle.pi05_gemm.argtypes = [C.POINTER(GemmArgs), C.c_void_p]
        handle.pi05_gemm.restype = C.c_int
        handle.pi05_gemm_static_scratch.argtypes = [C.POINTER(GemmArgs), C.c_void_p]
        handle.pi05_gemm_static_scratch.restype = C.c_int
        _declare_optional(handle)
        _lib = handle
    return _lib


def _declare_optional(handle: C.CDLL) -> None:
    from . import _abi_decls
    _abi_decls.declare(handle)


def check(code: int, where: str) -> None:
    if code != 0:
        detail = ""
        if code in (-4, -7):
            detail = (lib().pi05_last_cuda_error() or b"").decode()
        raise Pi05Error(code, where, detail)
