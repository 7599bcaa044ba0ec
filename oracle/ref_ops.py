"""Loader for the reference's own CUDA kernels compiled by oracle/Makefile into oracle/_ref
(test infrastructure: only tests may import this). The three libraries are the reference's
self-contained adapters crates/apxinf-cuda/adapters/{static_bf16_adapter,custom_kernels,
w8a8_adapter}.cu with the kernels of crates/apxinf-cuda/kernels/custom/*.cuh, built for sm_100a
from the reference tree; nothing of them is copied into this repository."""
import ctypes as C
from pathlib import Path

_DIR = Path(__file__).resolve().parent / "_ref"
_NAMES = {"bf16": "libref_static_bf16_adapter.so", "f16": "libref_custom_kernels.so",
          "w8a8": "libref_w8a8_adapter.so"}
_HANDLES = {}


def available() -> bool:
    return all((_DIR / name).exists() for name in _NAMES.values())


def lib(which: str) -> C.CDLL:
    """which: "bf16" (static BF16 operators), "f16" (F16/E4M3 operators) or "w8a8"."""
    if which not in _HANDLES:
        _HANDLES[which] = C.CDLL(str(_DIR / _NAMES[which]))  # RTLD_LOCAL: names stay private
    return _HANDLES[which]
