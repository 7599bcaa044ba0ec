"""ctypes prototypes for the engine-level and kernel-level C ABI (include/pi05_b200.h)."""
from __future__ import annotations

import ctypes as C


def declare(handle: C.CDLL) -> None:
    """Attach argtypes/restype to every exported symbol beyond pi05_gemm."""
    for name, restype, argtypes in PROTOTYPES:
        fn = getattr(handle, name)
        fn.restype = restype
        fn.argtypes = argtypes


PROTOTYPES: list = []
