"""TEST / BENCH INFRASTRUCTURE: loader of oracle/_ref/libcumo_ref_kernels.so, the reference's own CUDA kernels
expanded and compiled outside the Ruby extension by oracle/build_ref_kernels.py.  Its launch functions have the
reference's names and argument lists, i.e. exactly those of libcumo_b200.so, so one descriptor set can be handed
to both.  `lib()` returns None where the library has not been built (no reference checkout was ever available)."""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

LIB = Path(__file__).resolve().parent / "_ref" / "libcumo_ref_kernels.so"
_lib = None


def available() -> bool:
    return LIB.exists()


def lib():
    global _lib
    if _lib is None and LIB.exists():
        # local scope: its symbols carry the same names as libcumo_b200's and must not interpose them
        _lib = ctypes.CDLL(str(LIB), mode=os.RTLD_NOW | os.RTLD_LOCAL)
        _lib.refk_last_error.restype = ctypes.c_int
    return _lib
