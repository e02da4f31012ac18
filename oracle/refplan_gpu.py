"""BENCH INFRASTRUCTURE: ctypes loader for oracle/refplan_gpu.cu (the reference's execution plan
restated as CUDA).  Only bench.py uses it, to time that plan on the same GPU as the library."""
from __future__ import annotations

import ctypes
import subprocess
from ctypes import c_float, c_int, c_int64, c_uint64, c_void_p
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB = HERE / "librefplan_gpu.so"
_lib = None


def build() -> Path:
    src = HERE / "refplan_gpu.cu"
    if not LIB.exists() or src.stat().st_mtime > LIB.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), LIB.name], check=True, capture_output=True)
    return LIB


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(LIB))
        V = c_void_p
        L.refplan_ew_f32.argtypes = [c_int, V, V, V, c_uint64, c_uint64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64]
        L.refplan_mul_scalar_f32.argtypes = [V, c_float, V, c_uint64]
        L.refplan_mul_scalar_i32.argtypes = [V, c_int, V, c_uint64]
        L.refplan_sum_rows_f32.argtypes = [V, c_int64, c_int64, V, V]
        L.refplan_max_index_rows_f32.argtypes = [V, c_int64, c_int64, V]
        L.refplan_sum_cols_f32.argtypes = [V, c_int64, c_int64, V, V]
        L.refplan_gt_scalar_i32.argtypes = [V, c_int, V, c_uint64]
        L.refplan_count_true.argtypes = [V, c_uint64, V]
        for f in ("refplan_ew_f32", "refplan_mul_scalar_f32", "refplan_mul_scalar_i32", "refplan_sum_rows_f32",
                  "refplan_max_index_rows_f32", "refplan_sum_cols_f32", "refplan_gt_scalar_i32", "refplan_count_true"):
            getattr(L, f).restype = None
        _lib = L
    return _lib
