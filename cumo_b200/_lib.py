"""ctypes binding of libcumo_b200.so.

The library is the product: if it is missing this module raises, and nothing in
the package falls back to another implementation.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_int, c_int32, c_int64, c_size_t, c_uint32, c_uint64, c_void_p
from pathlib import Path

MAX_DIM = 12
LIB_PATH = Path(__file__).resolve().parent / "libcumo_b200.so"


class NaIndexer(ctypes.Structure):
    """cumo_na_indexer_t (ext/cumo/include/cumo/indexer.h:16-22)."""
    _fields_ = [("ndim", ctypes.c_ubyte), ("total_size", c_size_t), ("shape", c_size_t * MAX_DIM),
                ("index", c_uint64 * MAX_DIM), ("raw_index", c_uint64)]


class NaIArray(ctypes.Structure):
    """cumo_na_iarray_t (indexer.h:28-31): pointer and BYTE steps."""
    _fields_ = [("ptr", c_void_p), ("step", ctypes.c_ssize_t * MAX_DIM)]


class NaBitIArray(ctypes.Structure):
    """cumo_na_bit_iarray_t (indexer.h:40-44): word pointer, BIT position and BIT steps."""
    _fields_ = [("ptr", c_void_p), ("pos", c_size_t), ("step", ctypes.c_ssize_t * MAX_DIM)]


class NaReductionArg(ctypes.Structure):
    """cumo_na_reduction_arg_t (indexer.h:63-68)."""
    _fields_ = [("in_", NaIArray), ("out", NaIArray), ("in_indexer", NaIndexer), ("out_indexer", NaIndexer)]


_lib = None


def load() -> ctypes.CDLL:
    """Load the library (once).  Building it is `python -m cumo_b200.build`."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m cumo_b200.build` "
            "(nvcc, sm_100a). cumo_b200 has no other execution path.")
    lib = ctypes.CDLL(str(LIB_PATH), mode=os.RTLD_NOW | os.RTLD_GLOBAL)
    _declare(lib)
    _lib = lib
    return lib


def _declare(lib: ctypes.CDLL) -> None:
    H = c_void_p  # cb200_na_t*
    P64 = POINTER(c_int64)
    sig = {
        "cb200_host_error": (c_char_p, [POINTER(c_char_p)]),
        "cb200_na_new": (H, [c_int, c_int, P64]),
        "cb200_na_zeros": (H, [c_int, c_int, P64]),
        "cb200_na_wrap": (H, [c_int, c_int, P64, P64, c_void_p, c_int64]),
        "cb200_na_view": (H, [H, c_int, P64, P64, c_int64]),
        "cb200_na_release": (None, [H]),
        "cb200_na_dtype": (c_int, [H]),
        "cb200_na_ndim": (c_int, [H]),
        "cb200_na_size": (c_int64, [H]),
        "cb200_na_shape": (None, [H, P64]),
        "cb200_na_steps": (None, [H, P64]),
        "cb200_na_offset": (c_int64, [H]),
        "cb200_na_base": (c_void_p, [H]),
        "cb200_na_is_contiguous": (c_int, [H]),
        "cb200_na_set_inplace": (None, [H, c_int]),
        "cb200_na_store_host": (c_int, [H, c_void_p, c_size_t]),
        "cb200_na_read_host": (c_int, [H, c_void_p, c_size_t]),
        "cb200_na_read_host_async": (c_int, [H, c_void_p, c_size_t, c_void_p]),
        "cb200_synchronize": (c_int, []),
        "cb200_na_binary": (H, [c_char_p, H, H]),
        "cb200_na_binary_scalar": (H, [c_char_p, H, c_double, c_int64, c_int]),
        "cb200_na_pow_int": (H, [H, c_int32]),
        "cb200_na_unary": (H, [c_char_p, H]),
        "cb200_na_compare": (H, [c_char_p, H, H]),
        "cb200_na_compare_scalar": (H, [c_char_p, H, c_double, c_int64, c_int]),
        "cb200_na_reduce": (H, [c_char_p, H, c_uint32, c_int, c_int]),
        "cb200_na_minmax": (c_int, [H, c_uint32, c_int, c_int, POINTER(H), POINTER(H)]),
        "cb200_na_bincount": (H, [H, H, c_int64]),
        "cb200_na_cum": (H, [c_char_p, H, c_int, c_int]),
        "cb200_na_where": (H, [H, c_int]),
        "cb200_na_arg_with_value": (c_int, [c_char_p, H, c_uint32, c_int, POINTER(H), POINTER(H)]),
        "cb200_na_arg_with_value_into": (c_int, [c_char_p, H, c_uint32, c_int, c_int64, c_void_p, c_void_p, POINTER(H), POINTER(H)]),
        "cb200_peer_buffer_bytes": (c_size_t, [c_size_t, c_int]),
        "cb200_peer_buffer_create": (c_int, [c_size_t, c_int, POINTER(c_void_p), c_void_p]),
        "cb200_peer_buffer_open": (c_int, [c_void_p, POINTER(c_void_p)]),
        "cb200_peer_buffer_close": (c_int, [c_void_p]),
        "cb200_peer_buffer_destroy": (c_int, [c_void_p]),
        "cb200_peer_exchange_kernel_launch": (c_int, [c_void_p, c_size_t, POINTER(c_void_p), c_int, c_int, c_size_t, ctypes.c_ulonglong, ctypes.c_uint, c_void_p]),
        "cb200_peer_exchange_fold_kernel_launch": (c_int, [c_void_p, c_int, c_int, c_int64, c_double, c_int, c_void_p, POINTER(c_void_p), c_int, c_int,
                                                   c_size_t, ctypes.c_ulonglong, ctypes.c_uint, c_void_p]),
        "cb200_peer_exchange_arg_kernel_launch": (c_int, [c_void_p, c_int, c_int64, c_size_t, c_int, c_int, c_void_p, POINTER(c_void_p), c_int, c_int,
                                                  c_size_t, ctypes.c_ulonglong, ctypes.c_uint, c_void_p]),
        "cb200_tile_pipeline_status": (c_int, []),
        "cb200_tile_pipeline_launches": (ctypes.c_ulonglong, []),
        "cb200_sfloat_rank_fold_sum_kernel_launch": (None, [c_void_p, c_int64, c_int, c_int64, c_double, c_void_p]),
        "cb200_dfloat_rank_fold_sum_kernel_launch": (None, [c_void_p, c_int64, c_int, c_int64, c_double, c_void_p]),
        "cb200_sfloat_rank_fold_extreme_kernel_launch": (None, [c_void_p, c_int64, c_int, c_int64, c_int, c_int, c_void_p]),
        "cb200_dfloat_rank_fold_extreme_kernel_launch": (None, [c_void_p, c_int64, c_int, c_int64, c_int, c_int, c_void_p]),
        "cb200_int32_rank_fold_extreme_kernel_launch": (None, [c_void_p, c_int64, c_int, c_int64, c_int, c_int, c_void_p]),
        "cb200_int64_rank_fold_extreme_kernel_launch": (None, [c_void_p, c_int64, c_int, c_int64, c_int, c_int, c_void_p]),
        "cb200_sfloat_rank_fold_arg_kernel_launch": (None, [c_void_p, c_void_p, c_int64, c_int, c_int64, c_int, c_int, c_void_p, c_void_p]),
        "cb200_dfloat_rank_fold_arg_kernel_launch": (None, [c_void_p, c_void_p, c_int64, c_int, c_int64, c_int, c_int, c_void_p, c_void_p]),
        "cb200_int32_rank_fold_arg_kernel_launch": (None, [c_void_p, c_void_p, c_int64, c_int, c_int64, c_int, c_int, c_void_p, c_void_p]),
        "cb200_int64_rank_fold_arg_kernel_launch": (None, [c_void_p, c_void_p, c_int64, c_int, c_int64, c_int, c_int, c_void_p, c_void_p]),
        "cb200_na_take": (H, [H, c_int, H]),
        "cb200_na_mask": (H, [H, H]),
        "cb200_na_count": (H, [H, c_uint32, c_int, c_int]),
        "cb200_na_bit_op": (H, [c_char_p, H, H]),
        "cb200_na_bit_reduce": (H, [c_char_p, H, c_uint32, c_int]),
        "cb200_na_mulsum": (H, [H, H, c_uint32, c_int, c_int]),
        "cb200_na_clip": (H, [H, c_int, H, c_double, c_int64, c_int, H, c_double, c_int64]),
        "cb200_na_fill": (c_int, [H, c_double, c_int64]),
        "cb200_na_seq": (c_int, [H, c_double, c_double]),
        "cb200_na_divmod": (c_int, [H, H, POINTER(H), POINTER(H)]),
        "cb200_na_modf": (c_int, [H, POINTER(H), POINTER(H)]),
        "cb200_na_frexp": (c_int, [H, POINTER(H), POINTER(H)]),
        "cb200_na_cast": (H, [H, c_int]),
        "cb200_na_copy": (H, [H]),
        "cb200_set_stream": (None, [c_void_p]),
        "cb200_get_stream": (c_void_p, []),
        "cb200_last_error": (c_int, [POINTER(c_char_p)]),
        "cb200_launch_count": (c_uint64, []),
        "cb200_pool_total_bytes": (c_size_t, []),
        "cb200_pool_used_bytes": (c_size_t, []),
        "cb200_pool_free_all_blocks": (None, []),
        "cb200_version": (c_char_p, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


def launch_count() -> int:
    return int(load().cb200_launch_count())
