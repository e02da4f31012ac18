"""cumo_b200 -- the data-parallel core of Cumo::NArray on B200 (sm_100a).

The product is `libcumo_b200.so` (hand-written CUDA kernels behind the reference's
`cumo_..._kernel_launch` C ABI, see `include/cumo_b200.h`).  This package holds its
sources (`csrc/`), its build (`build.py`), a ctypes binding, the Python face of the
host layer (`narray`), and leading-axis sharding over several GPUs (`sharded`).
"""
from .narray import (Bit, CudaError, CumoError, DFloat, Int32, Int64, NArray, NMath, OperationError, SFloat, ShapeError,
                     UInt32, UInt64, pack_bits, synchronize, unpack_bits)

__all__ = ["Bit", "CudaError", "CumoError", "DFloat", "Int32", "Int64", "NArray", "NMath", "OperationError", "SFloat",
           "ShapeError", "UInt32", "UInt64", "pack_bits", "synchronize", "unpack_bits"]
