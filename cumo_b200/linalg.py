"""Matrix products of SFloat arrays on the tensor cores.

`dot(a, b)` is the reference's `a.dot(b)` for 2-D single-precision operands (ext/cumo/narray/gen/tmpl/gemm.c:252-297
hands it to cublasSgemm); here it runs `cb200_sgemm_nt_tc`, a tcgen05 kernel that keeps fp32-grade accuracy by
splitting every operand into two TF32 numbers.  The kernel wants the second operand with K contiguous
(`bt[n, k]`): `dot` makes that copy with the library's own strided-copy kernel, `gemm_nt` takes it as given.
"""
from __future__ import annotations

from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p, create_string_buffer

from . import _lib
from .narray import CumoError, SFloat


def gemm_nt(a: SFloat, bt: SFloat) -> SFloat:
    """a (M, K) . bt (N, K)^T -> (M, N).  Rows must be contiguous (the row steps may be larger than K)."""
    if not (isinstance(a, SFloat) and isinstance(bt, SFloat) and a.ndim == 2 and bt.ndim == 2 and a.shape[1] == bt.shape[1]):
        raise TypeError("gemm_nt needs SFloat a (M, K) and bt (N, K)")
    if not a.contiguous():
        a = a.dup()
    if not bt.contiguous():
        bt = bt.dup()
    m, k = a.shape
    n = bt.shape[0]
    out = SFloat(m, n)
    fn = _lib.load().cb200_sgemm_nt_tc
    fn.restype = c_int
    fn.argtypes = [c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_char_p, c_size_t]
    err = create_string_buffer(256)
    if fn(m, n, k, a.data_ptr, k, bt.data_ptr, k, out.data_ptr, n, err, len(err)):
        raise CumoError(err.value.decode())
    return out


def dot(a: SFloat, b: SFloat) -> SFloat:
    """a (M, K) . b (K, N) -> (M, N); a 1-D second operand gives (M,)."""
    if not (isinstance(a, SFloat) and isinstance(b, SFloat)):
        raise TypeError("the tensor-core product is built for SFloat operands")
    if a.ndim == 2 and b.ndim == 2:
        return gemm_nt(a, b.transpose().dup())
    if a.ndim == 2 and b.ndim == 1:
        return gemm_nt(a, b.reshape(1, b.shape[0])).reshape(a.shape[0])
    raise TypeError("dot takes a 2-D first operand and a 1-D or 2-D second one")
