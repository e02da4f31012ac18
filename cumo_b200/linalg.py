"""Matrix products: SFloat on the tensor cores, DFloat and the batched / transposed / alpha-beta forms through
`cb200_{s,d}gemm_strided_batched` (the argument list of the cuBLAS call in the reference's gemm.c:277-296).

`dot(a, b)` is the reference's `a.dot(b)` on float matrices (ext/cumo/narray/gen/tmpl/gemm.c:252-297 hands it to
cuBLAS).  `gemm_nt` calls `cb200_sgemm_nt_tc` directly: a tcgen05 kernel that keeps fp32-grade accuracy by splitting
every operand into two TF32 numbers and wants both operands with K contiguous.
"""
from __future__ import annotations

from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p, create_string_buffer

from . import _lib
from .narray import CumoError, DFloat, SFloat


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


def gemm(a, b, alpha=1.0, beta=0.0, c=None):
    """The reference's `Cumo::NArray#gemm` for SFloat / DFloat operands (row-major, the last two axes are the
    matrices, leading axes are batches; either operand may be a transposed view; an operand that holds one matrix is
    used for every batch of the other): alpha * a . b + beta * c.
    It hands cuBLAS's column-major bookkeeping to the library exactly as gemm.c does: c^T = b^T . a^T."""
    from ctypes import byref, c_double, c_float, c_longlong

    from .narray import ShapeError

    T = type(a)
    if T not in (SFloat, DFloat) or type(b) is not T or a.ndim < 2 or b.ndim < 2:
        raise TypeError("gemm needs two SFloat or two DFloat arrays of two or more dimensions")
    m, k = a.shape[-2:]
    k2, n = b.shape[-2:]
    if k != k2:
        raise ShapeError(f"shape mismatch: {a.shape} . {b.shape}")
    if 0 in (m, n, k):
        raise ShapeError("gemm of an empty operand")
    batch_a, batch_b = a.shape[:-2], b.shape[:-2]
    if batch_a and batch_b and batch_a != batch_b:
        raise ShapeError(f"batch dimensions differ: {batch_a} and {batch_b}")
    batch_shape = batch_a or batch_b                       # (gemm.c takes them from whichever operand has them)
    es = 4 if T is SFloat else 8

    def layout(x):
        """(array usable as it is or a contiguous copy, trans flag, leading dimension, batch stride in elements)"""
        st = x.steps
        rows, cols = x.shape[-2:]
        batch_ok = all(st[d] == (x.shape[d + 1] * st[d + 1] if d + 1 < x.ndim - 2 else rows * cols * es) for d in range(x.ndim - 2))
        stride = rows * cols if x.ndim > 2 else 0          # one matrix serves every batch
        if batch_ok and st[-1] == es and st[-2] >= cols * es and st[-2] % es == 0 and (x.ndim == 2 or st[-2] == cols * es):
            return x, 0, st[-2] // es, stride               # row-major: column-major of its transpose, no flag
        if batch_ok and st[-2] == es and st[-1] >= rows * es and st[-1] % es == 0 and (x.ndim == 2 or st[-1] == rows * es):
            return x, 1, st[-1] // es, stride               # a transposed view: flag T
        y = x.dup()
        return y, 0, cols, stride
    a2, ta, lda, sa = layout(a)
    b2, tb, ldb, sb = layout(b)
    batch = 1
    for d in batch_shape:
        batch *= d
    if c is not None and tuple(c.shape) != tuple(batch_shape) + (m, n):
        raise ShapeError(f"c has shape {c.shape}, the product {tuple(batch_shape) + (m, n)}")
    out = T(*batch_shape, m, n) if c is None or beta == 0.0 else c.dup()
    lib = _lib.load()
    fn = lib.cb200_sgemm_strided_batched if T is SFloat else lib.cb200_dgemm_strided_batched
    fn.restype = c_int
    fn.argtypes = None
    cT = c_float if T is SFloat else c_double
    rc = fn(c_int(tb), c_int(ta), c_int(n), c_int(m), c_int(k), byref(cT(alpha)), c_void_p(b2.data_ptr), c_int(ldb), c_longlong(sb),
            c_void_p(a2.data_ptr), c_int(lda), c_longlong(sa), byref(cT(beta)), c_void_p(out.data_ptr), c_int(n), c_longlong(m * n), c_int(batch))
    if rc:
        raise CumoError(f"gemm failed with status {rc}")
    return out


def dot(a, b):
    """a (M, K) . b (K, N) -> (M, N); a 1-D second operand gives (M,).  Both SFloat or both DFloat: the reference's
    `dot` on float matrices is `gemm` (lib/cumo/narray/extra.rb:1145-1196).  Large single-precision products run on the
    tensor cores, the rest on the CUDA-core kernel."""
    if not ((isinstance(a, SFloat) and isinstance(b, SFloat)) or (isinstance(a, DFloat) and isinstance(b, DFloat))):
        raise TypeError("dot is built for two SFloat or two DFloat operands (NArray#dot takes the other types)")
    return a.dot(b)
