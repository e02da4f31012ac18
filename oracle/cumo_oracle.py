"""TEST INFRASTRUCTURE -- numpy-facing wrapper of the CPU oracle (oracle/cumo_oracle.c).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this.
It restates nothing itself: arguments are turned into (pointer, shape, byte steps)
and handed to the C loops, which cite the reference lines they follow.  The
arrays may have any numpy strides; broadcasting follows ndloop's rule
(ext/cumo/narray/ndloop.c:494-516) via numpy's zero strides.
"""
from __future__ import annotations

import ctypes
import subprocess
from ctypes import POINTER, c_char_p, c_double, c_int, c_int32, c_int64, c_uint32, c_uint64, c_void_p
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "libcumo_oracle.so"

DT = {np.dtype(np.float32): 0, np.dtype(np.float64): 1, np.dtype(np.int32): 2, np.dtype(np.int64): 3}
KIND_BINARY, KIND_UNARY, KIND_COMPARE = 0, 1, 2

_BINARY = ["add", "sub", "mul", "div", "mod", "pow", "copysign", "atan2", "hypot", "ldexp", "maximum", "minimum",
           "maximum_nan", "minimum_nan", "bit_and", "bit_or", "bit_xor", "left_shift", "right_shift"]
_UNARY = ["minus", "reciprocal", "sign", "square", "abs", "floor", "round", "ceil", "trunc", "rint", "bit_not",
          "sqrt", "cbrt", "log", "log2", "log10", "exp", "exp2", "exp10", "sin", "cos", "tan", "asin", "acos", "atan",
          "sinh", "cosh", "tanh", "asinh", "acosh", "atanh", "sinc", "erf", "erfc", "log1p", "expm1"]
_COMPARE = ["eq", "ne", "gt", "ge", "lt", "le", "nearly_eq", "isnan", "isinf", "isposinf", "isneginf", "isfinite", "signbit"]
OPS = {n: i for i, n in enumerate(_BINARY)}
OPS.update({n: 100 + i for i, n in enumerate(_UNARY)})
OPS.update({n: 200 + i for i, n in enumerate(_COMPARE)})
RED = {n: i for i, n in enumerate(["sum", "prod", "mean", "min", "max", "ptp", "minmax", "min_index", "max_index",
                                   "argmin", "argmax", "var", "stddev", "rms", "kahan_sum"])}

_lib = None


def build() -> Path:
    """Compile the oracle with the Makefile beside it (gcc, no fast-math)."""
    if not LIB.exists() or any(p.stat().st_mtime > LIB.stat().st_mtime for p in (HERE / "cumo_oracle.c", HERE / "oracle_type.inc")):
        subprocess.run(["make", "-C", str(HERE)], check=True, capture_output=True)
    return LIB


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(LIB))
        P = POINTER(c_int64)
        L.oracle_elementwise.restype = c_int
        L.oracle_elementwise.argtypes = [c_int, c_int, c_int, c_int, P, c_void_p, P, c_void_p, P, c_void_p, P,
                                         c_double, c_int64, POINTER(c_int), c_void_p, c_uint64]
        L.oracle_pow_int32.restype = c_int
        L.oracle_pow_int32.argtypes = [c_int, c_int, P, c_void_p, P, c_void_p, P, c_void_p, P, c_double, c_int64, c_int32]
        L.oracle_multi.restype = c_int
        L.oracle_multi.argtypes = [c_int, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_double, c_double, c_double, POINTER(c_int)]
        L.oracle_reduce.restype = c_int
        L.oracle_reduce.argtypes = [c_int, c_int, c_int, c_int, P, P, P, P, c_int, P, P, c_void_p, c_void_p, c_void_p, c_int]
        L.oracle_mulsum.restype = c_int
        L.oracle_mulsum.argtypes = [c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64]
        L.oracle_bit_count.restype = c_uint64
        L.oracle_bit_count.argtypes = [c_void_p, c_uint64, c_int64, c_uint64, c_int]
        L.oracle_sum_f64ref.restype = c_double
        L.oracle_sum_f64ref.argtypes = [c_int, c_void_p, c_int64]
        L.oracle_threads.restype = c_int
        L.oracle_set_threads.argtypes = [c_int]
        _lib = L
    return _lib


def threads() -> int:
    return int(lib().oracle_threads())


def set_threads(n: int) -> None:
    lib().oracle_set_threads(int(n))


def _i64(values):
    return (c_int64 * max(1, len(values)))(*[int(v) for v in values])


def _scalar_args(value, dtype):
    if np.issubdtype(dtype, np.floating):
        return float(value), 0
    return 0.0, int(value)


def _is_array(x):
    return isinstance(x, np.ndarray)


def _elementwise(kind, op, a, b, out=None):
    """a, b: ndarrays (same dtype) or python scalars (at most one of them)."""
    arrs = [x for x in (a, b) if _is_array(x)]
    dtype = arrs[0].dtype
    shape = np.broadcast_shapes(*[x.shape for x in arrs])
    sv = next((x for x in (a, b) if x is not None and not _is_array(x)), 0)
    sv_f, sv_i = _scalar_args(sv, dtype)
    va = np.broadcast_to(a, shape) if _is_array(a) else None
    vb = np.broadcast_to(b, shape) if _is_array(b) else None
    flag = c_int(0)
    if kind == KIND_COMPARE:
        n = int(np.prod(shape, dtype=np.int64))
        words = np.zeros((n + 31) // 32, dtype=np.uint32)
        steps, s = [], 1
        for ext in reversed(shape):
            steps.append(s); s *= ext
        sc = _i64(list(reversed(steps)))
        rc = lib().oracle_elementwise(DT[dtype], kind, OPS[op], len(shape), _i64(shape),
                                      va.ctypes.data if va is not None else None, _i64(va.strides) if va is not None else _i64([]),
                                      vb.ctypes.data if vb is not None else None, _i64(vb.strides) if vb is not None else _i64([]),
                                      None, sc, sv_f, sv_i, ctypes.byref(flag), words.ctypes.data, 0)
        if rc:
            raise ValueError(f"oracle: {op} is not defined for {dtype}")
        bits = np.unpackbits(words.view(np.uint8), bitorder="little")[:n].astype(bool).reshape(shape)
        return bits, words
    if out is None:
        out = np.zeros(shape, dtype=dtype)
    rc = lib().oracle_elementwise(DT[dtype], kind, OPS[op], len(shape), _i64(shape),
                                  va.ctypes.data if va is not None else None, _i64(va.strides) if va is not None else _i64([]),
                                  vb.ctypes.data if vb is not None else None, _i64(vb.strides) if vb is not None else _i64([]),
                                  out.ctypes.data, _i64(out.strides), sv_f, sv_i, ctypes.byref(flag), None, 0)
    if rc:
        raise ValueError(f"oracle: {op} is not defined for {dtype}")
    return out, flag.value


def binary(op, a, b, out=None):
    """(result, flag): flag is 1 when an integer division by zero was met (those elements are left alone)."""
    return _elementwise(KIND_BINARY, op, a, b, out)


def unary(op, a, out=None):
    return _elementwise(KIND_UNARY, op, a, None, out)


def compare(op, a, b=None):
    """(bool array, packed uint32 words)."""
    return _elementwise(KIND_COMPARE, op, a, b)


def pow_int(a, exponent: int):
    out = np.zeros(a.shape, dtype=a.dtype)
    lib().oracle_pow_int32(DT[a.dtype], a.ndim, _i64(a.shape), a.ctypes.data, _i64(a.strides), None, _i64([]),
                           out.ctypes.data, _i64(out.strides), 0.0, 0, int(exponent))
    return out


def pow_int32(base, exponent):
    """x ** e with an Int32 exponent by repeated multiplication; either side may be an array (the exponent an int32
    array) or a host numeric: the array forms of gen/tmpl/pow_kernel.cu:22-32 and its `_s` / `_s_left` forms."""
    arr = base if _is_array(base) else None
    exp = np.ascontiguousarray(exponent, dtype=np.int32) if _is_array(exponent) else None
    like = arr if arr is not None else exp
    dtype = arr.dtype if arr is not None else np.dtype(type(base)) if isinstance(base, np.generic) else None
    if dtype is None:
        raise TypeError("a scalar base must be a numpy scalar of the element type")
    shape = like.shape
    out = np.zeros(shape, dtype=dtype)
    sv_f, sv_i = _scalar_args(base if arr is None else 0, dtype)
    lib().oracle_pow_int32(DT[np.dtype(dtype)], len(shape), _i64(shape), arr.ctypes.data if arr is not None else None,
                           _i64(arr.strides) if arr is not None else _i64([]), exp.ctypes.data if exp is not None else None,
                           _i64(exp.strides) if exp is not None else _i64([]), out.ctypes.data, _i64(out.strides), sv_f, sv_i,
                           0 if exp is not None else int(exponent))
    return out


MULTI = {"clip": 0, "clip_min": 1, "clip_max": 2, "divmod": 3, "modf": 4, "frexp": 5, "seq": 6}


def multi(op, inputs=(), shape=None, dtype=None, beg=0.0, step=0.0, count=0.0):
    """clip (x, lo, hi), clip_min (x, lo), clip_max (x, hi), divmod (x, y), modf (x), frexp (x): `inputs` are arrays
    of one element type, repeated here to their common shape; seq takes `shape` and `dtype` instead.  Answers
    (out0, out1 or None, flag): the flag is 1 when clip met lo > hi or an integer divmod met a zero divisor, and
    those elements of the outputs are left as zero."""
    if op == "seq":
        shape, dtype = tuple(shape), np.dtype(dtype)
        ins = []
    else:
        shape = np.broadcast_shapes(*[x.shape for x in inputs])
        dtype = inputs[0].dtype
        ins = [np.ascontiguousarray(np.broadcast_to(x, shape)) for x in inputs]
    n = int(np.prod(shape, dtype=np.int64))
    o0 = np.zeros(shape, dtype=dtype)
    o1 = None
    if op in ("divmod", "modf"):
        o1 = np.zeros(shape, dtype=dtype)
    elif op == "frexp":
        o1 = np.zeros(shape, dtype=np.int32)
    ptr = [x.ctypes.data for x in ins] + [None] * (3 - len(ins))
    flag = c_int(0)
    rc = lib().oracle_multi(DT[dtype], MULTI[op], n, ptr[0], ptr[1], ptr[2], o0.ctypes.data,
                            o1.ctypes.data if o1 is not None else None, float(beg), float(step), float(count), ctypes.byref(flag))
    if rc:
        raise ValueError(f"oracle: {op} is not defined for {dtype}")
    return o0, o1, flag.value


def reduce(op, a, axis=None, nan=False, keepdims=False, idx64=None):
    """Reduction of `a` (any strides) over `axis` (None: all).  For max_index/min_index the
    answer is the element offset from a's first element in units of elements, which for a
    C-contiguous `a` is the flat index, as in the reference."""
    nd = a.ndim
    axes = tuple(range(nd)) if axis is None else ((axis,) if isinstance(axis, int) else tuple(axis))
    axes = tuple(sorted(ax % nd for ax in axes)) if nd else ()
    keep = [d for d in range(nd) if d not in axes]
    out_shape = [a.shape[d] for d in keep]
    index_op = op in ("max_index", "min_index", "argmax", "argmin")
    if idx64 is None:
        idx64 = a.size > 0xFFFFFFFF
    if index_op:
        out_dtype = np.int64 if idx64 else np.int32
    elif op in ("sum", "prod") and np.issubdtype(a.dtype, np.integer):
        out_dtype = np.int64
    else:
        out_dtype = a.dtype
    out = np.zeros(out_shape, dtype=out_dtype)
    out2 = np.zeros(out_shape, dtype=out_dtype) if op == "minmax" else None
    lib().oracle_reduce(DT[a.dtype], RED[op], int(nan), len(keep), _i64(out_shape), _i64([a.strides[d] for d in keep]),
                        _i64(out.strides), _i64(out2.strides) if out2 is not None else None,
                        len(axes), _i64([a.shape[d] for d in axes]), _i64([a.strides[d] for d in axes]),
                        a.ctypes.data, out.ctypes.data, out2.ctypes.data if out2 is not None else None, int(bool(idx64)))
    if keepdims:
        ks = [1 if d in axes else a.shape[d] for d in range(nd)]
        out = out.reshape(ks)
        if out2 is not None:
            out2 = out2.reshape(ks)
    return (out, out2) if op == "minmax" else out


def mulsum(a, b, axis=None, nan=False):
    """(a*b) summed over `axis`, accumulated the way the host loop does: one output at a time, z = x*y + z."""
    shape = np.broadcast_shapes(a.shape, b.shape)
    va, vb = np.broadcast_to(a, shape), np.broadcast_to(b, shape)
    nd = len(shape)
    axes = tuple(range(nd)) if axis is None else ((axis,) if isinstance(axis, int) else tuple(axis))
    axes = tuple(sorted(ax % nd for ax in axes))
    keep = [d for d in range(nd) if d not in axes]
    out = np.zeros([shape[d] for d in keep], dtype=a.dtype)
    red_shape = [shape[d] for d in axes]
    for oi in np.ndindex(*out.shape):
        for ri in np.ndindex(*red_shape):
            idx = [0] * nd
            for d, i in zip(keep, oi):
                idx[d] = i
            for d, i in zip(axes, ri):
                idx[d] = i
            pa = va.ctypes.data + sum(i * s for i, s in zip(idx, va.strides))
            pb = vb.ctypes.data + sum(i * s for i, s in zip(idx, vb.strides))
            po = out.ctypes.data + sum(i * s for i, s in zip(oi, out.strides))
            lib().oracle_mulsum(DT[a.dtype], int(nan), pa, pb, po, 0, 0, 0, 1)
    return out


def mulsum_1d(a, b, nan=False):
    """Full mulsum of two 1-D arrays in one C loop."""
    out = np.zeros((), dtype=a.dtype)
    lib().oracle_mulsum(DT[a.dtype], int(nan), a.ctypes.data, b.ctypes.data, out.ctypes.data, a.strides[0], b.strides[0], 0, a.size)
    return out


def bit_count(words: np.ndarray, pos: int, step: int, n: int, want_false: bool = False) -> int:
    return int(lib().oracle_bit_count(words.ctypes.data, pos, step, n, int(want_false)))


def sum_f64ref(a: np.ndarray) -> float:
    """Pairwise float64 sum of a contiguous float array: the yardstick of the stated tolerances."""
    a = np.ascontiguousarray(a)
    return float(lib().oracle_sum_f64ref(DT[a.dtype], a.ctypes.data, a.size))


def gemm_nt_f64(a: np.ndarray, bt: np.ndarray):
    """(a . bt^T in float64, sum of |a||b| per element) for float32 a (M, K) and bt (N, K)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bt = np.ascontiguousarray(bt, dtype=np.float32)
    m, k = a.shape
    n = bt.shape[0]
    c = np.empty((m, n), dtype=np.float64)
    cabs = np.empty((m, n), dtype=np.float64)
    fn = lib().oracle_gemm_nt_f64
    fn.restype = None
    fn.argtypes = [c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]
    fn(m, n, k, a.ctypes.data, bt.ctypes.data, c.ctypes.data, cabs.ctypes.data)
    return c, cabs


def where(bits: np.ndarray, invert: bool = False) -> np.ndarray:
    """Row-major positions of the one (invert: zero) elements of a boolean array: int32, int64 beyond 2^32-1 elements."""
    flat = np.ascontiguousarray(bits, dtype=bool).reshape(-1).view(np.uint8)
    out = np.empty(flat.size, dtype=np.int64)
    fn = lib().oracle_where
    fn.restype = c_int64
    fn.argtypes = [c_void_p, c_int64, c_int, c_void_p]
    hits = fn(flat.ctypes.data, flat.size, int(invert), out.ctypes.data)
    return out[:hits].astype(np.int64 if flat.size > 4294967295 else np.int32)


def cum(op: str, a: np.ndarray, axis=None, nan: bool = False) -> np.ndarray:
    """cumsum / cumprod: over all elements in row-major order (axis None) or along one axis."""
    fn = lib().oracle_cum
    fn.restype = c_int
    fn.argtypes = [c_int, c_int, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64]
    out = np.empty(a.shape, dtype=a.dtype)
    if a.size == 0:
        return out
    prod = int(op == "cumprod")
    if axis is None:
        src = np.ascontiguousarray(a).reshape(-1)
        dst = out.reshape(-1)
        fn(DT[a.dtype], prod, int(nan), src.ctypes.data, dst.ctypes.data, src.strides[0], dst.strides[0], src.size)
        return out
    src, dst = np.moveaxis(a, axis, -1), np.moveaxis(out, axis, -1)
    for lead in np.ndindex(*src.shape[:-1]):
        r, w = src[lead], dst[lead]
        fn(DT[a.dtype], prod, int(nan), r.ctypes.data, w.ctypes.data, r.strides[0], w.strides[0], r.shape[0])
    return out


def bincount(a: np.ndarray, weight=None, minlength: int = 0) -> np.ndarray:
    """Cumo's bincount along the last axis (narray/gen/tmpl/bincount.c:176-240): length = max+1 or minlength,
    UInt32 counts (UInt64 beyond 2^32-1 bins), float32 weights summed as float32, any other weight as float64;
    a negative item raises ValueError (the reference's ArgumentError)."""
    if a.dtype not in (np.int32, np.int64) or a.ndim < 1:
        raise TypeError("bincount needs an Int32 / Int64 array of at least one dimension")
    if weight is not None:
        weight = np.asarray(weight)
        if weight.dtype != np.float32:
            weight = weight.astype(np.float64)
        if weight.shape[-1:] != a.shape[-1:]:
            raise ValueError("size mismatch along last axis between self and weight")
        weight = np.broadcast_to(weight, a.shape)
    length = 0
    if a.size:
        if int(a.min()) < 0:
            raise ValueError("array items must be non-negative")
        length = int(a.max()) + 1
    length = max(length, int(minlength))
    if weight is None:
        kind, odt = (1, np.uint64) if length > 4294967295 else (0, np.uint32)
    else:
        kind, odt = (2, np.float32) if weight.dtype == np.float32 else (3, np.float64)
    out = np.zeros(a.shape[:-1] + (length,), dtype=odt)
    fn = lib().oracle_bincount
    fn.restype = c_int
    fn.argtypes = [c_int, c_void_p, c_int64, c_int64, c_int, c_void_p, c_int64, c_void_p, c_int64, c_int64, POINTER(c_int64)]
    bad = c_int64(0)
    for lead in np.ndindex(*a.shape[:-1]):
        row = a[lead]
        w = weight[lead] if weight is not None else None
        o = out[lead]
        if fn(int(a.dtype == np.int64), row.ctypes.data, row.strides[0] if row.ndim else 0, row.shape[0], kind,
              w.ctypes.data if w is not None else None, (w.strides[0] if w is not None else 0), o.ctypes.data, o.strides[0] if length else 0,
              length, bad):
            raise IndexError(f"item {bad.value} is out of range of the output(size:{length})")
    return out


def kmeans_assign(x: np.ndarray, c: np.ndarray):
    """(labels int32, best float64, second float64) of the assignment step in float64."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    c = np.ascontiguousarray(c, dtype=np.float32)
    n, d = x.shape
    k = c.shape[0]
    labels = np.empty(n, dtype=np.int32)
    best = np.empty(n, dtype=np.float64)
    second = np.empty(n, dtype=np.float64)
    fn = lib().oracle_kmeans_assign
    fn.restype = None
    fn.argtypes = [c_void_p, c_int64, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p]
    fn(x.ctypes.data, n, d, c.ctypes.data, k, labels.ctypes.data, best.ctypes.data, second.ctypes.data)
    return labels, best, second
