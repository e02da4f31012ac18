"""TEST INFRASTRUCTURE -- the CPU oracle dressed in the same method names as
cumo_b200.narray, so one test body can run against either: `xp.SFloat[[1, 2], [3, 4]].sum(axis=0)`.

Arrays are numpy arrays (views keep their strides); every computation goes to
oracle/cumo_oracle.py, none is done with numpy arithmetic.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from oracle import cumo_oracle as orc  # noqa: E402


def _axes(axis):
    return axis


class ONArray:
    np_dtype = None

    def __init__(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        self.a = np.zeros(shape, dtype=self.np_dtype)

    new = classmethod(lambda cls, *shape: cls(*shape))

    @classmethod
    def _wrap(cls, a):
        klass = _BY_DTYPE[np.dtype(a.dtype)]
        o = object.__new__(klass)
        o.a = a
        return o

    def __class_getitem__(cls, item):
        data = list(item) if isinstance(item, tuple) else [item]
        return cls.cast(data)

    @classmethod
    def cast(cls, data):
        if isinstance(data, ONArray):
            return cls._wrap(data.a.astype(cls.np_dtype))
        if isinstance(data, OBit):                              # 0 or 1 in the element type (gen/tmpl/store_bit.c:14-27)
            return cls._wrap(data.b.astype(cls.np_dtype))
        return cls._wrap(np.array(data, dtype=cls.np_dtype))

    from_numpy = cast

    @classmethod
    def zeros(cls, *shape):
        return cls(*shape)

    @classmethod
    def ones(cls, *shape):
        return cls(*shape).fill(1)

    def fill(self, v):
        self.a[...] = v
        return self

    def seq(self, start=0, step=1):
        vals, _, _ = orc.multi("seq", shape=self.a.shape, dtype=self.a.dtype, beg=start, step=step)
        self.a[...] = vals
        return self

    def _bound(self, b):
        """A clip bound as an array of this type: numerics convert the way NUM2INT / NUM2DBL do (truncation)."""
        if isinstance(b, ONArray):
            return b.a.astype(self.a.dtype) if b.a.dtype != self.a.dtype else b.a
        if isinstance(b, (list, tuple, np.ndarray)):
            return np.array(b, dtype=self.a.dtype)
        if np.issubdtype(self.a.dtype, np.integer):
            return np.array(int(b), dtype=self.a.dtype)
        return np.array(b, dtype=self.a.dtype)

    def clip(self, min=None, max=None):
        if min is None and max is None:
            raise ValueError("min and max are not given")
        if min is not None and max is not None:
            res, _, flag = orc.multi("clip", [self.a, self._bound(min), self._bound(max)])
            if flag:
                raise OperationErrorO("min is greater than max")
        elif min is not None:
            res, _, _ = orc.multi("clip_min", [self.a, self._bound(min)])
        else:
            res, _, _ = orc.multi("clip_max", [self.a, self._bound(max)])
        if getattr(self, "_inplace", False) and res.shape == self.a.shape:
            self._inplace = False
            self.a[...] = res
            return self
        return self._wrap(res)

    def poly(self, *coefs):
        """Horner's rule with the oracle's own multiply and add (gen/tmpl/poly_kernel.cu:9-16)."""
        if not coefs:
            return self._wrap(np.array(self.a))
        cs = [np.broadcast_to(self._bound(c), self.a.shape) for c in coefs]
        y = np.ascontiguousarray(cs[-1])
        for c in reversed(cs[:-1]):
            y, _ = orc.binary("mul", self.a, y)
            y, _ = orc.binary("add", y, np.ascontiguousarray(c))
        return self._wrap(y)

    def eye(self, element=1, offset=0):
        if self.a.ndim < 2:
            raise ShapeErrorO("less than 2-d array")
        n0, n1 = self.a.shape[-2:]
        if (offset >= 0 and offset >= n1) or (offset < 0 and -offset >= n0):
            raise ValueError("invalid diagonal offset")
        rows, cols = np.indices((n0, n1))
        self.a[...] = np.where(rows + offset == cols, np.array(element, dtype=self.a.dtype), np.array(0, dtype=self.a.dtype))
        return self

    def divmod(self, o):
        x, y = self._operand(o)
        if not isinstance(y, np.ndarray):
            y = np.array(y, dtype=x.dtype)
        q, r, flag = orc.multi("divmod", [x, y])
        if flag:
            raise ZeroDivisionError("divided by 0")
        return self._wrap(q), self._wrap(r)

    __divmod__ = divmod

    def modf(self):
        if not np.issubdtype(self.a.dtype, np.floating):
            raise AttributeError("modf needs a float array")
        f, w, _ = orc.multi("modf", [self.a])
        return self._wrap(f), self._wrap(w)

    # facts / host copies
    shape = property(lambda self: tuple(self.a.shape))
    ndim = property(lambda self: self.a.ndim)
    size = property(lambda self: int(self.a.size))

    def to_numpy(self):
        return np.array(self.a)

    def to_a(self):
        return self.a.tolist()

    def extract(self):
        return self.a.reshape(()).item()

    __float__ = lambda self: float(self.extract())
    __int__ = lambda self: int(self.extract())

    # views
    def __getitem__(self, key):
        if isinstance(key, OBit):
            return key.mask(self)
        if not isinstance(key, tuple):
            key = (key,)
        key = tuple(slice(None) if k is True else k for k in key)
        return self._wrap(self.a[key])

    def store(self, other):
        """self[...] = other, converted to this type and repeated along missing or unit dimensions (a copy loop, no arithmetic)."""
        src = other.a if isinstance(other, ONArray) else np.array(other if isinstance(other, (list, tuple, np.ndarray)) else [other])
        if src.size == 1:
            src = src.reshape(())
        self.a[...] = np.broadcast_to(src.astype(self.np_dtype), self.a.shape)
        return self

    def __setitem__(self, key, value):
        if not isinstance(key, tuple):
            key = (key,)
        key = tuple(slice(None) if k is True else k for k in key)
        src = value.a if isinstance(value, ONArray) else np.array(value)
        self.a[key] = src.reshape(()) if src.size == 1 else src          # numpy repeats it; the assignment converts

    def transpose(self, *perm):
        return self._wrap(self.a.transpose(*perm) if perm else self.a.T)

    def reverse(self, axis=None):
        return self._wrap(np.flip(self.a, axis))

    def reshape(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        return self._wrap(np.array(self.a).reshape(shape))

    def flatten(self):
        return self.reshape(self.a.size)

    def dup(self):
        return self._wrap(np.array(self.a))

    copy = dup

    def contiguous(self):
        return bool(self.a.flags["C_CONTIGUOUS"])

    def inplace(self):
        self._inplace = True
        return self

    # elementwise
    def _operand(self, o):
        """(array_self, other) with the reference's casting: arrays upcast, a Python float
        against an integer array upcasts the array to DFloat."""
        a = self.a
        if isinstance(o, ONArray):
            t = _upcast(a.dtype, o.a.dtype)
            return a.astype(t) if a.dtype != t else a, o.a.astype(t) if o.a.dtype != t else o.a
        if isinstance(o, (list, tuple, np.ndarray)):
            return a, np.array(o, dtype=a.dtype)
        if isinstance(o, (float, np.floating)) and np.issubdtype(a.dtype, np.integer):
            a = a.astype(np.float64)
        return a, o

    def _binary(self, op, o, reflected=False):
        x, y = self._operand(o)
        if reflected:
            x, y = y, x
        out = None
        if getattr(self, "_inplace", False) and isinstance(x, np.ndarray) and x is self.a:
            self._inplace = False
            out = self.a
        res, flag = orc.binary(op, x, y, out)
        if flag:
            raise ZeroDivisionError("divided by 0")
        return self._wrap(res)

    __add__ = lambda s, o: s._binary("add", o)
    __radd__ = lambda s, o: s._binary("add", o, True)
    __sub__ = lambda s, o: s._binary("sub", o)
    __rsub__ = lambda s, o: s._binary("sub", o, True)
    __mul__ = lambda s, o: s._binary("mul", o)
    __rmul__ = lambda s, o: s._binary("mul", o, True)
    __truediv__ = lambda s, o: s._binary("div", o)
    __rtruediv__ = lambda s, o: s._binary("div", o, True)
    __mod__ = lambda s, o: s._binary("mod", o)
    __rmod__ = lambda s, o: s._binary("mod", o, True)
    __and__ = lambda s, o: s._binary("bit_and", o)
    __or__ = lambda s, o: s._binary("bit_or", o)
    __xor__ = lambda s, o: s._binary("bit_xor", o)
    __lshift__ = lambda s, o: s._binary("left_shift", o)
    __rshift__ = lambda s, o: s._binary("right_shift", o)

    def __pow__(self, o):
        if isinstance(o, (int, np.integer)) and not isinstance(o, bool):
            return self._wrap(orc.pow_int(self.a, int(o)))
        return self._binary("pow", o)

    __rpow__ = lambda s, o: s._binary("pow", o, True)
    copysign = lambda s, o: s._binary("copysign", o)

    @classmethod
    def maximum(cls, a, b, nan=False):
        return cls.cast(a)._binary("maximum_nan" if nan else "maximum", cls.cast(b))

    @classmethod
    def minimum(cls, a, b, nan=False):
        return cls.cast(a)._binary("minimum_nan" if nan else "minimum", cls.cast(b))

    def _unary(self, op):
        if np.issubdtype(self.a.dtype, np.integer) and op in ("floor", "round", "ceil", "trunc", "rint"):
            return self._wrap(self.a)
        res, flag = orc.unary(op, self.a)
        if flag:
            if op == "abs":
                raise ValueError("cannot convert the minimum integer")
            raise ZeroDivisionError("divided by 0")
        return self._wrap(res)

    __neg__ = lambda s: s._unary("minus")
    __abs__ = lambda s: s._unary("abs")
    __invert__ = lambda s: s._unary("bit_not")
    for _n in ("abs", "minus", "reciprocal", "sign", "square", "floor", "round", "ceil", "trunc", "rint"):
        locals()[_n] = (lambda n: lambda s: s._unary(n))(_n)
    del _n

    def _compare(self, op, o, reflected=False):
        x, y = self._operand(o)
        if reflected:
            x, y = y, x
        if op == "nearly_eq" and np.issubdtype((x if isinstance(x, np.ndarray) else y).dtype, np.integer):
            op = "eq"
        bits, _ = orc.compare(op, x, y)
        return OBit._wrap_bits(bits)

    for _n in ("eq", "ne", "gt", "ge", "lt", "le", "nearly_eq"):
        locals()[_n] = (lambda n: lambda s, o: s._compare(n, o))(_n)
    del _n
    __gt__ = lambda s, o: s._compare("gt", o)
    __ge__ = lambda s, o: s._compare("ge", o)
    __lt__ = lambda s, o: s._compare("lt", o)
    __le__ = lambda s, o: s._compare("le", o)
    for _n in ("isnan", "isinf", "isposinf", "isneginf", "isfinite", "signbit"):
        locals()[_n] = (lambda n: lambda s: OBit._wrap_bits(orc.compare(n, s.a)[0]))(_n)
    del _n

    # reductions
    def _reduce(self, op, axis=None, keepdims=False, nan=False):
        if self.a.size == 0 and op != "sum":
            raise ShapeErrorO("cannot reduce an empty array")
        a = self.a
        if op in ("max_index", "min_index") and not a.flags["C_CONTIGUOUS"]:
            a = np.ascontiguousarray(a)        # accum_index.c:121-129 copies a non-contiguous operand
        return self._wrap(orc.reduce(op, a, axis=axis, nan=nan, keepdims=keepdims))

    for _n in ("sum", "prod", "mean", "var", "stddev", "rms", "kahan_sum", "min", "max", "ptp"):
        locals()[_n] = (lambda n: lambda s, axis=None, keepdims=False, nan=False: s._reduce(n, axis, keepdims, nan))(_n)
    for _n in ("max_index", "min_index", "argmax", "argmin"):
        locals()[_n] = (lambda n: lambda s, axis=None, nan=False: s._reduce(n, axis, False, nan))(_n)
    del _n

    def minmax(self, axis=None, keepdims=False, nan=False):
        lo, hi = orc.reduce("minmax", self.a, axis=axis, nan=nan, keepdims=keepdims)
        return self._wrap(lo), self._wrap(hi)

    def cumsum(self, axis=None, nan=False): return self._wrap(orc.cum("cumsum", self.a, axis, nan))
    def cumprod(self, axis=None, nan=False): return self._wrap(orc.cum("cumprod", self.a, axis, nan))

    def bincount(self, weight=None, minlength=0):
        w = weight.a if isinstance(weight, ONArray) else weight
        return self._wrap(orc.bincount(self.a, w, minlength))

    def arg_with_value(self, op, axis=None, nan=False):
        """(index as Int64, value): the index reduction and the matching extreme, two oracle calls."""
        idx = OracleXP.Int64.cast(self._reduce(op, axis, False, nan))
        val = self._reduce("max" if "max" in op else "min", axis, False, nan)
        return idx, val

    def gemm(self, b, c=None, alpha=1, beta=0):
        """alpha * a . b + beta * c over the last two axes, spelled with the oracle's mulsum (one output at a time)."""
        if not isinstance(b, ONArray) or type(b) is not type(self):
            b = type(self).cast(b)
        m, k = self.a.shape[-2:]
        k2, n = b.a.shape[-2:]
        ba, bb = self.a.shape[:-2], b.a.shape[:-2]
        if k != k2 or 0 in (m, n, k) or (ba and bb and ba != bb):
            raise ShapeErrorO(f"gemm of {self.a.shape} and {b.a.shape}")
        prod = self._wrap(orc.mulsum(self.a[..., :, :, None], b.a[..., None, :, :], axis=-2))
        if alpha != 1:
            prod = prod * type(self).cast([alpha]).a.reshape(()).item()
        if c is not None:
            if tuple(c.a.shape) != tuple(prod.a.shape):
                raise ShapeErrorO("c has another shape than the product")
            if beta != 0:
                prod = prod + c * beta
        return prod

    def dot(self, b):
        """lib/cumo/narray/extra.rb:1145-1196 on the oracle's operations."""
        if not isinstance(b, ONArray):
            b = type(self).cast(b)
        t = _upcast(self.a.dtype, b.a.dtype)
        T = _BY_DTYPE[np.dtype(t)]
        if self.a.ndim == 0 and b.a.ndim == 0:
            return self * b
        a, b = T.cast(self) if type(self) is not T else self, T.cast(b) if type(b) is not T else b
        if np.issubdtype(t, np.floating):
            if a.a.ndim == 1:
                if b.a.ndim == 1:
                    return a.mulsum(b, axis=-1)
                return a[None, ...].gemm(b).flatten()
            if b.a.ndim == 1:
                return a.gemm(b[..., None]).flatten()
            return a.gemm(b)
        if b.a.ndim == 1:
            return a.mulsum(b, axis=-1)
        if a.a.ndim == 0:
            return b.mulsum(a, axis=-2)
        if a.a.ndim == 1:
            return a[True, None].mulsum(b, axis=-2)
        return a[..., None].mulsum(b[..., None, True, True], axis=-2)

    def mulsum(self, other, axis=None, keepdims=False, nan=False):
        x, y = self._operand(other)
        try:
            np.broadcast_shapes(x.shape, np.shape(y))
        except ValueError as e:
            raise ShapeErrorO(str(e)) from None
        return self._wrap(orc.mulsum(x, y, axis=axis, nan=nan))


class OperationErrorO(Exception):
    pass


class ShapeErrorO(Exception):
    pass


class OSFloat(ONArray):
    np_dtype = np.float32


class ODFloat(ONArray):
    np_dtype = np.float64


class OInt32(ONArray):
    np_dtype = np.int32


class OInt64(ONArray):
    np_dtype = np.int64


class OUInt64(ONArray):
    np_dtype = np.uint64


class OUInt32(ONArray):
    np_dtype = np.uint32


class OBit:
    """Bits kept unpacked for views, packed on demand for the counting loop."""

    def __init__(self, bits):
        self.b = np.asarray(bits, dtype=bool)

    _wrap_bits = classmethod(lambda cls, bits: cls(bits))

    def __class_getitem__(cls, item):
        data = list(item) if isinstance(item, tuple) else [item]
        return cls(np.array(data).astype(bool))

    @classmethod
    def cast(cls, data):
        """A bit is set where the value is not zero (types/bit.h:12-18), so a NaN sets it."""
        if isinstance(data, ONArray):
            return cls(data.a != 0)
        if isinstance(data, OBit):
            return cls(np.array(data.b))
        return cls(np.array(data) != 0)

    from_numpy = cast
    new = classmethod(lambda cls, *shape: cls(np.zeros(shape, dtype=bool)))
    zeros = new

    def fill(self, v):
        self.b[...] = bool(int(v) & 1)
        return self

    def transpose(self, *perm):
        return OBit._view_of(self.b.transpose(*perm) if perm else self.b.T)

    @classmethod
    def _view_of(cls, bits):
        o = object.__new__(cls)
        o.b = bits                                              # a numpy view: writes go through to the parent
        return o
    shape = property(lambda self: tuple(self.b.shape))
    ndim = property(lambda self: self.b.ndim)
    size = property(lambda self: int(self.b.size))

    def to_numpy(self):
        return np.array(self.b)

    def to_a(self):
        return self.b.astype(np.int64).tolist()

    def where(self):
        return ONArray._wrap(orc.where(self.b))

    def where2(self):
        return ONArray._wrap(orc.where(self.b)), ONArray._wrap(orc.where(self.b, invert=True))

    def mask(self, array):
        """gen/tmpl_bit/mask.c:45-81 (the host loop): the masked array's elements at the one bits, row-major."""
        return ONArray._wrap(np.array(array.a)[self.b])

    def __getitem__(self, key):
        if not isinstance(key, tuple):
            key = (key,)
        return OBit(self.b[tuple(slice(None) if k is True else k for k in key)])

    def reshape(self, *shape):
        return OBit(np.array(self.b).reshape(shape))

    def _count(self, axis, keepdims, want_false):
        nd = self.b.ndim
        axes = tuple(range(nd)) if axis is None else ((axis,) if isinstance(axis, int) else tuple(axis))
        axes = tuple(ax % nd for ax in axes)
        keep = [d for d in range(nd) if d not in axes]
        moved = np.ascontiguousarray(self.b.transpose(keep + list(axes)))
        n_red = int(np.prod([self.b.shape[d] for d in axes], dtype=np.int64)) if axes else 1
        flat = moved.reshape(-1)
        pad = (-flat.size) % 32
        words = np.packbits(np.concatenate([flat, np.zeros(pad, bool)]), bitorder="little").view(np.uint32)
        n_out = flat.size // n_red if n_red else 0
        out = np.array([orc.bit_count(words, o * n_red, 1, n_red, want_false) for o in range(n_out)], dtype=np.uint64)
        out = out.reshape([self.b.shape[d] for d in keep])
        if keepdims:
            out = out.reshape([1 if d in axes else self.b.shape[d] for d in range(nd)])
        return OUInt64._wrap(out)

    def count_true(self, axis=None, keepdims=False):
        return self._count(axis, keepdims, False)

    def count_false(self, axis=None, keepdims=False):
        return self._count(axis, keepdims, True)

    count = count_1 = count_true
    count_0 = count_false

    # Bit o Bit and all? / any? / none?, spelled with the host loops' meaning (one bit at a time: numpy's boolean operators)
    def _other(self, o):
        return o.b if isinstance(o, OBit) else np.array(o).astype(bool)

    __and__ = lambda s, o: OBit(np.logical_and(s.b, s._other(o)))
    __or__ = lambda s, o: OBit(np.logical_or(s.b, s._other(o)))
    __xor__ = lambda s, o: OBit(np.logical_xor(s.b, s._other(o)))
    __rand__, __ror__, __rxor__ = __and__, __or__, __xor__
    __invert__ = lambda s: OBit(np.logical_not(s.b))
    eq = lambda s, o: OBit(np.logical_not(np.logical_xor(s.b, s._other(o))))
    dup = copy = lambda s: OBit(np.array(s.b))

    def _reduce(self, f, axis, keepdims):
        if self.b.size == 0:
            return False
        if axis is None and not keepdims:
            return bool(f(self.b))
        ax = axis if axis is None or isinstance(axis, int) else tuple(axis)
        return OBit(f(self.b, axis=ax, keepdims=keepdims))

    def all(self, axis=None, keepdims=False): return self._reduce(np.all, axis, keepdims)
    def any(self, axis=None, keepdims=False): return self._reduce(np.any, axis, keepdims)

    def none(self, axis=None, keepdims=False):
        r = self.any(axis=axis, keepdims=keepdims)
        return (not r) if isinstance(r, bool) else ~r


_BY_DTYPE = {np.dtype(np.float32): OSFloat, np.dtype(np.float64): ODFloat, np.dtype(np.int32): OInt32,
             np.dtype(np.int64): OInt64, np.dtype(np.uint64): OUInt64, np.dtype(np.uint32): OUInt32}


def _upcast(ta, tb):
    """gen/def/{sfloat,dfloat,int32,int64}.rb: any float beats any integer; wider wins within a kind."""
    ta, tb = np.dtype(ta), np.dtype(tb)
    if ta == tb:
        return ta
    if np.float64 in (ta, tb):
        return np.dtype(np.float64)
    if np.float32 in (ta, tb):
        return np.dtype(np.float32)
    return np.dtype(np.int64)


class _ONMath:
    _one = ("sqrt cbrt log log2 log10 exp exp2 exp10 sin cos tan asin acos atan sinh cosh tanh "
            "asinh acosh atanh sinc erf erfc log1p expm1").split()

    def __getattr__(self, name):
        if name in self._one:
            def f(x):
                if np.issubdtype(x.a.dtype, np.integer):
                    x = ODFloat.cast(x)
                return x._unary(name)
            return f
        if name in ("atan2", "hypot", "ldexp"):
            return lambda x, y: x._binary(name, y) if isinstance(x, ONArray) else y._binary(name, x, True)
        raise AttributeError(name)

    def frexp(self, x):
        if np.issubdtype(x.a.dtype, np.integer):
            x = ODFloat.cast(x)
        m, e, _ = orc.multi("frexp", [x.a])
        return ONArray._wrap(m), ONArray._wrap(e)


class OracleXP:
    """Namespace with the same names as the cumo_b200 package."""
    SFloat, DFloat, Int32, Int64, UInt64, UInt32, Bit = OSFloat, ODFloat, OInt32, OInt64, OUInt64, OUInt32, OBit
    NMath = _ONMath()
    ShapeError = ShapeErrorO
    OperationError = OperationErrorO
    name = "oracle"
