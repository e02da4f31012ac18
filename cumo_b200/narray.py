"""Python face of the host layer: `SFloat`, `DFloat`, `Int32`, `Int64`, `Bit`, `NMath`.

Method names and argument meanings are those of `Cumo::NArray`
(ext/cumo/narray/gen/spec.rb:113-461; Ruby keyword arguments `axis:`, `keepdims:`,
`nan:` become Python keywords), so that a test written against the reference's
test/narray_test.rb reads the same here.  Every operation goes through
include/cumo_b200_host.h into the kernel-launch ABI; this file only converts
arguments and owns handles.  Reductions return 0-dimensional arrays, as the
reference does outside its compatible mode (gen/tmpl/extract.c:15-22); `extract()`
reads one back.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_ssize_t, c_uint64, c_void_p

import numpy as np

from . import _lib

SFLOAT, DFLOAT, INT32, INT64, BIT, UINT64, UINT32 = range(7)
_NP = {SFLOAT: np.float32, DFLOAT: np.float64, INT32: np.int32, INT64: np.int64, UINT64: np.uint64, UINT32: np.uint32}
_ESZ = {SFLOAT: 4, DFLOAT: 8, INT32: 4, INT64: 8, BIT: 1, UINT64: 8, UINT32: 4}   # Bit: unit is one bit


class CumoError(Exception):
    pass


class ShapeError(CumoError):
    pass


class CudaError(CumoError):
    pass


class OperationError(CumoError):
    """`Cumo::NArray::OperationError`"""


_ERRORS = {"ShapeError": ShapeError, "ZeroDivisionError": ZeroDivisionError, "ValueError": ValueError,
           "TypeError": TypeError, "CudaError": CudaError, "NoMethodError": AttributeError,
           "IndexError": IndexError, "ArgumentError": ValueError, "OperationError": OperationError}


def _raise_last():
    lib = _lib.load()
    klass = c_char_p()
    msg = lib.cb200_host_error(byref(klass))
    exc = _ERRORS.get((klass.value or b"").decode(), CumoError)
    raise exc((msg or b"").decode())


def _arr64(values):
    return (c_int64 * max(1, len(values)))(*values)


def _axis_mask(axis, ndim):
    if axis is None:
        return 0
    axes = [axis] if isinstance(axis, int) else list(axis)
    mask = 0
    for ax in axes:
        if ax < 0:
            ax += ndim
        if not 0 <= ax < ndim:
            raise ValueError(f"axis {ax} out of range for ndim {ndim}")
        mask |= 1 << ax
    if ndim and mask == 0:
        raise ValueError("empty axis list")
    return mask


class NArray:
    """A typed device array or a view of one."""

    dtype_code: int = -1
    _types: dict[int, type] = {}

    def __init_subclass__(cls, **kw):
        super().__init_subclass__(**kw)
        if cls.dtype_code >= 0:
            NArray._types[cls.dtype_code] = cls

    # ---- construction -------------------------------------------------------------------
    def __init__(self, *shape):
        """`SFloat.new(2, 3)`: an uninitialised array of that shape."""
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        lib = _lib.load()
        self._keep = None
        self._h = lib.cb200_na_new(self.dtype_code, len(shape), _arr64(shape))
        if not self._h:
            _raise_last()

    new = classmethod(lambda cls, *shape: cls(*shape))

    @classmethod
    def _from_handle(cls, h, keep=None):
        if not h:
            _raise_last()
        lib = _lib.load()
        klass = NArray._types[lib.cb200_na_dtype(h)]
        obj = object.__new__(klass)
        obj._h = h
        obj._keep = keep
        return obj

    def __del__(self):
        h = getattr(self, "_h", None)
        if h and _lib._lib is not None:
            _lib._lib.cb200_na_release(h)
            self._h = None

    def __class_getitem__(cls, item):
        """`SFloat[[1, 2, 3], [5, 7, 11]]`, the reference's `Cumo::SFloat[...]` literal."""
        data = list(item) if isinstance(item, tuple) else [item]
        return cls.cast(data)

    @classmethod
    def cast(cls, data):
        """From a nested list / numpy array (host data is uploaded) or another NArray (converted)."""
        if isinstance(data, NArray):
            if data.dtype_code == cls.dtype_code:
                return data
            return NArray._from_handle(_lib.load().cb200_na_cast(data._h, cls.dtype_code))
        if cls.dtype_code == BIT:
            return cls.from_numpy(np.asarray(data).astype(bool))
        return cls.from_numpy(np.asarray(data, dtype=_NP[cls.dtype_code]))

    @classmethod
    def from_numpy(cls, x: np.ndarray):
        lib = _lib.load()
        if cls.dtype_code == BIT:
            x = np.ascontiguousarray(x).astype(bool)
            words = pack_bits(x.reshape(-1))
            out = cls(*x.shape)
            if lib.cb200_na_store_host(out._h, words.ctypes.data_as(c_void_p), words.nbytes):
                _raise_last()
            lib.cb200_synchronize()
            return out
        x = np.ascontiguousarray(x, dtype=_NP[cls.dtype_code])
        out = cls(*x.shape)
        if x.size and lib.cb200_na_store_host(out._h, x.ctypes.data_as(c_void_p), x.nbytes):
            _raise_last()
        lib.cb200_synchronize()   # x may be a temporary; the copy must have left it
        return out

    @classmethod
    def from_host_pointer(cls, ptr: int, shape, nbytes: int):
        """Asynchronous upload from (pinned) host memory the caller keeps alive until it synchronises."""
        out = cls(*shape)
        if _lib.load().cb200_na_store_host(out._h, c_void_p(ptr), nbytes):
            _raise_last()
        return out

    def read_into_host_async(self, ptr: int, nbytes: int, copy_stream: int):
        """Queue the copy of this (contiguous) array into pinned host memory on `copy_stream` (a cudaStream_t handle),
        behind the kernels queued so far; the caller keeps both alive and synchronises that stream before reading."""
        if _lib.load().cb200_na_read_host_async(self._h, c_void_p(ptr), nbytes, c_void_p(copy_stream)):
            _raise_last()

    @classmethod
    def from_torch(cls, t):
        """Borrow a CUDA tensor's memory (no copy); the tensor is kept alive by the view."""
        import torch

        want = {SFLOAT: torch.float32, DFLOAT: torch.float64, INT32: torch.int32, INT64: torch.int64}[cls.dtype_code]
        if t.dtype != want or not t.is_cuda:
            raise TypeError(f"{cls.__name__}.from_torch needs a CUDA tensor of {want}")
        es = t.element_size()
        h = _lib.load().cb200_na_wrap(cls.dtype_code, t.dim(), _arr64(list(t.shape)),
                                      _arr64([s * es for s in t.stride()]), c_void_p(t.data_ptr()), 0)
        return NArray._from_handle(h, keep=t)

    @classmethod
    def from_device_pointer(cls, ptr: int, shape, keep=None):
        """Borrow device-accessible memory the caller owns (cudaMalloc, cudaMallocManaged, another library's buffer) as a
        contiguous array of this type; `keep` is held for as long as the array lives."""
        shape = [int(n) for n in shape]
        es = _ESZ[cls.dtype_code]
        steps, st = [], es
        for n in reversed(shape):
            steps.append(st)
            st *= n
        h = _lib.load().cb200_na_wrap(cls.dtype_code, len(shape), _arr64(shape), _arr64(list(reversed(steps))), c_void_p(ptr), 0)
        return NArray._from_handle(h, keep=keep)

    @classmethod
    def zeros(cls, *shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        return NArray._from_handle(_lib.load().cb200_na_zeros(cls.dtype_code, len(shape), _arr64(shape)))

    @classmethod
    def ones(cls, *shape):
        return cls.zeros(*shape).fill(1)

    def fill(self, value):
        """`a.fill(v)` (gen/tmpl/fill.c:18-27): every element of `a` -- an array or any view of one -- takes `v`,
        converted to the element type the way a cast converts it."""
        if self.dtype_code == BIT:                                       # Bit#fill: the value's low bit
            if _lib.load().cb200_na_fill(self._h, 0.0, int(value) & 1):
                _raise_last()
            return self
        if self.dtype_code not in (SFLOAT, DFLOAT, INT32, INT64):       # index and count types: filled from the host
            self._store(type(self).from_numpy(np.full(self.shape, value, dtype=_NP[self.dtype_code])))
            return self
        f, i = self._numeric(value)
        if _lib.load().cb200_na_fill(self._h, f, i):
            _raise_last()
        return self

    def seq(self, start=0, step=1):
        """`a.seq(beg, step)` (gen/tmpl/seq.c:21-117): element i, counted in row-major order over `a`'s own shape,
        takes beg + i*step."""
        if self.dtype_code not in (SFLOAT, DFLOAT, INT32, INT64):
            host = (start + step * np.arange(self.size)).astype(_NP[self.dtype_code]).reshape(self.shape)
            self._store(type(self).from_numpy(host))
            return self
        if _lib.load().cb200_na_seq(self._h, float(start), float(step)):
            _raise_last()
        return self

    def _numeric(self, value):
        """A host numeric as the (float, int) pair the host layer picks from by element type."""
        if self.dtype_code in (SFLOAT, DFLOAT):
            return float(value), 0
        return 0.0, int(value)                                # a Float against an integer type truncates (NUM2INT)

    def _store(self, other):
        """self[...] = other through the store kernel (same shape)."""
        lib = _lib.load()
        name = f"cumo_iter_{self._tname}_store_{other._tname}_kernel_launch"
        fn = getattr(lib, name)
        fn.restype = None
        ix, dst = self._descriptors()
        _, src = other._descriptors()
        fn(byref(dst), byref(src), byref(ix))
        _check_launch()

    def store(self, other):
        """`self.store(other)` of the reference (gen/tmpl/store.c, store_from.c): every element of `self` -- an array or
        any view of one -- takes the matching element of `other`, which is converted to this type and repeated along
        the dimensions where its extent is 1 or that it lacks (ndloop.c:494-516).  Returns self."""
        if not isinstance(other, NArray):
            other = type(self).cast(other if isinstance(other, (list, tuple, np.ndarray)) else [other])
        shp = self.shape
        oshp, ostp = other.shape, other.steps
        if other.size == 1:
            oshp, ostp = (), ()                              # a single element is repeated everywhere
        if len(oshp) > len(shp):
            raise ShapeError(f"cannot store an array of shape {oshp} into one of shape {shp}")
        steps = []
        for d in range(len(shp)):
            od = d - (len(shp) - len(oshp))
            if od < 0 or oshp[od] == 1:
                steps.append(0)
            elif oshp[od] == shp[d]:
                steps.append(ostp[od])
            else:
                raise ShapeError(f"cannot store an array of shape {oshp} into one of shape {shp}")
        self._store(other._view(list(shp), steps, 0))
        return self

    def __setitem__(self, key, value):
        """`a[key] = value`: a store into the view that `a[key]` names (integers, slices, `True`, None, Ellipsis)."""
        self[key].store(value)

    # ---- facts --------------------------------------------------------------------------------
    @property
    def _tname(self):
        return ["sfloat", "dfloat", "int32", "int64", "bit", "uint64", "uint32"][self.dtype_code]

    @property
    def ndim(self):
        return _lib.load().cb200_na_ndim(self._h)

    @property
    def shape(self):
        n = self.ndim
        buf = (c_int64 * max(1, n))()
        _lib.load().cb200_na_shape(self._h, buf)
        return tuple(buf[:n])

    @property
    def steps(self):
        """Byte steps (bit steps for Bit)."""
        n = self.ndim
        buf = (c_int64 * max(1, n))()
        _lib.load().cb200_na_steps(self._h, buf)
        return tuple(buf[:n])

    @property
    def offset(self):
        return _lib.load().cb200_na_offset(self._h)

    @property
    def size(self):
        return int(_lib.load().cb200_na_size(self._h))

    @property
    def data_ptr(self):
        base = _lib.load().cb200_na_base(self._h) or 0
        return base + (self.offset if self.dtype_code != BIT else 0)

    def contiguous(self):
        return bool(_lib.load().cb200_na_is_contiguous(self._h))

    def _descriptors(self):
        """(cumo_na_indexer_t, cumo_na_iarray_t) of this array as ndloop would build them."""
        ix = _lib.NaIndexer()
        ia = _lib.NaIArray()
        shp, stp = self.shape, self.steps
        ix.ndim = len(shp)
        ix.total_size = int(np.prod(shp, dtype=np.int64)) if shp else 1
        for d, (n, s) in enumerate(zip(shp, stp)):
            ix.shape[d] = n
            ia.step[d] = s if n != 1 else 0
        ia.ptr = self.data_ptr
        return ix, ia

    @property
    def __cuda_array_interface__(self):
        if self.dtype_code == BIT:
            raise TypeError("a Bit array has no element-addressable interface")
        return {"shape": self.shape, "typestr": np.dtype(_NP[self.dtype_code]).str, "data": (self.data_ptr, False),
                "version": 3, "strides": self.steps if not self.contiguous() else None}

    # ---- host copies ------------------------------------------------------------------------------
    def to_numpy(self) -> np.ndarray:
        lib = _lib.load()
        src = self if self.contiguous() else self.dup()
        if self.dtype_code == BIT:
            raise TypeError("use Bit.to_numpy")
        out = np.empty(src.shape, dtype=_NP[self.dtype_code])
        if out.size and lib.cb200_na_read_host(src._h, out.ctypes.data_as(c_void_p), out.nbytes):
            _raise_last()
        return out

    def to_a(self):
        return self.to_numpy().tolist()

    def extract(self):
        """The single element of a 0-d (or 1-element) array as a Python number; synchronises."""
        if self.size != 1:
            raise ValueError("extract needs exactly one element")
        return self.to_numpy().reshape(()).item()

    def __float__(self):
        return float(self.extract())

    def __int__(self):
        return int(self.extract())

    def __repr__(self):
        return f"{type(self).__name__}{list(self.shape)}"

    # ---- views ------------------------------------------------------------------------------------
    def _view(self, shape, steps, offset):
        h = _lib.load().cb200_na_view(self._h, len(shape), _arr64(list(shape)), _arr64(list(steps)), offset)
        return NArray._from_handle(h, keep=self._keep)

    def __getitem__(self, key):
        """Integers, slices (any step), None (new axis) and Ellipsis; `True` means `:` as in Ruby.  One list or
        integer array among the keys picks positions along that axis (`a[[5, 0, 3], true]`), and a Bit array of
        the same shape selects where it is one (`a[mask]`); both return the copy that the reference makes when
        such a view is next used (gen/tmpl/store_from.c:82-89, gen/tmpl_bit/mask.c:95-140)."""
        if isinstance(key, Bit):
            return key.mask(self)
        if not isinstance(key, tuple):
            key = (key,)
        picks = [i for i, k in enumerate(key) if isinstance(k, (list, np.ndarray, NArray))]
        if picks:
            if len(picks) > 1:
                raise IndexError("one index array per expression on this path")
            at = picks[0]
            axis = sum(1 for k in key[:at] if k is not None and k is not Ellipsis and (k is True or not isinstance(k, int)))
            rest = tuple(True if i == at else k for i, k in enumerate(key))
            return self[rest].take(key[at], axis)
        shp, stp = self.shape, self.steps
        n_real = sum(1 for k in key if k is not None and k is not Ellipsis)
        if n_real > len(shp):
            raise IndexError("too many indices")
        out_shape, out_steps, off, d = [], [], 0, 0
        for k in key:
            if k is Ellipsis:
                for _ in range(len(shp) - n_real):
                    out_shape.append(shp[d]); out_steps.append(stp[d]); d += 1
            elif k is None:
                out_shape.append(1); out_steps.append(0)
            elif k is True:
                out_shape.append(shp[d]); out_steps.append(stp[d]); d += 1
            elif isinstance(k, slice):
                start, stop, step = k.indices(shp[d])
                n = len(range(start, stop, step))
                out_shape.append(n); out_steps.append(stp[d] * step); off += start * stp[d]; d += 1
            else:
                i = int(k)
                if i < 0:
                    i += shp[d]
                if not 0 <= i < shp[d]:
                    raise IndexError(f"index {k} out of range for extent {shp[d]}")
                off += i * stp[d]; d += 1
        while d < len(shp):
            out_shape.append(shp[d]); out_steps.append(stp[d]); d += 1
        return self._view(out_shape, out_steps, off)

    def take(self, index, axis=0):
        """The elements at `index` (a list or an Int32/Int64 array of positions, negative ones counting from the end)
        along `axis`, as a new array."""
        if not isinstance(index, NArray):
            pos = np.asarray(index, dtype=np.int64)
            n = self.shape[axis]
            if pos.size and (pos.min() < -n or pos.max() >= n):
                raise IndexError(f"index out of range for extent {n}")
            index = Int64.from_numpy(np.where(pos < 0, pos + n, pos))
        return NArray._from_handle(_lib.load().cb200_na_take(self._h, int(axis), index._h))

    def transpose(self, *perm):
        shp, stp = self.shape, self.steps
        if not perm:
            perm = tuple(reversed(range(len(shp))))
        if sorted(perm) != list(range(len(shp))):
            raise ValueError("transpose needs a permutation of the axes")
        return self._view([shp[p] for p in perm], [stp[p] for p in perm], 0)

    def reverse(self, axis=None):
        shp, stp = self.shape, self.steps
        axes = range(len(shp)) if axis is None else ([axis] if isinstance(axis, int) else axis)
        steps, off = list(stp), 0
        for ax in axes:
            if shp[ax]:
                off += (shp[ax] - 1) * stp[ax]
            steps[ax] = -stp[ax]
        return self._view(shp, steps, off)

    def reshape(self, *shape):
        """A new array with the same elements; like the reference's reshape it copies
        (narray/data.c:501-518) unless the array is already contiguous, where a view suffices."""
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        shape = list(shape)
        if shape.count(-1) == 1:
            known = int(np.prod([s for s in shape if s != -1], dtype=np.int64))
            shape[shape.index(-1)] = self.size // known if known else 0
        if int(np.prod(shape, dtype=np.int64)) != self.size:
            raise ShapeError(f"cannot reshape {self.shape} into {tuple(shape)}")
        src = self if self.contiguous() else self.dup()
        unit = _ESZ[self.dtype_code]
        steps, s = [], unit
        for n in reversed(shape):
            steps.append(s); s *= n
        v = src._view(shape, list(reversed(steps)), 0)
        v._parent = src
        return v

    def flatten(self):
        return self.reshape(self.size)

    def dup(self):
        return NArray._from_handle(_lib.load().cb200_na_copy(self._h))

    copy = dup

    def inplace(self):
        """`x.inplace + y` writes the result into x."""
        _lib.load().cb200_na_set_inplace(self._h, 1)
        return self

    # ---- elementwise --------------------------------------------------------------------------------
    def _binary(self, op, other, reflected=False):
        lib = _lib.load()
        if isinstance(other, NArray):
            a, b = (other, self) if reflected else (self, other)
            return NArray._from_handle(lib.cb200_na_binary(op.encode(), a._h, b._h))
        if isinstance(other, (list, tuple, np.ndarray)):
            return self._binary(op, type(self).cast(other), reflected)
        a, f, i = self._scalar_operand(other)
        return NArray._from_handle(lib.cb200_na_binary_scalar(op.encode(), a._h, f, i, 1 if reflected else 0))

    def _scalar_operand(self, value):
        """A Python float against an integer array upcasts the array to DFloat, as
        `upcast_rb "Float", "DFloat"` says (gen/def/int32.rb:23); an int keeps the array's type."""
        a = self
        if isinstance(value, (float, np.floating)) and self.dtype_code in (INT32, INT64):
            a = DFloat.cast(self)
        if a.dtype_code in (SFLOAT, DFLOAT):
            return a, float(value), 0
        return a, 0.0, int(value)

    def __add__(self, o): return self._binary("add", o)
    def __radd__(self, o): return self._binary("add", o, True)
    def __sub__(self, o): return self._binary("sub", o)
    def __rsub__(self, o): return self._binary("sub", o, True)
    def __mul__(self, o): return self._binary("mul", o)
    def __rmul__(self, o): return self._binary("mul", o, True)
    def __truediv__(self, o): return self._binary("div", o)
    def __rtruediv__(self, o): return self._binary("div", o, True)
    def __floordiv__(self, o): return self._binary("div", o)
    def __mod__(self, o): return self._binary("mod", o)
    def __rmod__(self, o): return self._binary("mod", o, True)
    def __and__(self, o): return self._binary("bit_and", o)
    def __or__(self, o): return self._binary("bit_or", o)
    def __xor__(self, o): return self._binary("bit_xor", o)
    def __lshift__(self, o): return self._binary("left_shift", o)
    def __rshift__(self, o): return self._binary("right_shift", o)

    def __pow__(self, o):
        # an Integer exponent multiplies repeatedly (gen/tmpl/pow.c: the pow_int32 path)
        if isinstance(o, (int, np.integer)) and not isinstance(o, bool):
            return NArray._from_handle(_lib.load().cb200_na_pow_int(self._h, int(o)))
        return self._binary("pow", o)

    def __rpow__(self, o): return self._binary("pow", o, True)
    pow = __pow__

    def copysign(self, o): return self._binary("copysign", o)

    @classmethod
    def maximum(cls, a, b, nan=False): return cls.cast(a)._binary("maximum_nan" if nan else "maximum", cls.cast(b))

    @classmethod
    def minimum(cls, a, b, nan=False): return cls.cast(a)._binary("minimum_nan" if nan else "minimum", cls.cast(b))

    def clip(self, min=None, max=None):
        """`a.clip(min, max)` (gen/tmpl/clip.c:218-276): each bound is None, a number or an array (converted to
        `a`'s type and repeated like any operand).  The result has `a`'s type; `a.inplace.clip(..)` writes into `a`.
        OperationError when min > max anywhere, ValueError when neither bound is given."""
        def bound(b):
            if b is None:
                return 0, None, 0.0, 0
            if isinstance(b, (list, tuple, np.ndarray)):
                b = type(self).cast(b)
            if isinstance(b, NArray):
                return 2, b._h, 0.0, 0
            f, i = self._numeric(b)
            return 1, None, f, i
        lo, hi = bound(min), bound(max)
        return NArray._from_handle(_lib.load().cb200_na_clip(self._h, *lo, *hi))

    def _repeated_to(self, shape):
        """A view of this array repeated to `shape` (extents of 1 and missing leading dimensions get step 0), as ndloop
        lines an operand up with the loop (ndloop.c:494-516)."""
        oshp, ostp = self.shape, self.steps
        if self.size == 1:
            oshp, ostp = (), ()
        if len(oshp) > len(shape):
            raise ShapeError(f"an operand of shape {oshp} does not fit a loop of shape {tuple(shape)}")
        steps = []
        for d in range(len(shape)):
            od = d - (len(shape) - len(oshp))
            if od < 0 or oshp[od] == 1:
                steps.append(0)
            elif oshp[od] == shape[d]:
                steps.append(ostp[od])
            else:
                raise ShapeError(f"an operand of shape {oshp} does not fit a loop of shape {tuple(shape)}")
        return self._view(list(shape), steps, 0)

    def poly(self, *coefs):
        """`x.poly(a0, a1, ..., an)` = a0 + a1*x + ... + an*x**n by Horner's rule in one launch (gen/tmpl/poly.c:46-88);
        a coefficient is a number or an array repeated to x's shape; no coefficient answers x."""
        T = type(self)
        numbers = [c for c in coefs if not isinstance(c, (NArray, list, tuple, np.ndarray))]
        held = T(len(numbers)) if numbers else None              # numeric coefficients: filled on the device, nothing to wait for
        for k, c in enumerate(numbers):
            held[k:k + 1].fill(c)
        ops, taken = [], 0
        for c in coefs:
            if isinstance(c, NArray):
                c = c if c.dtype_code == self.dtype_code else T.cast(c)
            elif isinstance(c, (list, tuple, np.ndarray)):
                c = T.cast(c)
            else:
                c = held[taken:taken + 1]
                taken += 1
            ops.append(c._repeated_to(self.shape))
        out = T(*self.shape)
        if self.size == 0:
            return out
        lib = _lib.load()
        fn = getattr(lib, f"cumo_iter_{self._tname}_poly_kernel_launch")
        fn.restype = None
        ix, dx = self._descriptors()
        _, dz = out._descriptors()
        arr = (_lib.NaIArray * max(1, len(ops)))()
        for i, c in enumerate(ops):
            _, dc = c._descriptors()
            arr[i] = dc
        fn(byref(dx), arr, c_int(len(ops)), byref(dz), byref(ix))
        _check_launch()
        return out

    def eye(self, element=1, offset=0):
        """`a.eye(element, offset)` (gen/tmpl/eye.c:58-104): every matrix of the last two dimensions gets `element` on the
        diagonal `offset` above (below, if negative) the main one and zero elsewhere.  Returns self."""
        shp, stp = self.shape, self.steps
        if len(shp) < 2:
            raise ShapeError("less than 2-d array")
        if (offset >= 0 and offset >= shp[-1]) or (offset < 0 and -offset >= shp[-2]):
            raise ValueError(f"invalid diagonal offset({offset})")
        lib = _lib.load()
        fn = getattr(lib, f"cumo_iter_{self._tname}_eye_stride_kernel_launch")
        fn.restype = None
        f, i = self._numeric(element)
        ctype = {SFLOAT: c_float, DFLOAT: c_double, INT32: c_int32, INT64: c_int64}[self.dtype_code]
        value = ctype(f if self.dtype_code in (SFLOAT, DFLOAT) else i)
        for lead in np.ndindex(*shp[:-2]):                     # one launch per matrix, as ndloop walks the leading dimensions
            ptr = self.data_ptr + sum(k * s for k, s in zip(lead, stp[:-2]))
            fn(c_void_p(ptr), c_ssize_t(stp[-2]), c_ssize_t(stp[-1]), c_ssize_t(offset), value, c_uint64(shp[-2]), c_uint64(shp[-1]))
        _check_launch()
        return self

    def divmod(self, other):
        """`a.divmod(b)` (gen/tmpl/binary2.c:58-95): quotient and remainder of one pass, both in the upcast type."""
        if not isinstance(other, NArray):
            if isinstance(other, (list, tuple, np.ndarray)):
                other = type(self).cast(other)
            else:
                a, f, i = self._scalar_operand(other)
                if a is not self:
                    return a.divmod(other)
                other = type(self).cast([other])
        q, r = c_void_p(), c_void_p()
        if _lib.load().cb200_na_divmod(self._h, other._h, byref(q), byref(r)):
            _raise_last()
        return NArray._from_handle(q.value), NArray._from_handle(r.value)

    def __divmod__(self, other): return self.divmod(other)

    def modf(self):
        """`a.modf` (gen/tmpl/unary_ret2.c:33-44): fractional and integral parts, float types only."""
        x, y = c_void_p(), c_void_p()
        if _lib.load().cb200_na_modf(self._h, byref(x), byref(y)):
            _raise_last()
        return NArray._from_handle(x.value), NArray._from_handle(y.value)

    def _unary(self, op):
        return NArray._from_handle(_lib.load().cb200_na_unary(op.encode(), self._h))

    def __neg__(self): return self._unary("minus")
    def __abs__(self): return self._unary("abs")
    def __invert__(self): return self._unary("bit_not")
    def abs(self): return self._unary("abs")
    def minus(self): return self._unary("minus")
    def reciprocal(self): return self._unary("reciprocal")
    def sign(self): return self._unary("sign")
    def square(self): return self._unary("square")
    def floor(self): return self._unary("floor")
    def round(self): return self._unary("round")
    def ceil(self): return self._unary("ceil")
    def trunc(self): return self._unary("trunc")
    def rint(self): return self._unary("rint")

    def _compare(self, op, other, reflected=False):
        lib = _lib.load()
        if isinstance(other, NArray):
            a, b = (other, self) if reflected else (self, other)
            return NArray._from_handle(lib.cb200_na_compare(op.encode(), a._h, b._h))
        if isinstance(other, (list, tuple, np.ndarray)):
            return self._compare(op, type(self).cast(other), reflected)
        a, f, i = self._scalar_operand(other)
        return NArray._from_handle(lib.cb200_na_compare_scalar(op.encode(), a._h, f, i, 1 if reflected else 0))

    def eq(self, o): return self._compare("eq", o)
    def ne(self, o): return self._compare("ne", o)
    def gt(self, o): return self._compare("gt", o)
    def ge(self, o): return self._compare("ge", o)
    def lt(self, o): return self._compare("lt", o)
    def le(self, o): return self._compare("le", o)
    def nearly_eq(self, o): return self._compare("nearly_eq", o)
    __gt__ = gt
    __ge__ = ge
    __lt__ = lt
    __le__ = le

    def _classify(self, op):
        return NArray._from_handle(_lib.load().cb200_na_compare(op.encode(), self._h, None))

    def isnan(self): return self._classify("isnan")
    def isinf(self): return self._classify("isinf")
    def isposinf(self): return self._classify("isposinf")
    def isneginf(self): return self._classify("isneginf")
    def isfinite(self): return self._classify("isfinite")
    def signbit(self): return self._classify("signbit")

    # ---- reductions ------------------------------------------------------------------------------------
    def _reduce(self, op, axis=None, keepdims=False, nan=False):
        mask = _axis_mask(axis, self.ndim)
        return NArray._from_handle(_lib.load().cb200_na_reduce(op.encode(), self._h, mask, int(keepdims), int(nan)))

    def sum(self, axis=None, keepdims=False, nan=False): return self._reduce("sum", axis, keepdims, nan)
    def prod(self, axis=None, keepdims=False, nan=False): return self._reduce("prod", axis, keepdims, nan)
    def mean(self, axis=None, keepdims=False, nan=False): return self._reduce("mean", axis, keepdims, nan)
    def var(self, axis=None, keepdims=False, nan=False): return self._reduce("var", axis, keepdims, nan)
    def stddev(self, axis=None, keepdims=False, nan=False): return self._reduce("stddev", axis, keepdims, nan)
    def rms(self, axis=None, keepdims=False, nan=False): return self._reduce("rms", axis, keepdims, nan)
    def kahan_sum(self, axis=None, keepdims=False, nan=False): return self._reduce("kahan_sum", axis, keepdims, nan)
    def min(self, axis=None, keepdims=False, nan=False): return self._reduce("min", axis, keepdims, nan)
    def max(self, axis=None, keepdims=False, nan=False): return self._reduce("max", axis, keepdims, nan)
    def ptp(self, axis=None, keepdims=False, nan=False): return self._reduce("ptp", axis, keepdims, nan)
    def max_index(self, axis=None, nan=False): return self._reduce("max_index", axis, False, nan)
    def min_index(self, axis=None, nan=False): return self._reduce("min_index", axis, False, nan)
    def argmax(self, axis=None, nan=False): return self._reduce("argmax", axis, False, nan)
    def argmin(self, axis=None, nan=False): return self._reduce("argmin", axis, False, nan)

    def minmax(self, axis=None, keepdims=False, nan=False):
        lo, hi = c_void_p(), c_void_p()
        if _lib.load().cb200_na_minmax(self._h, _axis_mask(axis, self.ndim), int(keepdims), int(nan), byref(lo), byref(hi)):
            _raise_last()
        return NArray._from_handle(lo.value), NArray._from_handle(hi.value)

    def _cum(self, op, axis, nan):
        if axis is not None and not isinstance(axis, int):
            raise TypeError("cumsum / cumprod take one axis or none")
        ax = -1 if axis is None else (axis % self.ndim if self.ndim else 0)
        return NArray._from_handle(_lib.load().cb200_na_cum(op.encode(), self._h, ax, int(nan)))

    def cumsum(self, axis=None, nan=False): return self._cum("cumsum", axis, nan)
    def cumprod(self, axis=None, nan=False): return self._cum("cumprod", axis, nan)

    def bincount(self, weight=None, minlength=0):
        """Occurrences (or summed weights) of each value along the last axis (Int32 / Int64 only)."""
        if weight is not None and not isinstance(weight, NArray):
            weight = DFloat.cast(weight)
        return NArray._from_handle(_lib.load().cb200_na_bincount(self._h, weight._h if weight is not None else None, int(minlength)))

    def arg_with_value(self, op, axis=None, nan=False):
        """(index Int64, value) of max_index / min_index / argmax / argmin from one pass over the data."""
        idx, val = c_void_p(), c_void_p()
        if _lib.load().cb200_na_arg_with_value(op.encode(), self._h, _axis_mask(axis, self.ndim), int(nan), byref(idx), byref(val)):
            _raise_last()
        return NArray._from_handle(idx.value), NArray._from_handle(val.value)

    def gemm(self, b, c=None, alpha=1, beta=0):
        """`a.gemm(b, c, alpha:, beta:)` of the reference for the float types (gen/tmpl/gemm.c): alpha * a . b + beta * c
        over the last two axes, leading axes are batches; `b` is converted to this array's type."""
        from . import linalg
        if not isinstance(b, NArray) or type(b) is not type(self):
            b = type(self).cast(b)
        return linalg.gemm(self, b, alpha=float(alpha), beta=float(beta), c=c)

    def dot(self, b):
        """`a.dot(b)` as lib/cumo/narray/extra.rb:1145-1196 spells it: the float types go to gemm (vectors get a unit
        axis for the call), the integer types to mulsum over a new axis."""
        if not isinstance(b, NArray):
            b = type(self).cast(b)
        code = max(self.dtype_code, b.dtype_code) if {self.dtype_code, b.dtype_code} <= {INT32, INT64} else None
        if code is None:
            floats = [t for t in (self, b) if t.dtype_code in (SFLOAT, DFLOAT)]
            T = DFloat if any(t.dtype_code == DFLOAT for t in floats) else SFloat
        else:
            T = Int64 if code == INT64 else Int32
        if self.ndim == 0 and b.ndim == 0:
            return self * b
        a = self if type(self) is T else T.cast(self)
        b = b if type(b) is T else T.cast(b)
        if T in (SFloat, DFloat):
            if a.ndim == 1:
                if b.ndim == 1:
                    return a.mulsum(b, axis=-1)
                return a[None, ...].gemm(b).flatten()
            if b.ndim == 1:
                return a.gemm(b[..., None]).flatten()
            return a.gemm(b)
        if b.ndim == 1:
            return a.mulsum(b, axis=-1)
        if a.ndim == 0:
            return b.mulsum(a, axis=-2)
        if a.ndim == 1:
            return a[True, None].mulsum(b, axis=-2)
        return a[..., None].mulsum(b[..., None, True, True], axis=-2)

    def mulsum(self, other, axis=None, keepdims=False, nan=False):
        other = other if isinstance(other, NArray) else type(self).cast(other)
        nd = max(self.ndim, other.ndim)
        return NArray._from_handle(_lib.load().cb200_na_mulsum(self._h, other._h, _axis_mask(axis, nd), int(keepdims), int(nan)))


class SFloat(NArray):
    dtype_code = SFLOAT


class DFloat(NArray):
    dtype_code = DFLOAT


class Int32(NArray):
    dtype_code = INT32


class Int64(NArray):
    dtype_code = INT64


class UInt64(NArray):
    """Result type of count_true / count_false; no arithmetic is defined on it here."""
    dtype_code = UINT64


class UInt32(NArray):
    """Result type of bincount; no arithmetic is defined on it here."""
    dtype_code = UINT32


class Bit(NArray):
    """One bit per element, packed LSB-first into 32-bit words (narray.h:492-496)."""
    dtype_code = BIT

    def to_numpy(self) -> np.ndarray:
        lib = _lib.load()
        if not (self.contiguous() and self.offset % 32 == 0):
            return self.dup().to_numpy()                      # a view: through the copy kernel into words of its own
        n = self.size
        words = np.empty((n + 31) // 32, dtype=np.uint32)
        if words.size and lib.cb200_na_read_host(self._h, words.ctypes.data_as(c_void_p), words.nbytes):
            _raise_last()
        return unpack_bits(words, n).reshape(self.shape)

    def to_a(self):
        return self.to_numpy().astype(np.int64).tolist()

    def where(self):
        """Ascending row-major positions of the one bits (Int32; Int64 for arrays beyond 2^32-1 elements)."""
        return NArray._from_handle(_lib.load().cb200_na_where(self._h, 0))

    def where2(self):
        """(positions of the ones, positions of the zeros)."""
        lib = _lib.load()
        return NArray._from_handle(lib.cb200_na_where(self._h, 0)), NArray._from_handle(lib.cb200_na_where(self._h, 1))

    def mask(self, array):
        """The elements of `array` (same shape) where this mask is one, in row-major order, as a 1-D array."""
        return NArray._from_handle(_lib.load().cb200_na_mask(self._h, array._h))

    def count_true(self, axis=None, keepdims=False):
        return NArray._from_handle(_lib.load().cb200_na_count(self._h, _axis_mask(axis, self.ndim), int(keepdims), 0))

    def count_false(self, axis=None, keepdims=False):
        return NArray._from_handle(_lib.load().cb200_na_count(self._h, _axis_mask(axis, self.ndim), int(keepdims), 1))

    count = count_1 = count_true
    count_0 = count_false

    # ---- Bit o Bit (gen/spec.rb:169-174: copy, not, and, or, xor, eq) and all? / any? / none? (:185-186, tmpl_bit/none_p.c) --
    def _bit_operand(self, o):
        if isinstance(o, Bit):
            return o
        return Bit.cast(o if isinstance(o, (list, tuple, np.ndarray)) else [o])

    def _bit_op(self, op, o=None):
        other = None if o is None else self._bit_operand(o)
        return NArray._from_handle(_lib.load().cb200_na_bit_op(op.encode(), self._h, other._h if other is not None else None))

    def __and__(self, o): return self._bit_op("and", o)
    def __or__(self, o): return self._bit_op("or", o)
    def __xor__(self, o): return self._bit_op("xor", o)
    __rand__, __ror__, __rxor__ = __and__, __or__, __xor__
    def __invert__(self): return self._bit_op("not")
    def eq(self, o): return self._bit_op("eq", o)
    def dup(self): return self._bit_op("copy")
    copy = dup

    def _bit_reduce(self, op, axis, keepdims):
        out = NArray._from_handle(_lib.load().cb200_na_bit_reduce(op.encode(), self._h, _axis_mask(axis, self.ndim), int(keepdims)))
        if axis is None and not keepdims:
            return bool(out.to_numpy().reshape(-1)[0])          # without an axis the reference answers true / false
        return out

    def all(self, axis=None, keepdims=False):
        """`all?`: every bit is one (an empty array answers false, as in tmpl_bit/bit_reduce.c:137-139)."""
        return False if self.size == 0 else self._bit_reduce("all", axis, keepdims)

    def any(self, axis=None, keepdims=False):
        return False if self.size == 0 else self._bit_reduce("any", axis, keepdims)

    def none(self, axis=None, keepdims=False):
        r = self.any(axis=axis, keepdims=keepdims)
        return (not r) if isinstance(r, bool) else ~r

    @property
    def data_ptr(self):
        return _lib.load().cb200_na_base(self._h) or 0


class _NMath:
    """`Cumo::NMath`: functions dispatch on the argument's type (narray/math.c:80-103)."""

    _one = ("sqrt cbrt log log2 log10 exp exp2 exp10 sin cos tan asin acos atan sinh cosh tanh "
            "asinh acosh atanh sinc erf erfc log1p expm1").split()
    _two = ("atan2", "hypot", "ldexp")

    def __getattr__(self, name):
        if name in self._one:
            def f(x):
                x = x if isinstance(x, NArray) else DFloat.cast(x)
                if x.dtype_code in (INT32, INT64):
                    x = DFloat.cast(x)
                return x._unary(name)
            return f
        if name in self._two:
            def g(x, y):
                if isinstance(x, NArray):
                    return x._binary(name, y)
                return y._binary(name, x, True)
            return g
        raise AttributeError(name)

    def frexp(self, x):
        """`NMath.frexp(x)` (gen/tmpl/frexp.c:36-48): mantissas in x's type and exponents as an Int32 array."""
        x = x if isinstance(x, NArray) else DFloat.cast(x)
        if x.dtype_code in (INT32, INT64):
            x = DFloat.cast(x)
        m, e = c_void_p(), c_void_p()
        if _lib.load().cb200_na_frexp(x._h, byref(m), byref(e)):
            _raise_last()
        return NArray._from_handle(m.value), NArray._from_handle(e.value)


NMath = _NMath()


def pack_bits(flags: np.ndarray) -> np.ndarray:
    """bool[n] -> uint32 words, element i at bit i%32 of word i/32."""
    flags = np.asarray(flags, dtype=bool).reshape(-1)
    pad = (-flags.size) % 32
    if pad:
        flags = np.concatenate([flags, np.zeros(pad, dtype=bool)])
    return np.packbits(flags, bitorder="little").view(np.uint32).copy() if flags.size else np.zeros(0, np.uint32)


def unpack_bits(words: np.ndarray, n: int) -> np.ndarray:
    return np.unpackbits(np.ascontiguousarray(words).view(np.uint8), bitorder="little")[:n].astype(bool)


def _check_launch():
    msg = c_char_p()
    if _lib.load().cb200_last_error(byref(msg)):
        raise CudaError((msg.value or b"").decode())


def synchronize():
    if _lib.load().cb200_synchronize():
        _raise_last()
