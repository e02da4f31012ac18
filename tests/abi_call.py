"""Test helper: the reference's descriptors (cumo_na_iarray_t, cumo_na_indexer_t, cumo_na_bit_iarray_t,
cumo_na_reduction_arg_t, cumo_na_iarray_stridx_t) filled from torch tensors, the way the Ruby extension's
generated host code fills them from its loop arguments (ext/cumo/include/cumo/indexer.h:114-220).  The same
descriptors can be handed to libcumo_b200.so and to the reference's own kernels (oracle/_ref)."""
import ctypes
from ctypes import byref, c_double, c_float, c_int, c_int32, c_int64, c_size_t, c_ssize_t, c_uint64, c_void_p  # noqa: F401

import numpy as np

from cumo_b200 import _lib

MAX_DIM = _lib.MAX_DIM
TYPE_OF = {"sfloat": ("float32", c_float), "dfloat": ("float64", c_double), "int32": ("int32", c_int32), "int64": ("int64", c_int64)}


class Stridx(ctypes.Union):
    _fields_ = [("stride", c_ssize_t), ("index", c_void_p)]


class NaIArrayStridx(ctypes.Structure):
    _fields_ = [("ptr", c_void_p), ("stridx", Stridx * MAX_DIM)]


def torch_dtype(tname):
    import torch
    return getattr(torch, TYPE_OF[tname][0])


def scalar(tname, v):
    return TYPE_OF[tname][1](v)


def indexer(shape):
    ix = _lib.NaIndexer()
    ix.ndim = len(shape)
    ix.total_size = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
    for d, n in enumerate(shape):
        ix.shape[d] = n
    return ix


def iarray(t, shape=None):
    """Descriptor of tensor `t` as seen through broadcasting to `shape` (extent-1 dims get step 0)."""
    a = _lib.NaIArray()
    a.ptr = t.data_ptr()
    es = t.element_size()
    shape = tuple(t.shape) if shape is None else tuple(shape)
    lead = len(shape) - t.dim()
    for d in range(len(shape)):
        if d < lead:
            a.step[d] = 0
        else:
            td = d - lead
            a.step[d] = 0 if (t.shape[td] == 1 and shape[d] != 1) else t.stride(td) * es
    return a


def bit_iarray(words, pos=0, steps=(1,)):
    b = _lib.NaBitIArray()
    b.ptr, b.pos = words.data_ptr(), pos
    for d, s in enumerate(steps):
        b.step[d] = s
    return b


def contiguous_bit_steps(shape):
    steps, s = [], 1
    for n in reversed(shape):
        steps.append(s)
        s *= n
    return tuple(reversed(steps))


def reduction_arg(src, out, axes):
    """Reduce `axes` of `src` into `out` (whose dims are src's kept dims in order): the reduce dims go last
    (ndloop.c:421-451), out steps cover the kept dims (indexer.h:189-220)."""
    nd = src.dim()
    axes = sorted(a % nd for a in axes)
    keep = [d for d in range(nd) if d not in axes]
    order = keep + axes
    es = src.element_size()
    arg = _lib.NaReductionArg()
    arg.in_.ptr, arg.out.ptr = src.data_ptr(), out.data_ptr()
    arg.in_indexer.ndim = nd
    arg.in_indexer.total_size = src.numel()
    for i, d in enumerate(order):
        arg.in_indexer.shape[i] = src.shape[d]
        arg.in_.step[i] = src.stride(d) * es
    arg.out_indexer.ndim = len(keep)
    arg.out_indexer.total_size = int(np.prod([src.shape[d] for d in keep], dtype=np.int64)) if keep else 1
    for i, d in enumerate(keep):
        arg.out_indexer.shape[i] = src.shape[d]
        arg.out.step[i] = out.stride(i) * out.element_size()
    return arg


def stridx_iarray(t, index_arrays=None):
    """cumo_na_iarray_stridx_t of tensor `t`; index_arrays[d], when given, is a device int64 tensor of BYTE offsets
    that replaces dimension d's step (narray.h:329-330: a step is stored as (s << 1) | 1)."""
    a = NaIArrayStridx()
    a.ptr = t.data_ptr()
    es = t.element_size()
    for d in range(t.dim()):
        ia = (index_arrays or {}).get(d)
        if ia is not None:
            a.stridx[d].index = ia.data_ptr()
        else:
            a.stridx[d].stride = ((t.stride(d) * es) << 1) | 1
    return a


def fn(L, name, restype=None):
    f = getattr(L, name)
    f.restype = restype
    f.argtypes = None
    return f


def bits_equal(a, b):
    """Same bytes (NaN payloads included)."""
    import torch
    if a.dtype.is_floating_point:
        it = torch.int32 if a.element_size() == 4 else torch.int64
        return torch.equal(a.contiguous().view(it), b.contiguous().view(it))
    return torch.equal(a, b)


def same_values(a, b):
    """Equal where both are numbers, NaN exactly where the other is NaN."""
    import torch
    if a.dtype.is_floating_point:
        return bool(torch.all((a == b) | (torch.isnan(a) & torch.isnan(b))))
    return torch.equal(a, b)
