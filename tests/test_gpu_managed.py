"""The launch functions on MANAGED memory, which is what every Cumo buffer is (the reference's pool hands out
cudaMallocManaged blocks, ext/cumo/cuda/memory_pool_impl.cpp:16-22).  One entry point of each family is called through
the C ABI on managed buffers that the host has just written (so their pages live on the host: the kernel faults them
over, the "cold" case) and again after a prefetch to the device, and checked against the CPU oracle; results are read
back through the managed pointer on the host, as `extract_cpu` does.
"""
import ctypes
from ctypes import byref, c_int, c_int32, c_size_t, c_ssize_t, c_uint64, c_void_p

import numpy as np
import pytest

from oracle import cumo_oracle as orc

pytestmark = pytest.mark.gpu


class Managed:
    """A cudaMallocManaged block seen as a numpy array on the host and as a pointer on the device."""

    def __init__(self, shape, dtype):
        from cuda.bindings import runtime as rt

        self.rt = rt
        self.shape, self.dtype = tuple(shape), np.dtype(dtype)
        self.nbytes = max(1, int(np.prod(self.shape)) * self.dtype.itemsize)
        err, self.ptr = rt.cudaMallocManaged(self.nbytes, rt.cudaMemAttachGlobal)
        assert err == rt.cudaError_t.cudaSuccess, err
        buf = (ctypes.c_char * self.nbytes).from_address(int(self.ptr))
        self.host = np.frombuffer(buf, dtype=self.dtype, count=int(np.prod(self.shape))).reshape(self.shape)

    def prefetch_to_device(self):
        rt = self.rt
        loc = rt.cudaMemLocation()
        loc.type = rt.cudaMemLocationType.cudaMemLocationTypeDevice
        loc.id = 0
        try:
            (err,) = rt.cudaMemPrefetchAsync(self.ptr, self.nbytes, loc, 0, 0)
        except TypeError:                                  # older binding: (ptr, bytes, device, stream)
            (err,) = rt.cudaMemPrefetchAsync(self.ptr, self.nbytes, 0, 0)
        assert err == rt.cudaError_t.cudaSuccess, err

    def free(self):
        self.rt.cudaFree(self.ptr)


def sync():
    import torch
    torch.cuda.synchronize()


def desc(_lib, m, steps=None):
    a = _lib.NaIArray()
    a.ptr = int(m.ptr)
    st = steps if steps is not None else [s for s in m.host.strides]
    for d, s in enumerate(st):
        a.step[d] = s
    return a


def indexer(_lib, shape):
    ix = _lib.NaIndexer()
    ix.ndim = len(shape)
    ix.total_size = int(np.prod(shape))
    for d, n in enumerate(shape):
        ix.shape[d] = n
    return ix


@pytest.mark.parametrize("prefetch", [False, True], ids=["cold", "prefetched"])
def test_one_entry_point_of_each_family_on_managed_buffers(prefetch):
    import torch
    from cumo_b200 import _lib

    torch.cuda.set_device(0)
    L = _lib.load()
    rng = np.random.default_rng(9)
    r, c = 700, 3000
    x, y, out = Managed((r, 1), np.float32), Managed((1, c), np.float32), Managed((r, c), np.float32)
    x.host[...] = rng.standard_normal((r, 1))
    y.host[...] = rng.standard_normal((1, c))
    bufs = [x, y, out]
    try:
        if prefetch:
            for b in bufs:
                b.prefetch_to_device()
        # elementwise, broadcast: (r,1) + (1,c)
        f = L.cumo_iter_sfloat_add_kernel_launch
        f.restype, f.argtypes = None, None
        f(byref(desc(_lib, x, (4, 0))), byref(desc(_lib, y, (0, 4))), byref(desc(_lib, out)), byref(indexer(_lib, (r, c))), None)
        sync()
        want = x.host + y.host
        assert np.array_equal(out.host, want)
        # math
        e = Managed((r, c), np.float32)
        bufs.append(e)
        if prefetch:
            e.prefetch_to_device()
        g = L.cumo_iter_sfloat_math_s_exp_kernel_launch
        g.restype, g.argtypes = None, None
        g(byref(desc(_lib, out)), byref(desc(_lib, e)), byref(indexer(_lib, (r, c))))
        sync()
        assert np.allclose(e.host, orc.unary("exp", want)[0], rtol=2e-6)
        # reductions over both axes and an index reduction
        for axes_last, n_out in ((True, r), (False, c)):
            res = Managed((n_out,), np.float32)
            idx = Managed((n_out,), np.int32)
            bufs += [res, idx]
            if prefetch:
                res.prefetch_to_device(); idx.prefetch_to_device()
            arg = _lib.NaReductionArg()
            arg.in_.ptr, arg.in_indexer.ndim, arg.in_indexer.total_size = int(e.ptr), 2, r * c
            if axes_last:
                arg.in_indexer.shape[0], arg.in_indexer.shape[1] = r, c
                arg.in_.step[0], arg.in_.step[1] = 4 * c, 4
            else:
                arg.in_indexer.shape[0], arg.in_indexer.shape[1] = c, r
                arg.in_.step[0], arg.in_.step[1] = 4, 4 * c
            arg.out_indexer.ndim, arg.out_indexer.total_size = 1, n_out
            arg.out_indexer.shape[0] = n_out
            for sym, dst, es in (("cumo_sfloat_sum_kernel_launch", res, 4), ("cumo_sfloat_max_index_int32_kernel_launch", idx, 4)):
                arg.out.ptr = int(dst.ptr)
                arg.out.step[0] = es
                h = getattr(L, sym)
                h.restype, h.argtypes = None, None
                h(byref(arg))
            sync()
            axis = 1 if axes_last else 0
            ref = e.host.astype(np.float64).sum(axis=axis)
            assert np.all(np.abs(res.host - ref) <= 1e-5 * np.abs(ref))
            assert np.array_equal(idx.host, orc.reduce("max_index", e.host, axis=axis))
        # comparison into Bit words and the Bit count
        n = r * c
        words = Managed(((n + 31) // 32,), np.uint32)
        words.host[...] = 0
        total = Managed((1,), np.uint64)
        total.host[...] = 0
        bufs += [words, total]
        if prefetch:
            words.prefetch_to_device(); total.prefetch_to_device()
        bits = _lib.NaBitIArray()
        bits.ptr, bits.pos = int(words.ptr), 0
        bits.step[0] = 1
        gt = L.cumo_iter_sfloat_gt_s_kernel_launch
        gt.restype, gt.argtypes = None, None
        flat = _lib.NaIArray()
        flat.ptr = int(out.ptr)
        flat.step[0] = 4
        gt(byref(flat), ctypes.c_float(0.25), byref(bits), byref(indexer(_lib, (n,))), c_int(0))
        ct = L.cumo_iter_bit_count_true_stride_kernel_launch
        ct.restype, ct.argtypes = None, None
        ct(c_size_t(0), c_void_p(int(total.ptr)), c_void_p(int(words.ptr)), c_ssize_t(1), c_uint64(n))
        sync()
        assert int(total.host[0]) == int((want > 0.25).sum())
        assert np.array_equal(np.unpackbits(words.host.view(np.uint8), bitorder="little")[:n].astype(bool), (want > 0.25).reshape(-1))
        msg = ctypes.c_char_p()
        assert L.cb200_last_error(byref(msg)) == 0, msg.value
    finally:
        sync()
        for b in bufs:
            b.free()
