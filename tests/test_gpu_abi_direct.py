"""The C ABI called the way the Ruby extension's generated host code calls it: descriptors filled by hand,
no host layer of this repository in between.  Device memory comes from torch; answers are checked against the
CPU oracle (numpy only carries the bytes).  One case per family of entry points.
"""
import ctypes
from ctypes import byref, c_char_p, c_int, c_int32, c_size_t, c_ssize_t, c_uint64, c_void_p

import numpy as np
import pytest

from oracle import cumo_oracle as orc

pytestmark = pytest.mark.gpu


def iarray(_lib, t, steps_bytes):
    a = _lib.NaIArray()
    a.ptr = t.data_ptr()
    for d, s in enumerate(steps_bytes):
        a.step[d] = s
    return a


def indexer(_lib, shape):
    ix = _lib.NaIndexer()
    ix.ndim = len(shape)
    ix.total_size = int(np.prod(shape))
    for d, n in enumerate(shape):
        ix.shape[d] = n
    return ix


@pytest.fixture()
def lib():
    from cumo_b200 import _lib

    return _lib, _lib.load()


def test_binary_broadcast_with_zero_steps(lib):
    """cumo_iter_sfloat_add_kernel_launch on (R,1) + (1,C): the broadcast axes carry step 0 (ndloop.c:523-595)."""
    import torch

    _lib, L = lib
    fn = L.cumo_iter_sfloat_add_kernel_launch
    fn.restype = None
    fn.argtypes = [ctypes.POINTER(_lib.NaIArray)] * 3 + [ctypes.POINTER(_lib.NaIndexer), ctypes.POINTER(c_int)]
    g = torch.Generator(device="cuda").manual_seed(1)
    r, c = 301, 1030
    x, y = torch.randn(r, 1, device="cuda", generator=g), torch.randn(1, c, device="cuda", generator=g)
    out = torch.empty(r, c, device="cuda")
    fn(byref(iarray(_lib, x, (4, 0))), byref(iarray(_lib, y, (0, 4))), byref(iarray(_lib, out, (4 * c, 4))), byref(indexer(_lib, (r, c))), None)
    torch.cuda.synchronize()
    want, _ = orc.binary("add", np.broadcast_to(x.cpu().numpy(), (r, c)), np.broadcast_to(y.cpu().numpy(), (r, c)))
    assert np.array_equal(out.cpu().numpy(), want)


def test_reduction_arg_sum_and_max_index(lib):
    """cumo_sfloat_sum_kernel_launch and cumo_sfloat_max_index_int32_kernel_launch over the last axis of (R, C)."""
    import torch

    _lib, L = lib
    g = torch.Generator(device="cuda").manual_seed(2)
    r, c = 513, 4100
    src = torch.rand(r, c, device="cuda", generator=g)
    for name, out_dtype in (("cumo_sfloat_sum_kernel_launch", torch.float32), ("cumo_sfloat_max_index_int32_kernel_launch", torch.int32)):
        fn = getattr(L, name)
        fn.restype = None
        fn.argtypes = [ctypes.POINTER(_lib.NaReductionArg)]
        out = torch.empty(r, device="cuda", dtype=out_dtype)
        arg = _lib.NaReductionArg()
        arg.in_.ptr, arg.out.ptr = src.data_ptr(), out.data_ptr()
        arg.in_indexer = indexer(_lib, (r, c))
        arg.out_indexer = indexer(_lib, (r,))
        arg.in_.step[0], arg.in_.step[1] = 4 * c, 4
        arg.out.step[0] = 4
        fn(byref(arg))
        torch.cuda.synchronize()
        host = src.cpu().numpy()
        if out_dtype == torch.float32:
            ref = host.astype(np.float64).sum(axis=1)
            assert np.all(np.abs(out.cpu().numpy() - ref) <= 1e-5 * ref)
        else:
            assert np.array_equal(out.cpu().numpy(), orc.reduce("max_index", host, axis=1))


def test_compare_scalar_count_true_and_where(lib):
    """cumo_iter_int32_gt_s_kernel_launch -> Bit words, cumo_iter_bit_count_true_stride_kernel_launch,
    cumo_bit_where_scratch_new / cumo_bit_where_kernel_launch."""
    import torch

    _lib, L = lib
    n = 100_003
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randint(-50, 50, (n,), device="cuda", dtype=torch.int32, generator=g)
    words = torch.zeros((n + 31) // 32, device="cuda", dtype=torch.int32)
    gt = L.cumo_iter_int32_gt_s_kernel_launch
    gt.restype = None
    gt.argtypes = [ctypes.POINTER(_lib.NaIArray), c_int32, ctypes.POINTER(_lib.NaBitIArray), ctypes.POINTER(_lib.NaIndexer), c_int]
    bits = _lib.NaBitIArray()
    bits.ptr, bits.pos = words.data_ptr(), 0
    bits.step[0] = 1
    gt(byref(iarray(_lib, a, (4,))), 10, byref(bits), byref(indexer(_lib, (n,))), 0)
    count = torch.zeros(1, device="cuda", dtype=torch.int64)
    ct = L.cumo_iter_bit_count_true_stride_kernel_launch
    ct.restype = None
    ct.argtypes = [c_size_t, c_void_p, c_void_p, c_ssize_t, c_uint64]
    ct(0, count.data_ptr(), words.data_ptr(), 1, n)
    torch.cuda.synchronize()
    host = a.cpu().numpy()
    hits = int((host > 10).sum())
    assert count.item() == hits
    L.cumo_bit_where_scratch_new.restype = c_void_p
    L.cumo_bit_where_scratch_new.argtypes = []
    scratch = L.cumo_bit_where_scratch_new()
    assert scratch
    where = L.cumo_bit_where_kernel_launch
    where.restype = None
    where.argtypes = [c_void_p, c_size_t, c_ssize_t, c_void_p, c_uint64, c_int, c_void_p, c_size_t, c_uint64, c_void_p]
    idx = torch.empty(hits, device="cuda", dtype=torch.int32)
    half = n // 2                                      # two launches: the cursor in the scratch carries on from the first
    where(words.data_ptr(), 0, 1, None, half, 0, idx.data_ptr(), 4, 0, scratch)
    where(words.data_ptr(), half, 1, None, n - half, 0, idx.data_ptr(), 4, half, scratch)
    torch.cuda.synchronize()
    L.cumo_cuda_runtime_free.argtypes = [c_void_p]
    L.cumo_cuda_runtime_free(scratch)
    assert np.array_equal(idx.cpu().numpy(), orc.where(host > 10))


def test_bincount_and_cumsum_entries(lib):
    """cumo_iter_int32_bincount_32_kernel_launch with its flag words, cumo_sfloat_cumsum_kernel_launch on a strided run."""
    import torch

    _lib, L = lib
    g = torch.Generator(device="cuda").manual_seed(4)
    n, bins = 70_001, 300
    items = torch.randint(0, bins, (n,), device="cuda", dtype=torch.int32, generator=g)
    items[17] = bins + 4                                # one item outside the output: reported, skipped
    counts = torch.empty(bins, device="cuda", dtype=torch.int32)
    oor = torch.zeros(1, device="cuda", dtype=torch.int32)
    item = torch.zeros(1, device="cuda", dtype=torch.int64)
    bc = L.cumo_iter_int32_bincount_32_kernel_launch
    bc.restype = None
    bc.argtypes = [c_void_p, c_ssize_t, c_void_p, c_uint64, c_void_p, c_ssize_t, c_uint64, c_void_p, c_void_p]
    bc(items.data_ptr(), 4, None, n, counts.data_ptr(), 4, bins, oor.data_ptr(), item.data_ptr())
    torch.cuda.synchronize()
    host = items.cpu().numpy()
    assert oor.item() == 1 and item.item() == bins + 4
    keep = host[host < bins]
    assert np.array_equal(counts.cpu().numpy().astype(np.uint32), orc.bincount(keep, minlength=bins))

    x = torch.randint(-3, 4, (2 * n,), device="cuda", generator=g).float()
    out = torch.zeros(n, device="cuda")
    cs = L.cumo_sfloat_cumsum_kernel_launch
    cs.restype = c_int
    cs.argtypes = [c_void_p, c_void_p, c_ssize_t, c_ssize_t, c_uint64]
    assert cs(x.data_ptr(), out.data_ptr(), 8, 4, n) == 0               # every second element
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), orc.cum("cumsum", x.cpu().numpy()[::2]))
