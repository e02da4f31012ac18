"""The allocation-free float32 sum (cb200_sfloat_sum_noalloc_kernel_launch).

It exists for callers that cannot reach an allocator when they need a sum (a context in
which the host program's pool callback must not run, an embedder with a fixed device-memory
budget), so it keeps its partial sums in a fixed array inside the library.  The test calls
it through the C ABI, twice in a row per shape -- the second call finds the first call's
partials still in the shared array -- and holds it to the regular entry point's answer
within the fp32 sum tolerance the other tests use.  The file name sorts last so that a run
that stops at the first failure has already run every other test.
"""
import ctypes
from ctypes import byref, c_char_p, c_size_t, create_string_buffer

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

FP32_SUM_TOL = 1e-5


def reduction_arg(_lib, src, out, n_keep):
    """cumo_na_reduction_arg_t for summing the trailing axes of contiguous `src` into `out`."""
    arg = _lib.NaReductionArg()
    arg.in_.ptr = src.data_ptr()
    arg.out.ptr = out.data_ptr()
    arg.in_indexer.ndim = src.dim()
    arg.in_indexer.total_size = src.numel()
    for d in range(src.dim()):
        arg.in_indexer.shape[d] = src.shape[d]
        arg.in_.step[d] = src.stride(d) * 4
    arg.out_indexer.ndim = n_keep
    arg.out_indexer.total_size = out.numel()
    for d in range(n_keep):
        arg.out_indexer.shape[d] = src.shape[d]
        arg.out.step[d] = out.stride(d) * 4 if out.dim() else 0
    return arg


@pytest.mark.parametrize("shape,n_keep", [(((1 << 22) + 3,), 0), ((7, 300_000), 1), ((300, 4096), 1), ((5000, 33), 1), ((64,), 0)])
def test_noalloc_sum_matches_the_regular_entry_point(shape, n_keep):
    import torch
    from cumo_b200 import _lib

    lib = _lib.load()
    fn = lib.cb200_sfloat_sum_noalloc_kernel_launch
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(_lib.NaReductionArg), c_char_p, c_size_t]
    regular = lib.cumo_sfloat_sum_kernel_launch
    regular.restype = None
    regular.argtypes = [ctypes.POINTER(_lib.NaReductionArg)]

    g = torch.Generator(device="cuda").manual_seed(7)
    src = torch.rand(shape, device="cuda", generator=g) * 2 - 1
    out_shape = shape[:n_keep]
    want = torch.empty(out_shape, device="cuda")
    regular(byref(reduction_arg(_lib, src, want, n_keep)))
    scale = src.abs().double().sum(dim=tuple(range(n_keep, len(shape)))) if n_keep else src.abs().double().sum()
    err = create_string_buffer(256)
    for call in range(2):
        got = torch.full(out_shape, float("nan"), device="cuda")
        rc = fn(byref(reduction_arg(_lib, src, got, n_keep)), err, len(err))
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()
        assert torch.all((got.double() - want.double()).abs() <= FP32_SUM_TOL * scale), f"call {call}"
        ref64 = src.double().sum(dim=tuple(range(n_keep, len(shape)))) if n_keep else src.double().sum()
        assert torch.all((got.double() - ref64).abs() <= FP32_SUM_TOL * scale), f"call {call} vs float64"
    msg = c_char_p()
    assert lib.cb200_last_error(byref(msg)) == 0


def test_noalloc_sum_refuses_what_it_cannot_hold():
    import torch
    from cumo_b200 import _lib

    lib = _lib.load()
    fn = lib.cb200_sfloat_sum_noalloc_kernel_launch
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(_lib.NaReductionArg), c_char_p, c_size_t]
    err = create_string_buffer(256)
    # the bound is outputs x segments <= 2^18; 40000 rows of 8 segments (8192 floats each) exceed it.
    # The input is only allocated, never touched: the call must refuse before launching anything.
    src = torch.empty((40_000, 8 * 8192), device="cuda")
    out = torch.full((40_000,), -1.0, device="cuda")
    rc = fn(byref(reduction_arg(_lib, src, out, 1)), err, len(err))
    assert rc == 2 and b"fixed scratch" in err.value
    torch.cuda.synchronize()
    assert torch.all(out == -1.0)                    # nothing was launched
    # a column (strided) reduction is not the layout this variant covers
    m = torch.empty((512, 256), device="cuda")
    arg = reduction_arg(_lib, m.t(), torch.empty((256,), device="cuda"), 1)
    rc = fn(byref(arg), err, len(err))
    assert rc == 1 and b"contiguous" in err.value


def test_noalloc_sum_small_call_first_then_a_segmented_one():
    """A short, unsegmented call followed by a long one that needs the shared array: the first call on a device,
    whatever its shape, is the one that looks the array up, so a caller can warm up with any shape."""
    import torch
    from cumo_b200 import _lib

    lib = _lib.load()
    fn = lib.cb200_sfloat_sum_noalloc_kernel_launch
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(_lib.NaReductionArg), c_char_p, c_size_t]
    err = create_string_buffer(256)
    g = torch.Generator(device="cuda").manual_seed(11)
    for n in (64, (1 << 21) + 5):
        src = torch.rand((n,), device="cuda", generator=g)
        got = torch.full((), float("nan"), device="cuda")
        assert fn(byref(reduction_arg(_lib, src, got, 0)), err, len(err)) == 0, err.value.decode()
        torch.cuda.synchronize()
        ref = src.double().sum()
        assert abs(got.double() - ref) <= FP32_SUM_TOL * ref
