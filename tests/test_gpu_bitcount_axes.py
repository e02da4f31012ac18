"""count_true / count_false along axes in one launch (cb200_bit_count_axes_kernel_launch) against numpy counts:
row runs, column walks, several kept and counted dimensions, views that start inside a word, sliced counted ranges."""
import ctypes
from ctypes import c_int, c_size_t, c_ssize_t, c_void_p

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _bits(shape, seed):
    return np.random.default_rng(seed).random(shape) < 0.37


@pytest.mark.parametrize("shape,axis", [((300, 2048), 1), ((300, 2048), 0), ((7, 33, 130), (0, 2)), ((7, 33, 130), 1), ((7, 33, 130), (1, 2)),
                                        ((5, 4, 3, 70), (1, 3)), ((2, 70_000), 1), ((70_000, 3), 0), ((4, 100_000), 0), ((129, 65), 1)])
def test_counts_along_axes_match_numpy(shape, axis):
    import cumo_b200 as xp

    host = _bits(shape, sum(shape))
    m = xp.Bit.cast(host)
    for keepdims in (False, True):
        got_t = m.count_true(axis=axis, keepdims=keepdims).to_numpy()
        got_f = m.count_false(axis=axis, keepdims=keepdims).to_numpy()
        want = host.sum(axis=axis, keepdims=keepdims)
        total = np.prod([shape[a] for a in ((axis,) if isinstance(axis, int) else axis)])
        assert got_t.dtype == np.uint64 and np.array_equal(got_t, want.astype(np.uint64))
        assert np.array_equal(got_f, (total - want).astype(np.uint64))


def test_counts_along_axes_of_views():
    import cumo_b200 as xp

    host = _bits((37, 301), 5)
    m = xp.Bit.cast(host)
    cases = {
        "columns 3..": (m[True, 3:], host[:, 3:]),
        "reversed rows": (m[::-1, True], host[::-1, :]),
        "every other column": (m[True, ::2], host[:, ::2]),
        "transpose": (m.transpose(), host.T),
        "inner block": (m[5:30, 40:200], host[5:30, 40:200]),
    }
    for what, (view, ref) in cases.items():
        for axis in (0, 1):
            assert np.array_equal(view.count_true(axis=axis).to_numpy(), ref.sum(axis=axis).astype(np.uint64)), (what, axis)
            assert np.array_equal(view.count_false(axis=axis).to_numpy(), (ref.shape[axis] - ref.sum(axis=axis)).astype(np.uint64)), (what, axis)


def test_launch_function_adds_to_its_output_and_takes_negative_steps():
    """Through the C ABI: the count is added to what the output holds, and a counted dimension may walk backwards."""
    import torch
    from cumo_b200 import _lib

    L = _lib.load()
    fn = L.cb200_bit_count_axes_kernel_launch
    fn.restype = None
    rows, cols = 50, 1000
    host = _bits((rows, cols), 9)
    words = np.zeros((rows * cols + 31) // 32 + 2, dtype=np.uint32)
    flat = np.packbits(np.concatenate([np.zeros(13, dtype=bool), host.reshape(-1)]), bitorder="little")
    words.view(np.uint8)[:flat.size] = flat
    dev = torch.from_numpy(words.view(np.int32)).cuda()
    S, SS = c_size_t * 1, c_ssize_t * 1
    for want_false in (0, 1):
        out = torch.full((rows,), 5, dtype=torch.int64, device="cuda")
        # rows kept, columns counted from the last one backwards (bit step -1: the column walk)
        fn(c_void_p(dev.data_ptr()), c_size_t(13 + cols - 1), c_int(want_false), c_int(1), S(rows), SS(cols), SS(8), c_int(1), S(cols), SS(-1), c_void_p(out.data_ptr()))
        torch.cuda.synchronize()
        ones = host.sum(axis=1)
        assert np.array_equal(out.cpu().numpy(), 5 + (cols - ones if want_false else ones))
        out = torch.full((cols,), 7, dtype=torch.int64, device="cuda")
        fn(c_void_p(dev.data_ptr()), c_size_t(13), c_int(want_false), c_int(1), S(cols), SS(1), SS(8), c_int(1), S(rows), SS(cols), c_void_p(out.data_ptr()))
        torch.cuda.synchronize()
        ones = host.sum(axis=0)
        assert np.array_equal(out.cpu().numpy(), 7 + (rows - ones if want_false else ones))
    msg = ctypes.c_char_p()
    assert L.cb200_last_error(ctypes.byref(msg)) == 0, msg.value
