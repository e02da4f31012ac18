"""Tensor-core matrix product against a float64 reference.

Bar: every element within 2e-6 x sum_k |a_ik b_kj| of the float64 product -- the error bound of an fp32 dot
product of that length under any summation order is a small multiple of 6e-8 x that sum, and the split-TF32
scheme adds about 5e-7 x it.  Operands include zero rows, ragged tile edges and a K that is not a multiple of 32.
"""
import numpy as np
import pytest

from oracle import cumo_oracle as orc

pytestmark = pytest.mark.gpu

TOL = 2e-6


@pytest.mark.parametrize("m,n,k", [(1, 1, 4), (128, 256, 32), (127, 255, 36), (129, 257, 64), (300, 520, 100), (1000, 700, 512),
                                   (64, 3000, 256), (4096, 256, 64), (150 * 128, 256, 32), (256, 512, 4096), (100, 300, 8200)])
def test_gemm_nt_matches_float64(xp_gpu, m, n, k):
    from cumo_b200 import linalg

    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    bt = rng.standard_normal((n, k)).astype(np.float32)
    if m > 4:
        a[3] = 0
    got = linalg.gemm_nt(xp_gpu.SFloat.from_numpy(a), xp_gpu.SFloat.from_numpy(bt)).to_numpy().astype(np.float64)
    want, scale = orc.gemm_nt_f64(a, bt)
    assert got.shape == want.shape
    assert np.all(np.abs(got - want) <= TOL * scale + 1e-30), float(np.max(np.abs(got - want) / (scale + 1e-30)))


def test_dot_transposes_the_second_operand(xp_gpu):
    from cumo_b200 import linalg

    rng = np.random.default_rng(0)
    a = rng.standard_normal((200, 96)).astype(np.float32)
    b = rng.standard_normal((96, 333)).astype(np.float32)
    got = linalg.dot(xp_gpu.SFloat.from_numpy(a), xp_gpu.SFloat.from_numpy(b)).to_numpy().astype(np.float64)
    want, scale = orc.gemm_nt_f64(a, np.ascontiguousarray(b.T))
    assert np.all(np.abs(got - want) <= TOL * scale)
    v = rng.standard_normal(96).astype(np.float32)
    got = linalg.dot(xp_gpu.SFloat.from_numpy(a), xp_gpu.SFloat.from_numpy(v)).to_numpy().astype(np.float64)
    want, scale = orc.gemm_nt_f64(a, v[None, :])
    assert np.all(np.abs(got - want[:, 0]) <= TOL * scale[:, 0])


def test_gemm_refuses_unsupported_shapes(xp_gpu):
    from cumo_b200 import linalg

    with pytest.raises(xp_gpu.CumoError, match="multiples of 4"):
        linalg.gemm_nt(xp_gpu.SFloat.zeros(8, 6), xp_gpu.SFloat.zeros(8, 6))


def test_a_bounded_wait_that_runs_out_returns_an_error_code():
    """The waits between the warp roles of the tcgen05 kernels are bounded; when one runs out the kernel winds down and
    the entry point returns 5.  The self-test makes such a wait run out by its (short) limit on a barrier that nothing
    arrives at: the kernel returns, the code is 5, and the device keeps working."""
    import ctypes

    import torch
    from cumo_b200 import _lib

    L = _lib.load()
    f = L.cb200_selftest_bounded_wait
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_uint, ctypes.c_char_p, ctypes.c_size_t]
    err = ctypes.create_string_buffer(200)
    assert f(2000, err, len(err)) == 5, err.value
    assert b"ran out" in err.value
    x = torch.arange(10, device="cuda").sum().item()             # the context is still usable
    assert x == 45
