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


def _colmajor(a):
    """numpy (rows, cols) -> a CUDA tensor holding it column-major (as cuBLAS sees it), plus its leading dimension."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a.T)).cuda()          # memory: column after column
    return t, a.shape[0]


@pytest.mark.parametrize("dtype", ["float32", "float64"])
@pytest.mark.parametrize("transa,transb", [(0, 0), (1, 0), (0, 1), (1, 1)])
def test_gemm_strided_batched_against_float64(dtype, transa, transb):
    """cb200_{s,d}gemm_strided_batched with cuBLAS's column-major semantics: every transpose combination, alpha/beta,
    batches, sizes that are not multiples of any tile (CUDA-core kernel)."""
    import ctypes
    import torch
    from cumo_b200 import _lib

    L = _lib.load()
    f = L.cb200_sgemm_strided_batched if dtype == "float32" else L.cb200_dgemm_strided_batched
    f.restype = ctypes.c_int
    f.argtypes = None
    cT = ctypes.c_float if dtype == "float32" else ctypes.c_double
    rng = np.random.default_rng(transa * 2 + transb)
    m, n, k, batch = 131, 77, 45, 3
    A = rng.standard_normal((batch, k, m) if transa else (batch, m, k)).astype(dtype)
    B = rng.standard_normal((batch, n, k) if transb else (batch, k, n)).astype(dtype)
    C0 = rng.standard_normal((batch, m, n)).astype(dtype)
    alpha, beta = 1.5, -0.25
    dA = torch.from_numpy(np.ascontiguousarray(A.transpose(0, 2, 1))).cuda()      # each entry column-major
    dB = torch.from_numpy(np.ascontiguousarray(B.transpose(0, 2, 1))).cuda()
    dC = torch.from_numpy(np.ascontiguousarray(C0.transpose(0, 2, 1))).cuda()
    lda, ldb, ldc = A.shape[1], B.shape[1], m
    rc = f(ctypes.c_int(transa), ctypes.c_int(transb), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k), ctypes.byref(cT(alpha)),
           ctypes.c_void_p(dA.data_ptr()), ctypes.c_int(lda), ctypes.c_longlong(A.shape[1] * A.shape[2]),
           ctypes.c_void_p(dB.data_ptr()), ctypes.c_int(ldb), ctypes.c_longlong(B.shape[1] * B.shape[2]), ctypes.byref(cT(beta)),
           ctypes.c_void_p(dC.data_ptr()), ctypes.c_int(ldc), ctypes.c_longlong(m * n), ctypes.c_int(batch))
    assert rc == 0
    torch.cuda.synchronize()
    got = dC.cpu().numpy().transpose(0, 2, 1).astype(np.float64)
    opA = A.transpose(0, 2, 1) if transa else A
    opB = B.transpose(0, 2, 1) if transb else B
    want = alpha * np.matmul(opA.astype(np.float64), opB.astype(np.float64)) + beta * C0.astype(np.float64)
    scale = np.matmul(np.abs(opA).astype(np.float64), np.abs(opB).astype(np.float64)) * abs(alpha) + abs(beta) * np.abs(C0)
    tol = 2e-6 if dtype == "float32" else 1e-14
    assert np.all(np.abs(got - want) <= tol * scale + 1e-30)


@pytest.mark.parametrize("transa,transb", [(0, 0), (1, 0), (0, 1), (1, 1)])
def test_sgemm_strided_batched_takes_the_tensor_core_path(transa, transb):
    """Large single-precision products with alpha 1, beta 0 go to the tcgen05 kernel, whatever the transposes (an operand that
    is not K-contiguous is copied transposed first); beta = 0 must not read C (it starts as NaN here)."""
    import ctypes
    import torch
    from cumo_b200 import _lib

    L = _lib.load()
    f = L.cb200_sgemm_strided_batched
    f.restype = ctypes.c_int
    f.argtypes = None
    rng = np.random.default_rng(10 + transa * 2 + transb)
    m, n, k, batch = 520, 300, 256, 2
    A = rng.standard_normal((batch, k, m) if transa else (batch, m, k)).astype(np.float32)
    B = rng.standard_normal((batch, n, k) if transb else (batch, k, n)).astype(np.float32)
    dA = torch.from_numpy(np.ascontiguousarray(A.transpose(0, 2, 1))).cuda()
    dB = torch.from_numpy(np.ascontiguousarray(B.transpose(0, 2, 1))).cuda()
    dC = torch.full((batch, n, m), float("nan"), device="cuda")
    before = L.cb200_launch_count()
    rc = f(ctypes.c_int(transa), ctypes.c_int(transb), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k), ctypes.byref(ctypes.c_float(1.0)),
           ctypes.c_void_p(dA.data_ptr()), ctypes.c_int(A.shape[1]), ctypes.c_longlong(A.shape[1] * A.shape[2]),
           ctypes.c_void_p(dB.data_ptr()), ctypes.c_int(B.shape[1]), ctypes.c_longlong(B.shape[1] * B.shape[2]), ctypes.byref(ctypes.c_float(0.0)),
           ctypes.c_void_p(dC.data_ptr()), ctypes.c_int(m), ctypes.c_longlong(m * n), ctypes.c_int(batch))
    assert rc == 0
    torch.cuda.synchronize()
    assert L.cb200_launch_count() - before >= batch
    got = dC.cpu().numpy().transpose(0, 2, 1).astype(np.float64)
    opA = A.transpose(0, 2, 1) if transa else A
    opB = B.transpose(0, 2, 1) if transb else B
    want = np.matmul(opA.astype(np.float64), opB.astype(np.float64))
    scale = np.matmul(np.abs(opA).astype(np.float64), np.abs(opB).astype(np.float64))
    assert np.all(np.abs(got - want) <= 2e-6 * scale)


@pytest.mark.parametrize("tname", ["SFloat", "DFloat"])
def test_gemm_method_with_views_and_batches(xp_gpu, tname):
    """`gemm` the way the reference's method is used: row-major operands, a transposed view on either side (passed as a
    flag, not copied), leading batch axes, alpha and beta."""
    from cumo_b200 import linalg

    rng = np.random.default_rng(21)
    dt = np.float32 if tname == "SFloat" else np.float64
    T = getattr(xp_gpu, tname)
    a = rng.standard_normal((3, 70, 45)).astype(dt)
    b = rng.standard_normal((3, 45, 33)).astype(dt)
    c = rng.standard_normal((3, 70, 33)).astype(dt)
    tol = 2e-6 if dt == np.float32 else 1e-14
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    scale = np.matmul(np.abs(a).astype(np.float64), np.abs(b).astype(np.float64))
    got = linalg.gemm(T.from_numpy(a), T.from_numpy(b)).to_numpy()
    assert np.all(np.abs(got - want) <= tol * scale)
    got = linalg.gemm(T.from_numpy(a), T.from_numpy(b), alpha=2.0, beta=0.5, c=T.from_numpy(c)).to_numpy()
    assert np.all(np.abs(got - (2.0 * want + 0.5 * c)) <= tol * (2.0 * scale + np.abs(c)))
    # 2-D, second operand a transposed view; then the first
    a2, bt = a[0], np.ascontiguousarray(b[0].T)
    got = linalg.gemm(T.from_numpy(a2), T.from_numpy(bt).transpose()).to_numpy()
    assert np.all(np.abs(got - want[0]) <= tol * scale[0])
    at = np.ascontiguousarray(a2.T)
    got = linalg.dot(T.from_numpy(at).transpose(), T.from_numpy(b[0])).to_numpy()
    assert np.all(np.abs(got - want[0]) <= tol * scale[0])
