"""mulsum over a whole loop in one launch (cb200_<T>_mulsum*_axes_kernel_launch) against numpy: sums along the inner and
the outer axis, broadcast operands, several kept and summed dimensions, the integer dot, NaN pairs dropped."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CASES = [((300, 2048), (300, 2048), 1), ((300, 2048), (300, 2048), 0), ((300, 2048), (1, 2048), 1), ((300, 2048), (300, 1), 0),
         ((7, 33, 130), (7, 33, 130), (0, 2)), ((7, 33, 130), (7, 33, 130), 1), ((7, 33, 130), (33, 130), (1, 2)),
         ((5000, 9), (5000, 9), 1), ((70, 20_000), (70, 20_000), 1), ((20_000, 70), (20_000, 70), 0), ((100_000, 3), (100_000, 3), 0),
         ((200_000, 16), (200_000, 16), 1), ((100_000, 32), (100_000, 32), 1), ((90_000, 8), (90_000, 8), 1), ((80_000, 60), (80_000, 60), 1)]


@pytest.mark.parametrize("sa,sb,axis", CASES)
def test_integer_mulsum_over_axes_is_exact(sa, sb, axis):
    import cumo_b200 as xp

    rng = np.random.default_rng(sum(sa))
    for T, dt in ((xp.Int32, np.int32), (xp.Int64, np.int64)):
        a = rng.integers(-9, 10, size=sa).astype(dt)
        b = rng.integers(-9, 10, size=sb).astype(dt)
        got = T.from_numpy(a).mulsum(T.from_numpy(b), axis=axis).to_numpy()
        assert np.array_equal(got, (a * b).sum(axis=axis, dtype=dt))
        got = T.from_numpy(a).mulsum(T.from_numpy(b), axis=axis, keepdims=True).to_numpy()
        assert np.array_equal(got, (a * b).sum(axis=axis, dtype=dt, keepdims=True))


@pytest.mark.parametrize("sa,sb,axis", CASES)
def test_float_mulsum_over_axes(sa, sb, axis):
    import cumo_b200 as xp

    rng = np.random.default_rng(sum(sa) + 1)
    for T, dt, tol in ((xp.SFloat, np.float32, 1e-5), (xp.DFloat, np.float64, 1e-12)):
        a = rng.standard_normal(sa).astype(dt)
        b = rng.standard_normal(sb).astype(dt)
        got = T.from_numpy(a).mulsum(T.from_numpy(b), axis=axis).to_numpy()
        prod = a.astype(np.float64) * b.astype(np.float64)
        want, scale = prod.sum(axis=axis), np.abs(prod).sum(axis=axis)
        assert np.all(np.abs(got - want) <= tol * scale + 1e-30)
        an = a.copy()
        an.reshape(-1)[::41] = np.nan
        got = T.from_numpy(an).mulsum(T.from_numpy(b), axis=axis, nan=True).to_numpy()
        prod = np.where(np.isnan(an), 0, an).astype(np.float64) * b.astype(np.float64)
        assert np.all(np.abs(got - prod.sum(axis=axis)) <= tol * np.abs(prod).sum(axis=axis) + 1e-30)
        assert np.isnan(T.from_numpy(an).mulsum(T.from_numpy(b), axis=axis).to_numpy()).any()


def test_integer_dot_of_matrices_and_views():
    import cumo_b200 as xp

    rng = np.random.default_rng(8)
    a = rng.integers(-9, 10, size=(97, 130)).astype(np.int64)
    b = rng.integers(-9, 10, size=(130, 211)).astype(np.int64)
    A, B = xp.Int64.from_numpy(a), xp.Int64.from_numpy(b)
    assert np.array_equal(A.dot(B).to_numpy(), a @ b)
    assert np.array_equal(A.dot(B[True, ::-1]).to_numpy(), a @ b[:, ::-1])
    bt = xp.Int64.from_numpy(np.ascontiguousarray(b.T))
    assert np.array_equal(A.dot(bt.transpose()).to_numpy(), a @ b)
    a32, b32 = a.astype(np.int32), b.astype(np.int32)
    assert np.array_equal(xp.Int32.from_numpy(a32).dot(xp.Int32.from_numpy(b32)).to_numpy(), (a32 @ b32).astype(np.int32))
