"""cumsum / cumprod along an axis, every run in one launch (cb200_<T>_cum*_runs_kernel_launch), against numpy:
rows (a CTA per run, packed and ragged), columns (a thread per run), several outer dimensions, views, the nan forms."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SHAPES = [((300, 2048), 1), ((300, 2047), 1), ((2048, 300), 0), ((7, 33, 130), 1), ((7, 33, 130), 0), ((7, 33, 130), 2), ((5000, 9), 1),
          ((3, 10_000), 1), ((4, 3, 5000), 2), ((2, 3, 4, 700), 3), ((9000, 2), 0),
          ((1000, 1), 1), ((1000, 2), 1), ((777, 5), 1), ((3000, 31), 1), ((3000, 32), 1), ((3000, 33), 1), ((500, 255), 1), ((40, 50, 64), 2), ((100_000, 16), 1), ((90_000, 64), 1), ((80_000, 4), 1)]


@pytest.mark.parametrize("shape,axis", SHAPES)
def test_integer_scans_along_an_axis_are_exact(shape, axis):
    import cumo_b200 as xp

    rng = np.random.default_rng(sum(shape) + axis)
    for T, dt in ((xp.Int32, np.int32), (xp.Int64, np.int64)):
        host = rng.integers(-9, 10, size=shape).astype(dt)
        a = T.from_numpy(host)
        assert np.array_equal(a.cumsum(axis=axis).to_numpy(), np.cumsum(host, axis=axis, dtype=dt))
        ones = np.where(rng.random(shape) < 0.02, 2, 1).astype(dt) * np.where(rng.random(shape) < 0.1, -1, 1).astype(dt)
        with np.errstate(over="ignore"):
            want = np.cumprod(ones, axis=axis, dtype=dt)                      # wraps like the sequential loop
        assert np.array_equal(T.from_numpy(ones).cumprod(axis=axis).to_numpy(), want)


@pytest.mark.parametrize("shape,axis", SHAPES)
def test_float_scans_along_an_axis(shape, axis):
    import cumo_b200 as xp

    rng = np.random.default_rng(sum(shape) * 3 + axis)
    # multiples of 1/8 below 2^10: every partial sum is exact in fp32, so the comparison is bit for bit whatever the order
    host = rng.integers(-64, 65, size=shape) / 8.0
    for T, dt in ((xp.SFloat, np.float32), (xp.DFloat, np.float64)):
        h = host.astype(dt)
        assert np.array_equal(T.from_numpy(h).cumsum(axis=axis).to_numpy(), np.cumsum(h, axis=axis, dtype=dt))
        # general values: to the tolerance of the sums (fp32 1e-5, fp64 1e-12 of the sum of magnitudes)
        g = rng.standard_normal(shape).astype(dt)
        got = T.from_numpy(g).cumsum(axis=axis).to_numpy()
        want = np.cumsum(g.astype(np.float64), axis=axis)
        scale = np.cumsum(np.abs(g.astype(np.float64)), axis=axis)
        assert np.all(np.abs(got - want) <= (1e-5 if dt == np.float32 else 1e-12) * scale + 1e-30)
        # NaN: carried by the plain form, skipped by the nan form
        hn = h.copy()
        hn.reshape(-1)[::53] = np.nan
        got = T.from_numpy(hn).cumsum(axis=axis, nan=True).to_numpy()
        filled = np.where(np.isnan(hn), 0, hn)
        want = np.cumsum(filled, axis=axis, dtype=dt)
        seen = np.cumsum(~np.isnan(hn), axis=axis) > 0                        # NaN until the first value of the run
        assert np.array_equal(np.isnan(got), ~seen) and np.array_equal(got[seen], want[seen])
        plain = T.from_numpy(hn).cumsum(axis=axis).to_numpy()
        assert np.array_equal(np.isnan(plain), np.cumsum(np.isnan(hn), axis=axis) > 0)


def test_scans_along_an_axis_of_views():
    import cumo_b200 as xp

    host = np.random.default_rng(4).integers(-9, 10, size=(64, 300)).astype(np.int64)
    a = xp.Int64.from_numpy(host)
    cases = {"transpose": (a.transpose(), host.T), "column slice": (a[True, 3:290], host[:, 3:290]), "reversed": (a[True, ::-1], host[:, ::-1]),
             "row stride": (a[::3, True], host[::3, :])}
    for what, (view, ref) in cases.items():
        for axis in (0, 1):
            assert np.array_equal(view.cumsum(axis=axis).to_numpy(), np.cumsum(ref, axis=axis)), (what, axis)


@pytest.mark.parametrize("n", [64 * 4096, 64 * 4096 + 1, (1 << 22) + 5, 3_000_017])
def test_long_flat_scans(n):
    """Flat runs of 64 tiles and more (the three-launch plan): exact for integers, NaN rules kept, strided and reversed runs."""
    import cumo_b200 as xp

    rng = np.random.default_rng(n)
    host = rng.integers(-9, 10, size=n).astype(np.int64)
    a = xp.Int64.from_numpy(host)
    assert np.array_equal(a.cumsum().to_numpy(), np.cumsum(host))
    assert np.array_equal(a[::-1].cumsum().to_numpy(), np.cumsum(host[::-1]))
    h32 = host.astype(np.int32)
    assert np.array_equal(xp.Int32.from_numpy(h32).cumsum().to_numpy(), np.cumsum(h32, dtype=np.int32))
    wide = xp.Int32.from_numpy(np.repeat(h32[: n // 2], 2))[::2]                       # a strided run
    assert np.array_equal(wide.cumsum().to_numpy(), np.cumsum(h32[: n // 2], dtype=np.int32))
    f = (rng.integers(-64, 65, size=n) / 8.0).astype(np.float32)
    f[::4099] = np.nan
    got = xp.SFloat.from_numpy(f).cumsum(nan=True).to_numpy()
    want = np.cumsum(np.where(np.isnan(f), 0, f).astype(np.float64))
    seen = np.cumsum(~np.isnan(f)) > 0
    assert np.array_equal(np.isnan(got), ~seen) and np.allclose(got[seen], want[seen], rtol=0, atol=1e-5 * np.abs(f[~np.isnan(f)]).sum())
    ones = np.where(rng.random(n) < 0.001, 2.0, 1.0)
    ones[rng.random(n) < 0.001] = 0.5
    assert np.allclose(xp.DFloat.from_numpy(ones).cumprod().to_numpy(), np.cumprod(ones), rtol=1e-12)
