"""bincount of one unweighted run: counted and sized in one pass when the values are small (the probe's shared-memory range,
its global-atomic range, and the fall back to the output-sized kernel beyond it), against numpy."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("top", [0, 1, 255, 1023, 1024, 1025, 8191, 8192, 8193, 100_000])
@pytest.mark.parametrize("n", [1, 4097, 300_001])
def test_counts_match_numpy_around_the_probe_ranges(top, n):
    import cumo_b200 as xp

    rng = np.random.default_rng(top + n)
    for T, dt in ((xp.Int32, np.int32), (xp.Int64, np.int64)):
        host = rng.integers(0, top + 1, size=n).astype(dt)
        host[rng.integers(0, n)] = top                                       # the largest value is present
        got = T.from_numpy(host).bincount().to_numpy()
        assert np.array_equal(got, np.bincount(host).astype(got.dtype))
        got = T.from_numpy(host).bincount(minlength=top + 7).to_numpy()
        assert np.array_equal(got, np.bincount(host, minlength=top + 7).astype(got.dtype))
        view = T.from_numpy(np.repeat(host, 2))[::-2]                         # a reversed, strided run
        assert np.array_equal(view.bincount().to_numpy(), np.bincount(host).astype(got.dtype))


def test_negative_items_are_refused_and_minlength_beyond_the_probe_is_kept():
    import cumo_b200 as xp

    a = xp.Int32.from_numpy(np.array([3, 1, -2, 5], dtype=np.int32))
    with pytest.raises(ValueError):
        a.bincount()
    b = xp.Int64.from_numpy(np.array([3, 1, 2, 5] * 1000, dtype=np.int64))
    got = b.bincount(minlength=20_000).to_numpy()
    assert got.shape == (20_000,) and np.array_equal(got[:6], [0, 1000, 1000, 1000, 0, 1000]) and not got[6:].any()
