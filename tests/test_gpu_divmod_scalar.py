"""Integer `a / s` and `a % s` with a host scalar on the right run in a kernel that multiplies by a precomputed
reciprocal instead of dividing.  Checked bit for bit against C's truncating division computed with Python integers
(what the reference's `x / y` and `x % y` in binary_kernel.cu compute) and against the oracle, for both widths, both
signs, the extreme values, divisors up to the type's limits, ragged lengths, and views (which take the general path)."""
import numpy as np
import pytest

from oracle_narray import OracleXP as ox

pytestmark = pytest.mark.gpu


def c_divmod(x, d, bits):
    q = abs(x) // abs(d)
    if (x < 0) != (d < 0):
        q = -q
    r = x - q * d
    lo, hi = -(1 << (bits - 1)), (1 << (bits - 1)) - 1
    assert lo <= q <= hi and lo <= r <= hi
    return q, r


@pytest.mark.parametrize("tname,bits", [("Int32", 32), ("Int64", 64)])
def test_division_and_remainder_by_a_scalar(xp_gpu, tname, bits):
    rng = np.random.default_rng(bits)
    dt = np.int32 if bits == 32 else np.int64
    lo, hi = -(1 << (bits - 1)), (1 << (bits - 1)) - 1
    special = [0, 1, -1, 2, -2, 6, 7, 8, -7, lo, lo + 1, hi, hi - 1, 1 << (bits - 2), -(1 << (bits - 2))]
    n = 1000 * 4 + 3                                          # whole packets plus a ragged end
    h = np.concatenate([np.array(special, dtype=dt), rng.integers(lo, hi, n - len(special), dtype=dt, endpoint=True)])
    g = getattr(xp_gpu, tname).from_numpy(h)
    o = getattr(ox, tname).cast(h)
    divisors = [1, 2, 3, 7, -7, 10, -10, 641, 4096, -4096, 1000003, hi, -hi, lo, (1 << (bits - 2)) + 1, 6700417]
    for d in divisors:
        want = [c_divmod(int(x), d, bits) for x in h]
        wq = np.array([w[0] for w in want], dtype=dt)
        wr = np.array([w[1] for w in want], dtype=dt)
        assert np.array_equal((g / d).to_numpy(), wq), d
        assert np.array_equal((g % d).to_numpy(), wr), d
        assert np.array_equal((g % d).to_numpy(), (o % d).to_numpy()), d
        assert np.array_equal((g / d).to_numpy(), (o / d).to_numpy()), d


@pytest.mark.parametrize("tname", ["Int32", "Int64"])
def test_views_scalar_on_the_left_and_special_divisors_keep_their_meaning(xp_gpu, tname):
    rng = np.random.default_rng(9)
    dt = np.int32 if tname == "Int32" else np.int64
    h = rng.integers(-10**6, 10**6, (64, 50), dtype=dt)
    h[h == 0] = 5
    g, o = getattr(xp_gpu, tname).from_numpy(h), getattr(ox, tname).cast(h)
    assert np.array_equal((g[:, 1:] % 7).to_numpy(), (o[:, 1:] % 7).to_numpy())          # a view: general path
    assert np.array_equal((g.transpose() / 9).to_numpy(), (o.transpose() / 9).to_numpy())
    assert np.array_equal((1000 % g).to_numpy(), (1000 % o).to_numpy())                  # scalar on the left
    assert np.array_equal((g % -1).to_numpy(), np.zeros_like(h))
    assert np.array_equal((g / -1).to_numpy(), -h)
    with pytest.raises(ZeroDivisionError):
        (g % 0).to_numpy()
    with pytest.raises(ZeroDivisionError):
        (g / 0).to_numpy()
