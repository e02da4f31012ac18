"""The BASELINE configurations at their full sizes.

Where the CPU oracle finishes in seconds it is the yardstick itself (bit-exact for integers, indices,
counts, comparisons; a few ulp for exp); for the float sums the yardstick is a float64 reference
(fp32 <= 1e-5, fp64 <= 1e-12 relative) plus size-independent properties: the sum of the row sums and of
the column sums equals the full sum, and extremes planted as exact duplicates are found at their
first occurrence (one pair straddles a 32 KiB segment boundary, i.e. two CTAs).
"""
import numpy as np
import pytest

from oracle import cumo_oracle as orc
from oracle_narray import OracleXP as ox

pytestmark = pytest.mark.gpu


def test_config0_sfloat_4096_chain(xp_gpu):
    rng = np.random.default_rng(0)
    ha = rng.uniform(-1, 1, (4096, 4096)).astype(np.float32)
    hb = rng.uniform(-1, 1, (4096, 4096)).astype(np.float32)
    a, b = xp_gpu.SFloat.from_numpy(ha), xp_gpu.SFloat.from_numpy(hb)
    oa, ob = ox.SFloat.cast(ha), ox.SFloat.cast(hb)
    s1 = a.sum(axis=1)
    ref_s1 = ha.astype(np.float64).sum(axis=1)
    assert np.all(np.abs(s1.to_numpy() - ref_s1) <= 1e-5 * np.abs(ha).astype(np.float64).sum(axis=1))
    # the same row sums on both sides from here on, so that everything after is exactly comparable
    col = s1.reshape(4096, 1)
    ocol = ox.SFloat.cast(s1.to_numpy()).reshape(4096, 1)
    c = a * b + col
    oc = oa * ob + ocol
    assert np.array_equal(c.to_numpy(), oc.to_numpy())
    hc = oc.to_numpy().astype(np.float64)
    assert np.all(np.abs(c.sum(axis=0).to_numpy() - hc.sum(axis=0)) <= 1e-5 * np.abs(hc).sum(axis=0))
    assert np.array_equal(c.max_index(axis=1).to_numpy(), oc.max_index(axis=1).to_numpy())


def test_config1_broadcast_exp_chain(xp_gpu):
    rng = np.random.default_rng(1)
    hx = rng.standard_normal((8192, 1)).astype(np.float32)
    hy = rng.standard_normal((1, 16384)).astype(np.float32)
    x, y = xp_gpu.SFloat.from_numpy(hx), xp_gpu.SFloat.from_numpy(hy)
    t = x + y
    assert np.array_equal(t.to_numpy(), hx + hy)                     # one IEEE addition per element
    r = (xp_gpu.NMath.exp(t) * 0.5).to_numpy()
    want = (ox.NMath.exp(ox.SFloat.cast(hx) + ox.SFloat.cast(hy)) * 0.5).to_numpy()
    assert r.shape == (8192, 16384)
    assert np.allclose(r, want, rtol=2e-6, atol=0.0)                 # CUDA expf vs libm exp through double


@pytest.mark.parametrize("tname,tol", [("SFloat", 1e-5), ("DFloat", 1e-12)])
def test_config2_reductions(xp_gpu, tname, tol):
    dt = np.float32 if tname == "SFloat" else np.float64
    rng = np.random.default_rng(2)
    n = 1 << 28
    host = rng.random(n, dtype=dt)
    seg = (32 << 10) // host.itemsize                                # elements per CTA segment of a long row
    hi_pos = [5 * seg - 1, 5 * seg, n - 3]                           # a pair across two CTAs, and a late one
    lo_pos = [7 * seg + 11, 9 * seg + 1, n - 1]
    host[hi_pos] = 2.0
    host[lo_pos] = -1.0
    T = getattr(xp_gpu, tname)
    v = T.from_numpy(host)
    ref = float(host.sum(dtype=np.float64)) if dt == np.float32 else orc.sum_f64ref(host)
    assert abs(v.sum().extract() - ref) <= tol * ref
    assert abs(v.mean().extract() - ref / n) <= tol * ref / n
    assert v.max().extract() == 2.0 and v.min().extract() == -1.0
    assert v.argmax().extract() == hi_pos[0] and v.argmin().extract() == lo_pos[0]
    assert v.max_index().extract() == hi_pos[0] and v.min_index().extract() == lo_pos[0]
    # (65536, 4096): axis 0 is the strided, transposed-style reduction, axis 1 the contiguous one
    m = v.reshape(65536, 4096)
    hm = host.reshape(65536, 4096)
    s0, s1 = m.sum(axis=0).to_numpy().astype(np.float64), m.sum(axis=1).to_numpy().astype(np.float64)
    assert np.all(np.abs(s0 - hm.sum(axis=0, dtype=np.float64)) <= tol * np.abs(hm).sum(axis=0, dtype=np.float64))
    assert np.all(np.abs(s1 - hm.sum(axis=1, dtype=np.float64)) <= tol * np.abs(hm).sum(axis=1, dtype=np.float64))
    assert abs(s0.sum() - ref) <= tol * ref and abs(s1.sum() - ref) <= tol * ref
    assert np.array_equal(m.max(axis=0).to_numpy(), hm.max(axis=0))
    assert np.array_equal(m.min(axis=1).to_numpy(), hm.min(axis=1))
    assert np.array_equal(m.argmax(axis=0).to_numpy(), hm.argmax(axis=0).astype(np.int32))
    assert np.array_equal(m.argmax(axis=1).to_numpy(), hm.argmax(axis=1).astype(np.int32))
    assert np.array_equal(m.argmin(axis=0).to_numpy(), hm.argmin(axis=0).astype(np.int32))
    mean1 = m.mean(axis=1).to_numpy().astype(np.float64)
    assert np.all(np.abs(mean1 - hm.mean(axis=1, dtype=np.float64)) <= tol)


def test_config3_int32_path(xp_gpu):
    rng = np.random.default_rng(3)
    n = 1 << 27
    ha = rng.integers(-(1 << 20), 1 << 20, n, dtype=np.int32)
    hb = rng.integers(-(1 << 20), 1 << 20, n, dtype=np.int32)
    a, b = xp_gpu.Int32.from_numpy(ha), xp_gpu.Int32.from_numpy(hb)
    got = ((a * 3 + b) % 7).to_numpy()
    want = ((ox.Int32.cast(ha) * 3 + ox.Int32.cast(hb)) % 7).to_numpy()          # C truncation: results in -6..6
    assert np.array_equal(got, want)
    assert got.min() >= -6 and got.max() <= 6
    mask = a > 0
    assert np.array_equal(mask.to_numpy(), ha > 0)
    assert mask.count_true().extract() == int((ha > 0).sum())
    assert mask.count_false().extract() == int((ha <= 0).sum())
    m = a.reshape(32768, 4096)
    hm = ha.reshape(32768, 4096)
    want_idx = ox.Int32.cast(hm).max_index(axis=1).to_numpy()
    assert np.array_equal(m.max_index(axis=1).to_numpy(), want_idx)
    assert np.array_equal(want_idx, (hm.argmax(axis=1) + np.arange(32768) * 4096).astype(np.int32))
    assert a.sum().extract() == int(ha.sum(dtype=np.int64))
