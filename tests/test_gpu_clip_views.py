"""clip on operand layouts that take the row, row-share, tile and copy-engine tile kernels (large enough to leave the generic
kernel), against numpy: the two numeric bounds ride in the kernels' two scalar arguments, so every kernel family must pass
both on."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tname,dt", [("SFloat", np.float32), ("DFloat", np.float64), ("Int32", np.int32), ("Int64", np.int64)])
def test_clip_forms_on_large_views(tname, dt):
    import cumo_b200 as xp

    T = getattr(xp, tname)
    rng = np.random.default_rng(len(tname))
    host = rng.integers(-50, 51, size=(1024, 768)).astype(dt)
    a = T.from_numpy(host)
    lo, hi = -7, 12
    views = {
        "whole": (a, host),
        "transposed": (a.transpose(), host.T),
        "column slice": (a[True, 64:704], host[:, 64:704]),
        "row stride": (a[::2, True], host[::2, :]),
        "reversed": (a[True, ::-1], host[:, ::-1]),
    }
    for what, (v, h) in views.items():
        assert np.array_equal(v.clip(lo, hi).to_numpy(), np.clip(h, lo, hi)), (what, "clip")
        assert np.array_equal(v.clip(lo, None).to_numpy(), np.maximum(h, lo)), (what, "clip min")
        assert np.array_equal(v.clip(None, hi).to_numpy(), np.minimum(h, hi)), (what, "clip max")
    # array bounds: a full array against a transposed operand (tile kernels), a row vector and a column (row-share kernels)
    b = T.from_numpy(np.ascontiguousarray(host.T))
    assert np.array_equal(a.clip(b.transpose() - 3, None).to_numpy(), np.maximum(host, host - 3))
    row = rng.integers(-5, 6, size=(1, 768)).astype(dt)
    col = rng.integers(-5, 6, size=(1024, 1)).astype(dt)
    assert np.array_equal(a.clip(T.from_numpy(row), None).to_numpy(), np.maximum(host, row))
    assert np.array_equal(a.clip(None, T.from_numpy(col)).to_numpy(), np.minimum(host, col))
    assert np.array_equal(a.clip(T.from_numpy(row) - 20, T.from_numpy(col) + 20).to_numpy(), np.clip(host, row - 20, col + 20))
    # in place on a view
    c = T.from_numpy(host.copy())
    c[True, 64:704].inplace().clip(lo, hi)
    want = host.copy()
    want[:, 64:704] = np.clip(want[:, 64:704], lo, hi)
    assert np.array_equal(c.to_numpy(), want)
    with pytest.raises(xp.OperationError):
        a.clip(T.from_numpy(col) + 100, T.from_numpy(row) - 100)
