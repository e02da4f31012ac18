"""Arrays past 2^32 elements: offsets, tile counts and index results must be 64-bit end to end.
(accum_index.c:100-119: the index type becomes Int64 when the size exceeds 2^32-1.)"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_elementwise_and_reductions_past_2_to_32_elements(xp_gpu):
    import torch

    if torch.cuda.mem_get_info()[0] < 60 * (1 << 30):
        pytest.skip("needs 60 GiB of free device memory")
    n = (1 << 32) + 4099
    t = torch.ones(n, device="cuda")
    t[(1 << 32) + 17] = 3.0                       # the maximum, past the 32-bit boundary
    t[(1 << 32) + 19] = 3.0                       # and a later duplicate: the first one must win
    t[5] = -2.0
    a = xp_gpu.SFloat.from_torch(t)
    idx = a.argmax()
    assert type(idx).__name__ == "Int64"
    assert idx.extract() == (1 << 32) + 17
    assert a.max_index().extract() == (1 << 32) + 17
    assert a.argmin().extract() == 5
    total = a.sum().extract()
    assert abs(total - (n + 4.0 - 3.0)) <= 1e-5 * n
    b = a + a
    back = b[(1 << 32) + 10:(1 << 32) + 24].to_numpy()
    want = np.full(14, 2.0, dtype=np.float32)
    want[7] = want[9] = 6.0
    assert np.array_equal(back, want)
    assert (b > 5.0).count_true().extract() == 2
    pos = (b > 5.0).where()
    assert type(pos).__name__ == "Int64"
    assert pos.to_a() == [(1 << 32) + 17, (1 << 32) + 19]


def test_two_dimensional_array_past_2_to_32_elements(xp_gpu):
    """(2^20 + 3) x 4100 floats: broadcast add, both axis sums, flat max_index per row (Int64), argmax per column.
    Checked against torch on the same device buffers (the CPU oracle would need minutes at this size)."""
    import torch

    if torch.cuda.mem_get_info()[0] < 80 * (1 << 30):
        pytest.skip("needs 80 GiB of free device memory")
    r, c = (1 << 20) + 3, 4100
    g = torch.Generator(device="cuda").manual_seed(11)
    t = torch.rand(r, c, device="cuda", generator=g)
    t[r - 2, 7] = 5.0                              # flat offset (r-2)*4100 + 7 > 2^32
    t[r - 2, 9] = 5.0
    t[3, 4000] = 6.0
    a = xp_gpu.SFloat.from_torch(t)
    col = xp_gpu.SFloat.from_torch(torch.arange(r, device="cuda", dtype=torch.float32).reshape(r, 1))
    s = a + col
    got = s[r - 3:r, 5:11].to_numpy()
    want = (t[r - 3:r, 5:11] + torch.arange(r - 3, r, device="cuda", dtype=torch.float32).reshape(3, 1)).cpu().numpy()
    assert np.array_equal(got, want)
    del s
    mi = a.max_index(axis=1)
    assert type(mi).__name__ == "Int64"
    flat = mi.to_numpy()
    assert flat[r - 2] == (r - 2) * c + 7 and flat[3] == 3 * c + 4000
    assert np.array_equal(flat, (t.argmax(dim=1) + torch.arange(r, device="cuda") * c).cpu().numpy())
    assert np.array_equal(a.argmax(axis=0).to_numpy()[[7, 9, 4000]], np.array([r - 2, r - 2, 3]))
    row_sums = a.sum(axis=1).to_numpy().astype(np.float64)
    ref_rows = t.sum(dim=1, dtype=torch.float64).cpu().numpy()
    assert np.all(np.abs(row_sums - ref_rows) <= 1e-5 * ref_rows)
    col_sums = a.sum(axis=0).to_numpy().astype(np.float64)
    ref_cols = t.sum(dim=0, dtype=torch.float64).cpu().numpy()
    assert np.all(np.abs(col_sums - ref_cols) <= 1e-5 * ref_cols)
