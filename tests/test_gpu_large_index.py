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
