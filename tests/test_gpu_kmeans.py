"""k-means assignment: the fused kernel against a float64 restatement of the reference's formulation.

Labels must agree except where float32 rounding can legitimately decide a near-tie: a disagreement is
accepted only if the float64 gap between the winner and the runner-up is below 1e-5 of the distance
scale, and such flips must stay rare.  Counts are exact given the labels.
"""
import numpy as np
import pytest

from oracle import cumo_oracle as orc

pytestmark = pytest.mark.gpu


def mixture(rng, n, d, k):
    centres = (rng.standard_normal((k, d)) * 4).astype(np.float32)
    which = rng.integers(0, k, n)
    return (centres[which] + rng.standard_normal((n, d))).astype(np.float32), centres


def check(xp_gpu, x, c, algo="auto"):
    from cumo_b200 import kmeans

    labels, counts, dist = kmeans.assign(xp_gpu.SFloat.from_numpy(x), xp_gpu.SFloat.from_numpy(c), want_min_dist=True, algo=algo)
    got = labels.to_numpy()
    want, best, second = orc.kmeans_assign(x, c)
    flips = np.nonzero(got != want)[0]
    scale = np.abs(best) + (c.astype(np.float64) ** 2).sum(axis=1).max()
    assert np.all((second - best)[flips] <= 1e-5 * scale[flips]), "a disagreement that is not a near-tie"
    assert len(flips) <= max(2, 1e-4 * len(got)), f"{len(flips)} flips in {len(got)}"
    assert np.array_equal(counts.to_numpy(), np.bincount(got, minlength=c.shape[0]).astype(np.uint64))
    assert np.all(np.abs(dist.to_numpy() - best) <= 1e-4 * scale)
    return len(flips)


@pytest.mark.parametrize("n,d,k", [(1, 64, 256), (127, 64, 256), (1000, 64, 256), (100_003, 64, 256), (5000, 16, 7), (5000, 128, 120), (3000, 32, 600), (4096, 4, 1)])
@pytest.mark.parametrize("algo", ["cores", "tensor"])
def test_kmeans_assign_matches_float64(xp_gpu, n, d, k, algo):
    from cumo_b200 import kmeans

    if algo == "tensor" and not kmeans.tensor_core_form_fits(d, k):
        pytest.skip("shape outside the tensor-core form")
    rng = np.random.default_rng(n + d + k)
    x, c = mixture(rng, n, d, k)
    check(xp_gpu, x, c, algo)


@pytest.mark.parametrize("n,d,k", [(128, 32, 16), (129, 32, 1), (70_000, 32, 250), (20_000, 96, 100), (40_000, 64, 33), (148 * 128 * 3 + 5, 64, 256)])
def test_kmeans_tensor_core_form_shapes(xp_gpu, n, d, k):
    """Shapes that exercise the tensor-core form's edges: one K-block, padded centroid counts,
    a ragged last tile, more tiles than CTAs."""
    rng = np.random.default_rng(7 * n + d + k)
    x, c = mixture(rng, n, d, k)
    check(xp_gpu, x, c, "tensor")


def test_kmeans_tensor_core_form_refuses_other_shapes(xp_gpu):
    from cumo_b200 import kmeans

    with pytest.raises(xp_gpu.CumoError, match="multiple of 32"):
        kmeans.assign(xp_gpu.SFloat.zeros(256, 48), xp_gpu.SFloat.zeros(8, 48), algo="tensor")
    with pytest.raises(xp_gpu.CumoError, match="shared memory"):
        kmeans.assign(xp_gpu.SFloat.zeros(256, 128), xp_gpu.SFloat.zeros(256, 128), algo="tensor")


def test_kmeans_refuses_a_table_that_does_not_fit_shared_memory(xp_gpu):
    from cumo_b200 import kmeans

    x = xp_gpu.SFloat.zeros(256, 128)
    c = xp_gpu.SFloat.zeros(300, 128)
    with pytest.raises(xp_gpu.CumoError, match="shared memory"):
        kmeans.assign(x, c)


@pytest.mark.parametrize("algo", ["cores", "tensor"])
def test_kmeans_ties_take_the_lowest_index(xp_gpu, algo):
    from cumo_b200 import kmeans

    rng = np.random.default_rng(0)
    c = rng.standard_normal((256, 64)).astype(np.float32)
    c[200] = c[17]                       # two identical centroids: the earlier one must win
    c[130] = c[17]
    x = np.repeat(c[17][None, :], 300, axis=0) + (rng.standard_normal((300, 64)) * 1e-3).astype(np.float32)
    labels, counts = kmeans.assign(xp_gpu.SFloat.from_numpy(x), xp_gpu.SFloat.from_numpy(c), algo=algo)
    assert np.all(labels.to_numpy() == 17)
    assert counts.to_numpy()[17] == 300 and counts.to_numpy().sum() == 300


@pytest.mark.parametrize("algo", ["cores", "tensor"])
def test_kmeans_baseline_config_sample(xp_gpu, algo):
    """BASELINE config 4 at full size on the device (2^24 points, 64-D, 256 centres, a seeded mixture);
    the float64 check runs on every 97th point, the counts on all of them."""
    import torch
    from cumo_b200 import kmeans

    g = torch.Generator(device="cuda").manual_seed(4)
    n, d, k = 1 << 24, 64, 256
    centres = torch.randn(k, d, device="cuda", generator=g) * 4
    which = torch.randint(0, k, (n,), device="cuda", generator=g)
    x = centres[which] + torch.randn(n, d, device="cuda", generator=g)
    del which
    labels, counts = kmeans.assign(xp_gpu.SFloat.from_torch(x), xp_gpu.SFloat.from_torch(centres), algo=algo)
    got = labels.to_numpy()
    assert np.array_equal(counts.to_numpy(), np.bincount(got, minlength=k).astype(np.uint64))
    sample = slice(0, n, 97)
    hx, hc = x[sample].cpu().numpy(), centres.cpu().numpy()
    want, best, second = orc.kmeans_assign(hx, hc)
    flips = np.nonzero(got[sample] != want)[0]
    scale = np.abs(best) + (hc.astype(np.float64) ** 2).sum(axis=1).max()
    assert np.all((second - best)[flips] <= 1e-5 * scale[flips])
    assert len(flips) <= 1e-4 * len(want)
