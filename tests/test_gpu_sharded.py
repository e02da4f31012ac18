"""Row-sharded reductions on the CUDA backend: one rank always, two NCCL ranks when the box has two GPUs."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def check_rank(comm, xp, ox):
    """Shared body: every rank builds the same seeded host data, shards it, and compares with the oracle on the whole."""
    from cumo_b200.sharded import ShardedArray, partition

    rng = np.random.default_rng(3)
    n = 1_000_003
    vec = rng.uniform(0, 1, n).astype(np.float32)
    cut = partition(n, max(comm.world, 2), 1)[0]
    vec[[cut - 1, cut, 17]] = 2.0                    # the maximum three times, one pair across the shard boundary
    vec[[cut - 2, cut + 5, n - 1]] = -1.0
    sv = ShardedArray.scatter_from_numpy(comm, xp.SFloat, vec)
    ref64 = float(vec.astype(np.float64).sum())
    assert abs(sv.sum().extract() - ref64) <= 1e-5 * ref64
    assert abs(sv.mean().extract() - ref64 / n) <= 1e-5 * ref64 / n
    assert sv.max().extract() == 2.0 and sv.min().extract() == -1.0
    assert sv.argmax().extract() == 17
    assert sv.argmin().extract() == cut - 2
    assert sv.max_index().extract() == 17
    nanv = vec.copy()
    nanv[cut + 3] = np.nan
    sn = ShardedArray.scatter_from_numpy(comm, xp.SFloat, nanv)
    assert sn.argmax(nan=True).extract() == cut + 3
    assert sn.argmax().extract() == 17
    assert np.isnan(sn.sum().extract())

    mat = rng.integers(-1000, 1000, size=(4099, 257)).astype(np.int32)
    mat[[3, 3000], 5] = 5000
    sm = ShardedArray.scatter_from_numpy(comm, xp.Int32, mat)
    fm = ox.Int32.cast(mat)
    assert sm.sum().extract() == int(mat.astype(np.int64).sum())
    assert sm.sum(axis=0).to_a() == fm.sum(axis=0).to_a()
    assert sm.max(axis=0).to_a() == fm.max(axis=0).to_a()
    assert sm.argmax(axis=0).to_a() == fm.argmax(axis=0).to_a()
    assert sm.max_index(axis=0).to_a() == fm.max_index(axis=0).to_a()
    start, count = partition(4099, comm.world, comm.rank)
    assert sm.max_index(axis=1).local.to_a() == fm.max_index(axis=1).to_a()[start:start + count]
    assert ((sm * 3 + sm) % 7).local.to_a() == ((fm * 3 + fm) % 7).to_a()[start:start + count]
    assert (sm > 0).count_true().extract() == int((mat > 0).sum())
    fmat = rng.standard_normal((4099, 257))
    sd = ShardedArray.scatter_from_numpy(comm, xp.DFloat, fmat)
    got = np.array(sd.sum(axis=0).to_a())
    assert np.all(np.abs(got - fmat.sum(axis=0)) <= 1e-12 * np.abs(fmat).sum(axis=0))

    # k-means assignment: points sharded by rows, centroids replicated, per-cluster counts all-reduced
    from cumo_b200 import kmeans
    from oracle import cumo_oracle as orc

    k, d, npts = 256, 64, 30_011
    centres = (rng.standard_normal((k, d)) * 4).astype(np.float32)
    pts = (centres[rng.integers(0, k, npts)] + rng.standard_normal((npts, d))).astype(np.float32)
    want, best, second = orc.kmeans_assign(pts, centres)
    start, count = partition(npts, comm.world, comm.rank)
    for algo in ("tensor", "cores"):
        labels, counts = kmeans.assign_sharded(comm, xp.SFloat.from_numpy(pts[start:start + count]), xp.SFloat.from_numpy(centres), algo=algo)
        got = labels.to_numpy()
        flips = np.nonzero(got != want[start:start + count])[0] + start
        scale = np.abs(best) + (centres.astype(np.float64) ** 2).sum(axis=1).max()
        assert np.all((second - best)[flips] <= 1e-5 * scale[flips])
        if len(flips) == 0:          # (every rank sees the same seeded data; a near-tie flip on another rank can move one count)
            diff = np.abs(counts.to_numpy().astype(np.int64) - np.bincount(want, minlength=k))
            assert diff.sum() <= 2
        assert int(counts.to_numpy().sum()) == npts


def test_sharded_reductions_one_rank(xp_gpu):
    from cumo_b200.sharded import Comm
    from oracle_narray import OracleXP

    check_rank(Comm(xp_gpu), xp_gpu, OracleXP)


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import cumo_b200 as xp
        from cumo_b200.sharded import Comm
        from oracle_narray import OracleXP

        check_rank(Comm(xp), xp, OracleXP)
        torch.cuda.synchronize()
        (Path(out_dir) / f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_sharded_reductions_two_nccl_ranks(tmp_path):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
