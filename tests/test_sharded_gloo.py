"""The multi-rank path (partition, partial -> collective -> rank-order fold, index fix-ups)
run as two gloo ranks on the CPU, with the CPU oracle standing in for the array backend."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from cumo_b200.sharded import partition  # noqa: E402


def test_partition_covers_rows_contiguously():
    for n in (0, 1, 7, 8, 9, 65536, 2 ** 28 + 3):
        for world in (1, 2, 3, 4, 8):
            parts = [partition(n, world, r) for r in range(world)]
            assert parts[0][0] == 0
            assert sum(c for _, c in parts) == n
            for (s0, c0), (s1, _) in zip(parts, parts[1:]):
                assert s1 == s0 + c0
            assert max(c for _, c in parts) - min(c for _, c in parts) <= 1


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle_narray import OracleXP as xp
        from cumo_b200.sharded import Comm, ShardedArray
        comm = Comm(xp)
        rng = np.random.default_rng(0)
        n = 100_001
        vec = rng.uniform(0, 1, n).astype(np.float32)
        # duplicates of the extremes, one pair straddling the shard boundary
        cut = partition(n, world, 1)[0]
        vec[[cut - 1, cut, 17]] = 2.0
        vec[[cut - 2, cut + 5, n - 1]] = -1.0
        sv = ShardedArray.scatter_from_numpy(comm, xp.SFloat, vec)
        full = xp.SFloat.cast(vec)
        ref64 = float(vec.astype(np.float64).sum())
        assert abs(sv.sum().extract() - ref64) <= 1e-5 * ref64
        assert abs(sv.mean().extract() - ref64 / n) <= 1e-5 * ref64 / n
        assert sv.max().extract() == 2.0 and sv.min().extract() == -1.0
        assert sv.argmax().extract() == full.argmax().extract() == 17
        assert sv.argmin().extract() == full.argmin().extract() == cut - 2
        assert sv.max_index().extract() == 17
        nanv = vec.copy()
        nanv[cut + 3] = np.nan
        sn = ShardedArray.scatter_from_numpy(comm, xp.SFloat, nanv)
        assert sn.argmax(nan=True).extract() == cut + 3
        assert sn.argmax().extract() == 17
        assert np.isnan(sn.sum().extract())
        assert abs(sn.sum(nan=True).extract() - float(np.nansum(nanv.astype(np.float64)))) <= 1e-5 * ref64

        mat = rng.integers(-1000, 1000, size=(1001, 33)).astype(np.int32)
        mat[[3, 700], 5] = 5000                    # a tie across ranks in column 5
        sm = ShardedArray.scatter_from_numpy(comm, xp.Int32, mat)
        fm = xp.Int32.cast(mat)
        assert sm.sum().extract() == int(mat.astype(np.int64).sum())
        assert sm.sum(axis=0).to_a() == fm.sum(axis=0).to_a()
        assert sm.max(axis=0).to_a() == fm.max(axis=0).to_a()
        assert sm.argmax(axis=0).to_a() == fm.argmax(axis=0).to_a()
        assert sm.max_index(axis=0).to_a() == fm.max_index(axis=0).to_a()
        assert sm.argmin(axis=0).to_a() == fm.argmin(axis=0).to_a()
        # axis 1 is local; flat indices get the shard's element offset
        start, count = partition(1001, world, rank)
        assert sm.max_index(axis=1).local.to_a() == fm.max_index(axis=1).to_a()[start:start + count]
        assert sm.sum(axis=1).local.to_a() == fm.sum(axis=1).to_a()[start:start + count]
        # elementwise sweep and a Bit count
        expr = (sm * 3 + sm) % 7
        want = ((fm * 3 + fm) % 7).to_a()[start:start + count]
        assert expr.local.to_a() == want
        assert (sm > 0).count_true().extract() == int((mat > 0).sum())
        # fewer rows than ranks: every rank refuses from the global shape alone, before any collective
        try:
            ShardedArray.scatter_from_numpy(comm, xp.SFloat, np.zeros((world - 1, 3), np.float32))
            raise AssertionError("a shard without rows was accepted")
        except ValueError as e:
            assert "at least one row" in str(e)
        dist.barrier()                               # all ranks got here: nobody is stuck in a collective
        (Path(out_dir) / f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_agree_with_one_process(tmp_path):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
