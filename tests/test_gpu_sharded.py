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
    assert sn.max().extract() == 2.0 and sn.min().extract() == -1.0          # plain form: a NaN loses
    assert np.isnan(sn.max(nan=True).extract()) and np.isnan(sn.min(nan=True).extract())

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


def _worker(rank, world, port, out_dir, peer):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", CB200_PEER_EXCHANGE=peer)
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

        comm = Comm(xp)
        check_rank(comm, xp, OracleXP)
        comm.check()                                   # no bounded wait of a peer exchange ran out
        torch.cuda.synchronize()
        (Path(out_dir) / f"ok{rank}").write_text("peer" if comm.peer is not None else "nccl")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("peer", ["1", "0"])
def test_sharded_reductions_two_nccl_ranks(tmp_path, peer):
    """Two ranks on two GPUs; the partials are gathered through peer memory (peer == "1", when the GPUs can reach each
    other's memory) or by NCCL's all_gather."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path), peer), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
    used = {(tmp_path / f"ok{r}").read_text() for r in (0, 1)}
    assert len(used) == 1                              # both ranks made the same choice
    if peer == "0":
        assert used == {"nccl"}


def _exchange_setup(world, slot):
    import ctypes

    import torch
    from cumo_b200 import _lib

    lib = _lib.load()
    base = ctypes.c_void_p()
    handle = (ctypes.c_ubyte * 64)()
    assert lib.cb200_peer_buffer_create(slot, world, ctypes.byref(base), handle) == 0
    bases = (ctypes.c_void_p * world)(*([base.value] * world))     # every "rank" is this GPU: no second process needed
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    return lib, base, bases, status


def test_peer_exchange_kernel_with_a_message_made_on_the_host(xp_gpu):
    """One GPU plays rank 0 of two.  Rank 1's partial and flag are written into the buffer from the host beforehand, so
    the kernel finds its peer's flag already raised: nothing waits for another kernel."""
    import ctypes

    import torch

    world, slot, n = 2, 64 << 10, 12_000                # three CTAs' worth of bytes
    lib, base, bases, status = _exchange_setup(world, slot)
    try:
        seq = 1
        mine = torch.arange(n, dtype=torch.float32, device="cuda")
        theirs = torch.arange(n, dtype=torch.float32, device="cuda") * -2
        from cumo_b200.narray import UInt32
        total = lib.cb200_peer_buffer_bytes(slot, world)
        whole = torch.as_tensor(UInt32.from_device_pointer(base.value, (total // 4,)), device="cuda").view(torch.uint8)   # the buffer, as torch sees it
        data_off = ((seq & 1) * world + 1) * slot                                   # slot [seq & 1][rank 1]
        whole[data_off:data_off + n * 4] = theirs.view(torch.uint8)
        flags = whole[2 * world * slot:].view(torch.int64).view(2, world, 16)
        flags[seq & 1, 1, :] = seq                                                   # rank 1's flags, for every CTA
        torch.cuda.synchronize()
        rc = lib.cb200_peer_exchange_kernel_launch(mine.data_ptr(), n * 4, bases, world, 0, slot, seq, 1 << 12, status.data_ptr())
        assert rc == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        got = whole[(seq & 1) * world * slot:][:world * slot].view(torch.float32).view(world, slot // 4).cpu().numpy()
        assert np.array_equal(got[0, :n], mine.cpu().numpy())
        assert np.array_equal(got[1, :n], theirs.cpu().numpy())
        # and the fold kernel reads it where the exchange left it
        out = xp_gpu.SFloat(n)
        lib.cb200_sfloat_rank_fold_sum_kernel_launch(base.value + (seq & 1) * world * slot, slot, world, n, 0.0, out.data_ptr)
        assert np.array_equal(out.to_numpy(), (mine + theirs).cpu().numpy())
    finally:
        torch.cuda.synchronize()
        lib.cb200_peer_buffer_destroy(base)


@pytest.mark.parametrize("op,tname", [("sum", "SFloat"), ("sum", "DFloat"), ("max", "SFloat"), ("min", "Int32"), ("max", "Int64")])
def test_fused_exchange_and_fold_with_a_message_made_on_the_host(xp_gpu, op, tname):
    """The one-kernel form (exchange + element-wise rank fold) as rank 0 of two on one GPU, rank 1's partial and flags
    written from the host beforehand; a ragged length so that the last packet and the last CTA are partial."""
    import torch
    from cumo_b200.narray import UInt32

    world, slot, n = 2, 64 << 10, 4099
    lib, base, bases, status = _exchange_setup(world, slot)
    try:
        seq = 3
        rng = np.random.default_rng(7)
        T = getattr(xp_gpu, tname)
        dt = {"SFloat": np.float32, "DFloat": np.float64, "Int32": np.int32, "Int64": np.int64}[tname]
        h_mine = (rng.standard_normal(n) * 100).astype(dt)
        h_theirs = (rng.standard_normal(n) * 100).astype(dt)
        if tname.endswith("Float") and op != "sum":
            h_mine[5], h_theirs[9], h_mine[11], h_theirs[11] = np.nan, np.nan, np.nan, np.nan
        mine = T.from_numpy(h_mine)
        total = lib.cb200_peer_buffer_bytes(slot, world)
        whole = torch.as_tensor(UInt32.from_device_pointer(base.value, (total // 4,)), device="cuda").view(torch.uint8)
        data_off = ((seq & 1) * world + 1) * slot
        whole[data_off:data_off + h_theirs.nbytes] = torch.from_numpy(h_theirs.view(np.uint8)).cuda()
        whole[2 * world * slot:].view(torch.int64).view(2, world, 16)[seq & 1, 1, :] = seq
        torch.cuda.synchronize()
        out = T(n)
        code = {"SFloat": 0, "DFloat": 1, "Int32": 2, "Int64": 3}[tname]
        rc = lib.cb200_peer_exchange_fold_kernel_launch(mine.data_ptr, code, {"sum": 0, "min": 1, "max": 2}[op], n, 0.0, 0, out.data_ptr,
                                                        bases, world, 0, slot, seq, 1 << 12, status.data_ptr())
        assert rc == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        got = out.to_numpy()
        if op == "sum":
            want = (h_mine.astype(np.float64) + h_theirs.astype(np.float64)).astype(dt)
        else:
            f = np.fmax if op == "max" else np.fmin          # the plain form: a NaN loses unless both are NaN
            want = f(h_mine, h_theirs)
        assert np.array_equal(got, want, equal_nan=True)
    finally:
        torch.cuda.synchronize()
        lib.cb200_peer_buffer_destroy(base)


@pytest.mark.parametrize("tname,n", [("SFloat", 4099), ("DFloat", 1), ("Int32", 6), ("Int64", 2050)])
def test_fused_exchange_and_index_merge_with_a_message_made_on_the_host(xp_gpu, tname, n):
    """The one-kernel form for index reductions as rank 0 of two on one GPU: rank 1's {index, value} partial and its flags
    come from the host.  Ties go to the lower index, a NaN loses (plain form), lengths that are not whole packets."""
    import torch
    from cumo_b200.narray import UInt32

    world, slot = 2, 64 << 10
    lib, base, bases, status = _exchange_setup(world, slot)
    try:
        seq = 2
        rng = np.random.default_rng(n)
        dt = {"SFloat": np.float32, "DFloat": np.float64, "Int32": np.int32, "Int64": np.int64}[tname]
        es = np.dtype(dt).itemsize
        v0 = rng.integers(-50, 50, n).astype(dt)
        v1 = rng.integers(-50, 50, n).astype(dt)
        i0 = rng.integers(0, 1000, n).astype(np.int64)
        i1 = rng.integers(1000, 2000, n).astype(np.int64)
        if tname.endswith("Float") and n > 8:
            v0[3], v1[5] = np.nan, np.nan
        val_off = (n * 8 + 15) // 16 * 16
        nbytes = val_off + (n * es + 15) // 16 * 16

        def pack(idx, val):
            b = np.zeros(nbytes, dtype=np.uint8)
            b[:n * 8] = idx.view(np.uint8)
            b[val_off:val_off + n * es] = val.view(np.uint8)
            return b
        mine = torch.from_numpy(pack(i0, v0)).cuda()
        total = lib.cb200_peer_buffer_bytes(slot, world)
        whole = torch.as_tensor(UInt32.from_device_pointer(base.value, (total // 4,)), device="cuda").view(torch.uint8)
        data_off = ((seq & 1) * world + 1) * slot
        whole[data_off:data_off + nbytes] = torch.from_numpy(pack(i1, v1)).cuda()
        whole[2 * world * slot:].view(torch.int64).view(2, world, 16)[seq & 1, 1, :] = seq
        torch.cuda.synchronize()
        out = xp_gpu.Int64(n)
        code = {"SFloat": 0, "DFloat": 1, "Int32": 2, "Int64": 3}[tname]
        rc = lib.cb200_peer_exchange_arg_kernel_launch(mine.data_ptr(), code, n, val_off, 1, 0, out.data_ptr, bases, world, 0, slot, seq,
                                                       1 << 12, status.data_ptr())
        assert rc == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        f0, f1 = v0.astype(np.float64), v1.astype(np.float64)
        take1 = np.where(np.isnan(f0), ~np.isnan(f1), (f1 > f0))        # rank 0 keeps ties (its indices are the lower ones)
        take1 = np.where(np.isnan(f0) & np.isnan(f1), False, take1)
        assert np.array_equal(out.to_numpy(), np.where(take1, i1, i0))
    finally:
        torch.cuda.synchronize()
        lib.cb200_peer_buffer_destroy(base)


def test_peer_exchange_wait_runs_out_by_its_limit(xp_gpu):
    """A flag that nothing sets: the wait gives up after its (short) limit, the status word says so, the kernel returns
    and the context stays usable."""
    import torch

    world, slot = 2, 4096
    lib, base, bases, status = _exchange_setup(world, slot)
    try:
        mine = torch.ones(256, dtype=torch.float32, device="cuda")
        rc = lib.cb200_peer_exchange_kernel_launch(mine.data_ptr(), 1024, bases, world, 0, slot, 1, 2000, status.data_ptr())
        assert rc == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 1
        assert float((xp_gpu.SFloat.from_torch(mine) + 1).sum().extract()) == 512.0
        # refused arguments launch nothing
        assert lib.cb200_peer_exchange_kernel_launch(mine.data_ptr(), slot + 16, bases, world, 0, slot, 2, 0, status.data_ptr()) != 0
        assert lib.cb200_peer_exchange_kernel_launch(mine.data_ptr(), 1024, bases, world, 2, slot, 2, 0, status.data_ptr()) != 0
        assert lib.cb200_peer_exchange_kernel_launch(mine.data_ptr(), 1024, bases, world, 0, slot, 0, 0, status.data_ptr()) != 0
    finally:
        torch.cuda.synchronize()
        lib.cb200_peer_buffer_destroy(base)
