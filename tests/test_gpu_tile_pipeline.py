"""The copy-engine form of the tile kernel (operands whose contiguous axes differ, everything 16-byte aligned): results
against the CPU oracle bit for bit, proof that the kernel itself ran (its launch counter), and its status word."""
import ctypes

import numpy as np
import pytest

from oracle_narray import OracleXP as ox

pytestmark = pytest.mark.gpu

TYPES = ("SFloat", "DFloat", "Int32", "Int64")


def host(tname, shape, rng):
    if tname.endswith("Float"):
        return rng.standard_normal(shape).astype(np.float32 if tname == "SFloat" else np.float64)
    return rng.integers(-1000, 1000, shape).astype(np.int32 if tname == "Int32" else np.int64)


def counters():
    from cumo_b200 import _lib
    lib = _lib.load()
    lib.cb200_tile_pipeline_launches.restype = ctypes.c_ulonglong
    lib.cb200_tile_pipeline_status.restype = ctypes.c_int
    return lib.cb200_tile_pipeline_launches, lib.cb200_tile_pipeline_status


# extents are whole 16-byte packets; most are not whole tiles, so edge tiles are partly outside the arrays
@pytest.mark.parametrize("shape", [(128, 128), (260, 132), (1028, 516), (36, 4100), (4100, 20), (2048, 1024)])
@pytest.mark.parametrize("tname", TYPES)
def test_aligned_transposed_operands_run_in_the_pipeline_kernel(xp_gpu, tname, shape):
    launches, status = counters()
    rng = np.random.default_rng(shape[0] * 7 + shape[1])
    ha, hb = host(tname, shape, rng), host(tname, shape[::-1], rng)
    G, O = getattr(xp_gpu, tname), getattr(ox, tname)
    ga, gb, oa, ob = G.from_numpy(ha), G.from_numpy(hb), O.cast(ha), O.cast(hb)
    before = launches()
    assert np.array_equal((ga + gb.transpose()).to_numpy(), (oa + ob.transpose()).to_numpy())
    assert np.array_equal((gb.transpose() * ga).to_numpy(), (ob.transpose() * oa).to_numpy())
    assert np.array_equal((gb.transpose() - 3).to_numpy(), (ob.transpose() - 3).to_numpy())
    assert np.array_equal(gb.transpose().dup().to_numpy(), hb.T)
    gc, oc = G.from_numpy(hb + 1), O.cast(hb + 1)
    assert np.array_equal((gb.transpose() + gc.transpose()).to_numpy(), (ob.transpose() + oc.transpose()).to_numpy())
    assert launches() - before == 5, "the aligned cases must take the copy-engine kernel"
    # views whose first element is 16-byte aligned stay in it; an odd offset falls back and still agrees
    assert np.array_equal((ga[4:, 8:] + gb.transpose()[4:, 8:]).to_numpy(), (oa[4:, 8:] + ob.transpose()[4:, 8:]).to_numpy())
    assert np.array_equal((ga[3:, 2:] + gb.transpose()[3:, 2:]).to_numpy(), (oa[3:, 2:] + ob.transpose()[3:, 2:]).to_numpy())
    assert status() == 0


@pytest.mark.parametrize("src,dst", [("Int32", "SFloat"), ("SFloat", "Int32"), ("DFloat", "Int64"), ("Int64", "DFloat")])
def test_cast_between_types_of_one_size(xp_gpu, src, dst):
    launches, status = counters()
    rng = np.random.default_rng(11)
    h = host(src, (300, 1032), rng)
    g = getattr(xp_gpu, src).from_numpy(h)
    before = launches()
    got = getattr(xp_gpu, dst).cast(g.transpose()).to_numpy()
    want = getattr(ox, dst).cast(getattr(ox, src).cast(h).transpose()).to_numpy()
    assert np.array_equal(got, want)
    assert launches() - before == 1
    assert status() == 0


@pytest.mark.parametrize("tname", ("SFloat", "Int64"))
def test_batched_planes(xp_gpu, tname):
    launches, status = counters()
    rng = np.random.default_rng(6)
    h = host(tname, (5, 72, 92), rng)
    G, O = getattr(xp_gpu, tname), getattr(ox, tname)
    g, o = G.from_numpy(h), O.cast(h)
    before = launches()
    assert np.array_equal(g.transpose(0, 2, 1).dup().to_numpy(), h.transpose(0, 2, 1))
    assert np.array_equal(g.transpose(2, 1, 0).dup().to_numpy(), h.transpose(2, 1, 0))
    hb = host(tname, (5, 92, 72), rng)
    assert np.array_equal((g.transpose(0, 2, 1) + G.from_numpy(hb)).to_numpy(), (o.transpose(0, 2, 1) + O.cast(hb)).to_numpy())
    # one plane against every batch: the repeated operand's batch step is 0
    hp = host(tname, (92, 72), rng)
    assert np.array_equal((g.transpose(0, 2, 1) * G.from_numpy(hp)).to_numpy(), (o.transpose(0, 2, 1) * O.cast(hp)).to_numpy())
    h4 = host(tname, (2, 3, 48, 68), rng)
    g4, o4 = G.from_numpy(h4), O.cast(h4)
    assert np.array_equal(g4.transpose(0, 1, 3, 2).dup().to_numpy(), h4.transpose(0, 1, 3, 2))
    assert np.array_equal(g4.transpose(1, 0, 3, 2).dup().to_numpy(), h4.transpose(1, 0, 3, 2))
    assert launches() - before == 5
    assert status() == 0


def test_integer_division_by_zero_is_seen_only_inside_the_arrays(xp_gpu):
    """Edge tiles are zero-filled outside the arrays; those zeros must never reach the operation."""
    launches, status = counters()
    rng = np.random.default_rng(3)
    ha = rng.integers(1, 100, (132, 260)).astype(np.int32)
    hb = rng.integers(1, 100, (260, 132)).astype(np.int32)
    ga, gb = xp_gpu.Int32.from_numpy(ha), xp_gpu.Int32.from_numpy(hb)
    before = launches()
    got = (ga / gb.transpose()).to_numpy()          # raises on a zero divisor
    assert launches() - before == 1
    want = (ox.Int32.cast(ha) / ox.Int32.cast(hb).transpose()).to_numpy()
    assert np.array_equal(got, want)
    assert status() == 0
