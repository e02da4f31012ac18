"""Operands whose contiguous axes differ (a transposed operand): the shared-memory tile kernel against the CPU oracle,
bit for bit, on ragged shapes, every element type, mixed element sizes, batch dimensions, and both inputs transposed."""
import numpy as np
import pytest

from oracle_narray import OracleXP as ox

pytestmark = pytest.mark.gpu

TYPES = ("SFloat", "DFloat", "Int32", "Int64")


def host(tname, shape, rng):
    if tname.endswith("Float"):
        return rng.standard_normal(shape).astype(np.float32 if tname == "SFloat" else np.float64)
    return rng.integers(-1000, 1000, shape).astype(np.int32 if tname == "Int32" else np.int64)


@pytest.mark.parametrize("shape", [(257, 130), (1000, 33), (64, 64), (4099, 17), (129, 2050)])
@pytest.mark.parametrize("tname", TYPES)
def test_binary_with_a_transposed_operand(xp_gpu, tname, shape):
    rng = np.random.default_rng(hash(shape) % 1000)
    ha, hb = host(tname, shape, rng), host(tname, shape[::-1], rng)
    G, O = getattr(xp_gpu, tname), getattr(ox, tname)
    ga, gb, oa, ob = G.from_numpy(ha), G.from_numpy(hb), O.cast(ha), O.cast(hb)
    assert np.array_equal((ga + gb.transpose()).to_numpy(), (oa + ob.transpose()).to_numpy())
    assert np.array_equal((gb.transpose() * ga).to_numpy(), (ob.transpose() * oa).to_numpy())
    assert np.array_equal((gb.transpose() - 3).to_numpy(), (ob.transpose() - 3).to_numpy())
    assert np.array_equal(gb.transpose().dup().to_numpy(), hb.T)
    # both inputs transposed, result laid out row-major
    gc, oc = G.from_numpy(hb + 1), O.cast(hb + 1)
    assert np.array_equal((gb.transpose() + gc.transpose()).to_numpy(), (ob.transpose() + oc.transpose()).to_numpy())
    # a row-sliced transposed view: the lines of the transposed operand are longer than the tile reads
    assert np.array_equal((ga[3:, 2:] + gb.transpose()[3:, 2:]).to_numpy(), (oa[3:, 2:] + ob.transpose()[3:, 2:]).to_numpy())


@pytest.mark.parametrize("src,dst", [("Int32", "SFloat"), ("SFloat", "DFloat"), ("DFloat", "Int32"), ("Int64", "SFloat"), ("SFloat", "Int64")])
def test_cast_of_a_transposed_array(xp_gpu, src, dst):
    rng = np.random.default_rng(5)
    h = host(src, (300, 1025), rng)
    g = getattr(xp_gpu, src).from_numpy(h)
    got = getattr(xp_gpu, dst).cast(g.transpose()).to_numpy()
    want = getattr(ox, dst).cast(getattr(ox, src).cast(h).transpose()).to_numpy()
    assert np.array_equal(got, want)


@pytest.mark.parametrize("tname", ("SFloat", "Int64"))
def test_batched_planes_and_math_on_a_transposed_view(xp_gpu, tname):
    rng = np.random.default_rng(6)
    h = host(tname, (5, 70, 90), rng)
    G, O = getattr(xp_gpu, tname), getattr(ox, tname)
    g, o = G.from_numpy(h), O.cast(h)
    assert np.array_equal(g.transpose(0, 2, 1).dup().to_numpy(), h.transpose(0, 2, 1))
    assert np.array_equal(g.transpose(2, 1, 0).dup().to_numpy(), h.transpose(2, 1, 0))
    hb = host(tname, (5, 90, 70), rng)
    assert np.array_equal((g.transpose(0, 2, 1) + G.from_numpy(hb)).to_numpy(), (o.transpose(0, 2, 1) + O.cast(hb)).to_numpy())
    if tname == "SFloat":
        got = xp_gpu.NMath.exp(g.transpose(0, 2, 1)).to_numpy()
        want = ox.NMath.exp(o.transpose(0, 2, 1)).to_numpy()
        assert np.allclose(got, want, rtol=2e-6)
    else:
        m = G.from_numpy(np.where(hb == 0, 1, hb))
        mo = O.cast(np.where(hb == 0, 1, hb))
        assert np.array_equal((g.transpose(0, 2, 1) % m).to_numpy(), (o.transpose(0, 2, 1) % mo).to_numpy())
