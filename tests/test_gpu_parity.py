"""Parity of the CUDA path with the CPU oracle on seeded inputs.

Bar: bit-exact for integer arithmetic, comparisons, indices, counts, min/max and
for the IEEE-exact float operations (+ - * / fmod, rounding, sign games); float
sums and means within 1e-5 (fp32) / 1e-12 (fp64) of a float64 pairwise reference;
libm-style functions within a few units in the last place of the oracle's libm.
"""
import numpy as np
import pytest

from oracle import cumo_oracle as orc
from oracle_narray import OracleXP

pytestmark = pytest.mark.gpu

NP = {"SFloat": np.float32, "DFloat": np.float64, "Int32": np.int32, "Int64": np.int64}
FLOATS = ("SFloat", "DFloat")
INTS = ("Int32", "Int64")
FP32_SUM_TOL = 1e-5      # relative to a float64 reference sum
FP64_SUM_TOL = 1e-12
ULP_RTOL = {"SFloat": 1e-6, "DFloat": 2e-15 * 8}   # libm-style functions


def rng_array(rng, tname, shape, lo=-50, hi=50):
    if tname in FLOATS:
        return rng.uniform(-4, 4, size=shape).astype(NP[tname])
    return rng.integers(lo, hi, size=shape).astype(NP[tname])


def both(xp_gpu, tname, host):
    return getattr(xp_gpu, tname).from_numpy(host), getattr(OracleXP, tname).cast(host)


def same(gpu, ora, exact=True, rtol=0.0, atol=0.0):
    g = np.asarray(gpu.to_numpy())
    o = np.asarray(ora.to_numpy())
    assert g.shape == o.shape, (g.shape, o.shape)
    assert g.dtype == o.dtype, (g.dtype, o.dtype)
    if exact:
        assert np.array_equal(g, o, equal_nan=True), f"max |diff| {np.nanmax(np.abs(g.astype(np.float64) - o.astype(np.float64)))}"
    else:
        assert np.allclose(g, o, rtol=rtol, atol=atol, equal_nan=True), f"max rel {np.nanmax(np.abs(g - o) / np.maximum(np.abs(o), 1e-300))}"


# layouts applied identically to a GPU array and an oracle array ---------------------------------
S = slice
VIEWS_2D = {
    "whole": lambda x: x,
    "transposed": lambda x: x.transpose(),
    "cols_step3": lambda x: x[S(None), S(0, None, 3)],
    "rows_step2": lambda x: x[S(0, None, 2), S(None)],
    "inner_window": lambda x: x[S(1, None), S(1, -1)],
    "reversed_cols": lambda x: x[S(None), S(None, None, -1)],
    "reversed_rows": lambda x: x[S(None, None, -1), S(None)],
}

BINARY_EXACT = {"SFloat": ["add", "sub", "mul", "div", "mod", "copysign", "maximum", "minimum", "maximum_nan", "minimum_nan"],
                "DFloat": ["add", "sub", "mul", "div", "mod", "copysign", "maximum", "minimum", "maximum_nan", "minimum_nan"],
                "Int32": ["add", "sub", "mul", "bit_and", "bit_or", "bit_xor", "maximum", "minimum"],
                "Int64": ["add", "sub", "mul", "bit_and", "bit_or", "bit_xor", "maximum", "minimum"]}


@pytest.mark.parametrize("tname", list(NP))
@pytest.mark.parametrize("n", [1, 3, 31, 32, 33, 127, 1000, 4097, 70001])
def test_binary_contiguous_1d(xp_gpu, tname, n):
    rng = np.random.default_rng(n)
    ha, hb = rng_array(rng, tname, n), rng_array(rng, tname, n)
    if tname in FLOATS and n > 3:
        ha[1] = np.nan; hb[2] = np.inf; ha[3 % n] = -0.0
    ga, oa = both(xp_gpu, tname, ha)
    gb, ob = both(xp_gpu, tname, hb)
    for op in BINARY_EXACT[tname]:
        same(ga._binary(op, gb), oa._binary(op, ob))
    # an unaligned start: the 16-byte path must give way to the scalar one
    if n > 4:
        same(ga[1:] + gb[:-1], oa[1:] + ob[:-1])
        same(ga[1:] * gb[1:], oa[1:] * ob[1:])


@pytest.mark.parametrize("tname", list(NP))
def test_binary_scalar_forms(xp_gpu, tname):
    rng = np.random.default_rng(5)
    ha = rng_array(rng, tname, (37, 129))
    ga, oa = both(xp_gpu, tname, ha)
    sv = 3 if tname in INTS else 2.5
    for f in (lambda x: x + sv, lambda x: sv + x, lambda x: x - sv, lambda x: sv - x, lambda x: x * sv,
              lambda x: x / sv, lambda x: x % sv, lambda x: sv % (x * x + 1)):
        same(f(ga), f(oa))
    if tname in INTS:
        for f in (lambda x: x & 5, lambda x: x | 5, lambda x: x ^ 5, lambda x: (x & 7) << 2, lambda x: x >> 1, lambda x: ~x):
            same(f(ga), f(oa))
        # an int array against a Python float goes through DFloat
        same(ga * 0.5, oa * 0.5)
    same(ga ** 2, oa ** 2)
    same(ga ** 3, oa ** 3)
    same(ga ** 0, oa ** 0)
    same(-ga, -oa)
    same(abs(ga), abs(oa))
    same(ga.square(), oa.square())
    same(ga.sign(), oa.sign())


@pytest.mark.parametrize("tname", list(NP))
@pytest.mark.parametrize("shapes", [((4096, 1), (1, 512)), ((300, 784), (300, 1)), ((300, 784), (1, 784)), ((300, 784), (784,)),
                                    ((70, 1), (1, 2052)), ((67, 2056), (1, 2056)), ((33, 1500), (1500,)), ((1, 4100), (40, 4100)),
                                    ((7, 1, 33), (1, 5, 33)), ((6, 5, 1, 3), (5, 4, 1)), ((2, 3, 4, 5, 6), (2, 3, 4, 5, 6)), ((5, 3), (1,))])
def test_binary_broadcast(xp_gpu, tname, shapes):
    rng = np.random.default_rng(11)
    ha, hb = rng_array(rng, tname, shapes[0]), rng_array(rng, tname, shapes[1])
    ga, oa = both(xp_gpu, tname, ha)
    gb, ob = both(xp_gpu, tname, hb)
    same(ga + gb, oa + ob)
    same(gb - ga, ob - oa)
    same(ga * gb, oa * ob)
    same(ga.gt(gb), oa.gt(ob))
    same(ga.le(gb), oa.le(ob))


@pytest.mark.parametrize("tname", list(NP))
@pytest.mark.parametrize("va", list(VIEWS_2D))
@pytest.mark.parametrize("vb", ["whole", "transposed", "cols_step3", "reversed_cols"])
def test_binary_views(xp_gpu, tname, va, vb):
    rng = np.random.default_rng(7)
    base = (60, 60)
    ha, hb = rng_array(rng, tname, base), rng_array(rng, tname, base)
    ga, oa = both(xp_gpu, tname, ha)
    gb, ob = both(xp_gpu, tname, hb)
    xa, ya = VIEWS_2D[va](ga), VIEWS_2D[va](oa)
    # shape the second operand like the first by viewing a freshly cut block of the same extent
    r, c = ya.shape
    hb2 = rng_array(rng, tname, {"whole": (r, c), "transposed": (c, r), "cols_step3": (r, 3 * c), "reversed_cols": (r, c)}[vb])
    gb2, ob2 = both(xp_gpu, tname, hb2)
    xb, yb = VIEWS_2D[vb](gb2), VIEWS_2D[vb](ob2)
    assert xa.shape == ya.shape == yb.shape == xb.shape
    same(xa + xb, ya + yb)
    same(xa * xb, ya * yb)
    same(xa.lt(xb), ya.lt(yb))
    same(-xa, -ya)


@pytest.mark.parametrize("tname", list(NP))
def test_permuted_views_up_to_8d(xp_gpu, tname):
    # a permutation that leaves no pair of axes mergeable (test/narray_test.rb:41-52)
    for nd in range(3, 9):
        shape = [2 if i % 2 == 0 else 3 for i in range(nd)]
        perm = list(range(1, nd, 2)) + list(range(0, nd, 2))
        host = np.arange(int(np.prod(shape))).astype(NP[tname]).reshape(shape)
        g, o = both(xp_gpu, tname, host)
        gv, ov = g.transpose(*perm), o.transpose(*perm)
        same(gv + gv, ov + ov)
        same(-gv, -ov)
        same(gv.dup(), ov.dup())


@pytest.mark.parametrize("tname", list(NP))
def test_inplace_output(xp_gpu, tname):
    rng = np.random.default_rng(3)
    ha, hb = rng_array(rng, tname, (129, 65)), rng_array(rng, tname, (129, 1))
    ga, oa = both(xp_gpu, tname, ha)
    gb, ob = both(xp_gpu, tname, hb)
    r = ga.inplace() + gb
    same(r, oa + ob)
    same(ga, oa + ob)            # the left operand itself was overwritten
    r = ga.inplace() * 2
    same(ga, (oa + ob) * 2)


@pytest.mark.parametrize("tname", INTS)
def test_integer_division_exact_and_flag(xp_gpu, tname):
    rng = np.random.default_rng(9)
    ha = rng_array(rng, tname, 100_003, -(2 ** 20), 2 ** 20)
    hb = rng_array(rng, tname, 100_003, -9, 9)
    hb[hb == 0] = 7
    ga, oa = both(xp_gpu, tname, ha)
    gb, ob = both(xp_gpu, tname, hb)
    same(ga / gb, oa / ob)
    same(ga % gb, oa % ob)
    same((ga * 3 + gb) % 7, (oa * 3 + ob) % 7)
    info = np.iinfo(NP[tname])
    edge = np.array([info.min, info.min, info.max, -1, 0], dtype=NP[tname])
    div = np.array([-1, 1, -1, info.min, 5], dtype=NP[tname])
    ge, oe = both(xp_gpu, tname, edge)
    gd, od = both(xp_gpu, tname, div)
    same(ge / gd, oe / od)
    same(ge % gd, oe % od)
    hb[77] = 0
    gz, _ = both(xp_gpu, tname, hb)
    with pytest.raises(ZeroDivisionError):
        ga / gz
    with pytest.raises(ZeroDivisionError):
        ga % gz
    with pytest.raises(ZeroDivisionError):
        gz.reciprocal()
    with pytest.raises(ValueError):
        abs(ge)


UNARY_EXACT = ["minus", "square", "sign", "abs", "floor", "round", "ceil", "trunc", "rint", "reciprocal"]
MATH_FNS = ("sqrt cbrt log log2 log10 exp exp2 exp10 sin cos tan asin acos atan sinh cosh tanh "
            "asinh acosh atanh sinc erf erfc log1p expm1").split()


@pytest.mark.parametrize("tname", FLOATS)
def test_float_unary_and_math(xp_gpu, tname):
    rng = np.random.default_rng(21)
    host = rng.uniform(-3, 3, size=(257, 129)).astype(NP[tname])
    host[0, :6] = [np.nan, np.inf, -np.inf, 0.0, -0.0, 2.5]
    g, o = both(xp_gpu, tname, host)
    for op in UNARY_EXACT:
        same(g._unary(op), o._unary(op))
    for op in ("isnan", "isinf", "isposinf", "isneginf", "isfinite", "signbit"):
        same(getattr(g, op)(), getattr(o, op)())
    pos = np.abs(host) + 0.5
    unit = np.clip(host / 4, -0.99, 0.99)
    for fn in MATH_FNS:
        src = pos if fn in ("sqrt", "log", "log2", "log10", "acosh") else (unit if fn in ("asin", "acos", "atanh") else host)
        src = np.where(np.isfinite(src), src, 1.0).astype(NP[tname])
        if fn == "sinc":
            src = np.where(src == 0, 1.0, src).astype(NP[tname])
        gs, os_ = both(xp_gpu, tname, src)
        tol = ULP_RTOL[tname] * (64 if fn in ("sin", "cos", "tan", "erfc", "sinc") else 1)
        same(getattr(xp_gpu.NMath, fn)(gs), getattr(OracleXP.NMath, fn)(os_), exact=False, rtol=tol, atol=tol)
    gp, op_ = both(xp_gpu, tname, pos)
    gh, oh = both(xp_gpu, tname, np.where(np.isfinite(host), host, 1.0).astype(NP[tname]))
    same(gp ** gh, op_ ** oh, exact=False, rtol=ULP_RTOL[tname] * 4)
    same(xp_gpu.NMath.atan2(gh, gp), OracleXP.NMath.atan2(oh, op_), exact=False, rtol=ULP_RTOL[tname] * 4)
    same(xp_gpu.NMath.hypot(gh, gp), OracleXP.NMath.hypot(oh, op_), exact=False, rtol=ULP_RTOL[tname] * 4)
    same(gh ** 7, oh ** 7)
    same(gh ** -2, oh ** -2)
    same(gh.nearly_eq(gh + gh * 1e-9), oh.nearly_eq(oh + oh * 1e-9))


@pytest.mark.parametrize("tname", list(NP))
@pytest.mark.parametrize("n", [1, 31, 32, 33, 95, 96, 97, 1024, 4099, 8192, 100_000])
def test_compare_packs_bits_exactly(xp_gpu, tname, n):
    rng = np.random.default_rng(n + 1)
    ha, hb = rng_array(rng, tname, n, -3, 3), rng_array(rng, tname, n, -3, 3)
    ga, oa = both(xp_gpu, tname, ha)
    gb, ob = both(xp_gpu, tname, hb)
    for op in ("eq", "ne", "gt", "ge", "lt", "le"):
        same(getattr(ga, op)(gb), getattr(oa, op)(ob))
        same(getattr(ga, op)(1), getattr(oa, op)(1))
    same(ga > 0, oa > 0)
    if n > 40:
        same(ga[3:] > gb[:-3], oa[3:] > ob[:-3])          # misaligned inputs
        same(ga[::2] >= gb[::2], oa[::2] >= ob[::2])      # strided inputs


# ---- reductions ------------------------------------------------------------------------------------
VALUE_REDS = ["sum", "min", "max", "ptp", "prod"]
INDEX_REDS = ["max_index", "min_index", "argmax", "argmin"]
FLOAT_REDS = ["mean", "var", "stddev", "rms"]


def check_float_sum(tname, rg, ro, o, axis, keepdims, nan, mean):
    """Float sums/means: the CUDA result must lie within the stated tolerance of a float64
    reference (relative to the sum of magnitudes, which bounds any summation order's error);
    the oracle's sequential sum is itself only held to a loose sanity bound."""
    tol = FP32_SUM_TOL if tname == "SFloat" else FP64_SUM_TOL
    h = o.to_numpy().astype(np.float64)
    ax = None if axis is None else (axis if isinstance(axis, int) else tuple(axis))
    if nan:
        ref64 = np.nansum(h, axis=ax, keepdims=keepdims)
        count = np.sum(~np.isnan(h), axis=ax, keepdims=keepdims)
    else:
        ref64 = np.sum(h, axis=ax, keepdims=keepdims)
        count = np.sum(np.ones_like(h), axis=ax, keepdims=keepdims)
    scale = np.maximum(np.nansum(np.abs(h), axis=ax, keepdims=keepdims), 1e-30)
    if mean:
        with np.errstate(invalid="ignore", divide="ignore"):
            ref64, scale = ref64 / count, scale / np.maximum(count, 1)
    got, want = rg.to_numpy().astype(np.float64), ro.to_numpy().astype(np.float64)
    assert got.shape == np.shape(ref64)
    bad = np.isnan(ref64)
    assert np.array_equal(np.isnan(got), bad)
    ok = ~bad
    assert np.all(np.abs(got - ref64)[ok] <= (tol * scale)[ok] + 1e-300), float(np.max((np.abs(got - ref64) / scale)[ok]))
    assert np.all(np.abs(want - ref64)[ok] <= (1e-3 * scale)[ok] + 1e-300)


def check_reductions(xp_gpu, tname, g, o, axis, keepdims=False):
    n_red = o.size if axis is None else int(np.prod([o.shape[a] for a in ([axis] if isinstance(axis, int) else axis)]))
    for op in VALUE_REDS:
        if op == "prod" and n_red > 64:
            continue
        kw = dict(axis=axis, keepdims=keepdims)
        rg, ro = getattr(g, op)(**kw), getattr(o, op)(**kw)
        if tname in INTS or op in ("min", "max", "ptp"):
            same(rg, ro)
        elif op == "sum":
            check_float_sum(tname, rg, ro, o, axis, keepdims, False, False)
        else:
            same(rg, ro, exact=False, rtol=1e-4 if tname == "SFloat" else 1e-11)
    for op in INDEX_REDS:
        same(getattr(g, op)(axis=axis), getattr(o, op)(axis=axis))
    lo_g, hi_g = g.minmax(axis=axis)
    lo_o, hi_o = o.minmax(axis=axis)
    same(lo_g, lo_o)
    same(hi_g, hi_o)
    if tname in FLOATS:
        check_float_sum(tname, g.mean(axis=axis), o.mean(axis=axis), o, axis, False, False, True)
        check_float_sum(tname, g.sum(axis=axis, nan=True), o.sum(axis=axis, nan=True), o, axis, False, True, False)
        check_float_sum(tname, g.mean(axis=axis, nan=True), o.mean(axis=axis, nan=True), o, axis, False, True, True)
        for op in ("var", "stddev", "rms"):
            if n_red < 2 and op in ("var", "stddev"):
                continue
            for nan in (False, True):
                same(getattr(g, op)(axis=axis, nan=nan), getattr(o, op)(axis=axis, nan=nan), exact=False,
                     rtol=1e-3 if tname == "SFloat" else 1e-9, atol=1e-4 if tname == "SFloat" else 1e-11)
        for op in ("min", "max"):
            same(getattr(g, op)(axis=axis, nan=True), getattr(o, op)(axis=axis, nan=True))
        for op in INDEX_REDS:
            same(getattr(g, op)(axis=axis, nan=True), getattr(o, op)(axis=axis, nan=True))


def planted(rng, tname, shape):
    """Values with exact duplicates of the extremes (and NaNs for floats) so that ties are exercised."""
    host = rng_array(rng, tname, shape, -1000, 1000)
    flat = host.reshape(-1)
    n = flat.size
    if n >= 16:
        hi, lo = flat.max() + 1, flat.min() - 1
        for k in (n // 3, n // 3 + 1, n - 2):
            flat[k] = hi
        for k in (n // 5, n // 2, n - 1):
            flat[k] = lo
        if tname in FLOATS:
            flat[n // 7] = np.nan
    return host


@pytest.mark.parametrize("tname", list(NP))
@pytest.mark.parametrize("n", [1, 7, 32, 1000, 4097, 100_003, (1 << 20) + 7])
def test_full_reductions_1d(xp_gpu, tname, n):
    rng = np.random.default_rng(n)
    g, o = both(xp_gpu, tname, planted(rng, tname, n))
    check_reductions(xp_gpu, tname, g, o, None)
    if n > 64:
        check_reductions(xp_gpu, tname, g[3:-5], o[3:-5], None)      # unaligned start
        check_reductions(xp_gpu, tname, g[::3], o[::3], None)        # strided
        check_reductions(xp_gpu, tname, g[::-1], o[::-1], None)      # reversed


@pytest.mark.parametrize("tname", list(NP))
@pytest.mark.parametrize("shape", [(1000,), (300_000,), (40, 600), (600, 1030)])
def test_index_reduction_with_value(xp_gpu, tname, shape):
    """The one-pass {index, value} form against the separate index and extreme reductions of the oracle."""
    rng = np.random.default_rng(shape[0])
    g, o = both(xp_gpu, tname, planted(rng, tname, shape))
    for axis in ([None] if len(shape) == 1 else [None, 0, 1]):
        for op in INDEX_REDS:
            for nan in ((False, True) if tname in FLOATS else (False,)):
                gi, gv = g.arg_with_value(op, axis=axis, nan=nan)
                oi, ov = o.arg_with_value(op, axis=axis, nan=nan)
                same(gi, oi)
                same(gv, ov)


@pytest.mark.parametrize("n", [1, 31, 32, 33, 1000, 32767, 32768, 32769, 1_000_003, (1 << 25) + 77])
@pytest.mark.parametrize("density", [0.0, 0.03, 0.5, 1.0])
def test_bit_where(xp_gpu, n, density):
    rng = np.random.default_rng(n)
    host = rng.random(n) < density
    g, o = xp_gpu.Bit.from_numpy(host), OracleXP.Bit.cast(host)
    same(g.where(), o.where())
    ones, zeros = g.where2()
    o1, o0 = o.where2()
    same(ones, o1)
    same(zeros, o0)


def test_bit_where_of_a_comparison_and_2d(xp_gpu):
    rng = np.random.default_rng(1)
    host = rng.integers(-50, 50, (300, 1000)).astype(np.int32)
    g = xp_gpu.Int32.from_numpy(host) > 10
    assert np.array_equal(g.where().to_numpy(), np.flatnonzero(host > 10).astype(np.int32))


@pytest.mark.parametrize("tname", list(NP))
@pytest.mark.parametrize("n", [1, 15, 16, 17, 4095, 4096, 4097, 100_003, (1 << 24) + 5])
def test_cumsum_cumprod_1d(xp_gpu, tname, n):
    rng = np.random.default_rng(n)
    if tname in FLOATS:
        host = rng.integers(-3, 4, n).astype(NP[tname])            # small integers: float sums stay exact in any association
        hostp = np.where(np.arange(n) % 4 < 2, 2.0, 0.5).astype(NP[tname])      # products stay within [0.5, 4]: nothing overflows
    else:
        host = rng.integers(-(1 << 30), 1 << 30, n).astype(NP[tname])    # sums and products wrap: must wrap identically
        hostp = rng.integers(-3, 4, n).astype(NP[tname])
    g, o = both(xp_gpu, tname, host)
    same(g.cumsum(), o.cumsum())
    gp, op_ = both(xp_gpu, tname, hostp)
    same(gp.cumprod(), op_.cumprod())
    if n > 64 and n < (1 << 22):
        same(g[3:-5].cumsum(), o[3:-5].cumsum())
        same(g[::3].cumsum(), o[::3].cumsum())
        same(g[::-1].cumsum(), o[::-1].cumsum())
    if tname in FLOATS and n > 16:
        hn = host.copy()
        hn[[0, n // 2, n - 1]] = np.nan
        hn[5] = -0.0
        gn, on = both(xp_gpu, tname, hn)
        same(gn.cumsum(), on.cumsum())
        same(gn.cumsum(nan=True), on.cumsum(nan=True))
        hpn = hostp.copy()
        hpn[[0, n // 2, n - 1]] = np.nan
        gpn, opn = both(xp_gpu, tname, hpn)
        same(gpn.cumprod(), opn.cumprod())
        same(gpn.cumprod(nan=True), opn.cumprod(nan=True))
        hz = np.full(min(n, 5000), -0.0, dtype=NP[tname])
        gz, oz = both(xp_gpu, tname, hz)
        assert np.array_equal(np.signbit(gz.cumsum().to_numpy()), np.signbit(oz.cumsum().to_numpy()))   # -0.0 stays -0.0


@pytest.mark.parametrize("tname", ["SFloat", "Int64"])
def test_cumsum_along_axes_and_random_floats(xp_gpu, tname):
    rng = np.random.default_rng(2)
    host = rng.integers(-5, 6, (37, 5000)).astype(NP[tname])
    g, o = both(xp_gpu, tname, host)
    same(g.cumsum(axis=1), o.cumsum(axis=1))
    same(g[:, :300].cumsum(axis=0), o[:, :300].cumsum(axis=0))
    same(g.cumsum(), o.cumsum())
    same(g.transpose().cumsum(), o.transpose().cumsum())            # not one strided run: goes through a copy
    if tname == "SFloat":
        hf = rng.uniform(0, 1, 1 << 20).astype(np.float32)
        got = xp_gpu.SFloat.from_numpy(hf).cumsum().to_numpy().astype(np.float64)
        want = np.cumsum(hf.astype(np.float64))
        assert np.all(np.abs(got - want) <= 1e-5 * want)


@pytest.mark.parametrize("tname", INTS)
@pytest.mark.parametrize("n,bins", [(1, 1), (1000, 7), (100_003, 256), (300_000, 8192), (300_000, 8193), (50_000, 100_000)])
def test_bincount_counts_and_weights(xp_gpu, tname, n, bins):
    rng = np.random.default_rng(n + bins)
    host = rng.integers(0, bins, n).astype(NP[tname])
    host[rng.integers(0, n)] = bins - 1
    g, o = both(xp_gpu, tname, host)
    same(g.bincount(), o.bincount())
    same(g.bincount(minlength=bins + 5), o.bincount(minlength=bins + 5))
    same(g[::3].bincount(), o[::3].bincount())                                   # a strided run
    for wt, tol in (("SFloat", 1e-5), ("DFloat", 1e-12)):
        hw = rng.uniform(0, 1, n).astype(NP[wt])
        gw, ow = both(xp_gpu, wt, hw)
        got, want = g.bincount(gw).to_numpy(), o.bincount(ow).to_numpy()
        assert got.dtype == want.dtype and got.shape == want.shape
        exact = np.bincount(host.astype(np.int64), weights=hw.astype(np.float64), minlength=bins)
        assert np.all(np.abs(got - exact) <= tol * np.maximum(1.0, np.bincount(host.astype(np.int64), minlength=bins)))
    if n > 10:
        rows = host[: n // 4 * 4].reshape(4, -1)
        g2, o2 = both(xp_gpu, tname, rows)
        same(g2.bincount(), o2.bincount())                                          # one launch per leading index


def test_new_ops_on_empty_arrays(xp_gpu):
    for xp in (xp_gpu, OracleXP):
        e = xp.Int32.cast(np.array([], dtype=np.int32))
        assert e.bincount().to_a() == []
        assert e.bincount(minlength=3).to_a() == [0, 0, 0]
        assert e.cumsum().to_a() == []
        f = xp.SFloat.cast(np.zeros((0, 5), dtype=np.float32))
        assert f.cumsum(axis=1).shape == (0, 5)
        assert xp.Bit.cast(np.zeros(0, dtype=bool)).where().to_a() == []


def test_bincount_rejects_negative_items(xp_gpu):
    with pytest.raises(ValueError):
        xp_gpu.Int32.from_numpy(np.array([0, 5, -1, 2], dtype=np.int32)).bincount()
    with pytest.raises(AttributeError):
        xp_gpu.SFloat.from_numpy(np.array([0, 1], dtype=np.float32)).bincount()


def extreme_fills(tname):
    if tname in FLOATS:
        return {"all_nan": np.nan, "all_neg_inf": -np.inf, "all_pos_inf": np.inf, "all_zero": 0.0}
    info = np.iinfo(NP[tname])
    return {"all_min": info.min, "all_max": info.max, "all_zero": 0}


@pytest.mark.parametrize("tname", list(NP))
@pytest.mark.parametrize("shape", [(5,), (70_001,), (300_000,), (40, 600), (600, 40), (300, 1030), (9, 40_000)])
def test_index_reductions_on_extreme_values(xp_gpu, tname, shape):
    """Arrays where every element ranks equal to the identity of the scan (all NaN, all -inf, all INT_MIN ...),
    then the same with a few ordinary values and NaNs sprinkled in: the first index must win everywhere."""
    rng = np.random.default_rng(len(shape) * 1000 + shape[0])
    axes = [None] if len(shape) == 1 else [None, 0, 1]
    for name, fill in extreme_fills(tname).items():
        for sprinkle in (False, True):
            host = np.full(shape, fill, dtype=NP[tname])
            if sprinkle:
                flat = host.reshape(-1)
                pick = rng.choice(flat.size, size=min(7, flat.size), replace=False)
                flat[pick] = rng_array(rng, tname, len(pick))
                if tname in FLOATS:
                    flat[rng.integers(0, flat.size)] = np.nan
                    flat[rng.integers(0, flat.size)] = -0.0
            g, o = both(xp_gpu, tname, host)
            for axis in axes:
                for op in INDEX_REDS:
                    same(getattr(g, op)(axis=axis), getattr(o, op)(axis=axis))
                    if tname in FLOATS:
                        same(getattr(g, op)(axis=axis, nan=True), getattr(o, op)(axis=axis, nan=True))
                for op in ("min", "max"):
                    same(getattr(g, op)(axis=axis), getattr(o, op)(axis=axis))


@pytest.mark.parametrize("tname", list(NP))
@pytest.mark.parametrize("shape", [(96, 130), (3000, 33), (33, 3000), (4, 70_000), (70_000, 4), (1, 257), (257, 1), (513, 512), (700, 1030), (261, 2048)])
def test_axis_reductions_2d(xp_gpu, tname, shape):
    rng = np.random.default_rng(shape[0] * 7 + shape[1])
    g, o = both(xp_gpu, tname, planted(rng, tname, shape))
    for axis in (0, 1, None):
        check_reductions(xp_gpu, tname, g, o, axis)
    check_reductions(xp_gpu, tname, g, o, 1, keepdims=True)


@pytest.mark.parametrize("tname", ["SFloat", "Int64"])
@pytest.mark.parametrize("view", ["transposed", "cols_step3", "rows_step2", "inner_window", "reversed_cols"])
def test_axis_reductions_on_views(xp_gpu, tname, view):
    rng = np.random.default_rng(17)
    g, o = both(xp_gpu, tname, planted(rng, tname, (130, 96)))
    gv, ov = VIEWS_2D[view](g), VIEWS_2D[view](o)
    for axis in (0, 1, None):
        check_reductions(xp_gpu, tname, gv, ov, axis)


@pytest.mark.parametrize("tname", ["DFloat", "Int32"])
def test_reductions_nd_axis_subsets(xp_gpu, tname):
    rng = np.random.default_rng(23)
    shape = (5, 6, 7, 8)
    g, o = both(xp_gpu, tname, planted(rng, tname, shape))
    for axis in (0, 1, 2, 3, [0, 1], [1, 2], [2, 3], [0, 3], [0, 2], [1, 3], [0, 1, 2], [1, 2, 3], [0, 2, 3]):
        check_reductions(xp_gpu, tname, g, o, axis)
    gp, op_ = g.transpose(2, 0, 3, 1), o.transpose(2, 0, 3, 1)
    for axis in (0, 2, [1, 3], [0, 1]):
        check_reductions(xp_gpu, tname, gp, op_, axis)
    g5, o5 = both(xp_gpu, tname, planted(rng, tname, (3, 4, 5, 2, 6)))
    for axis in ([0, 3, 4], [1, 2], 2):
        check_reductions(xp_gpu, tname, g5, o5, axis)


def test_reduction_is_deterministic(xp_gpu):
    rng = np.random.default_rng(1)
    host = rng.uniform(-1, 1, size=(1 << 22) + 3).astype(np.float32)
    g = xp_gpu.SFloat.from_numpy(host)
    first = g.sum().to_numpy().tobytes()
    for _ in range(5):
        assert g.sum().to_numpy().tobytes() == first
    m = xp_gpu.SFloat.from_numpy(host[: 2048 * 2048].reshape(2048, 2048))
    c0 = m.sum(axis=0).to_numpy().tobytes()
    for _ in range(3):
        assert m.sum(axis=0).to_numpy().tobytes() == c0


# ---- Bit counts ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 31, 32, 33, 127, 128, 129, 4096, 100_003, (1 << 22) + 5])
def test_count_true_full(xp_gpu, n):
    rng = np.random.default_rng(n)
    bits = rng.random(n) < 0.37
    g = xp_gpu.Bit.from_numpy(bits)
    assert g.count_true().extract() == int(bits.sum())
    assert g.count_false().extract() == int(n - bits.sum())
    words = xp_gpu.pack_bits(bits)
    assert orc.bit_count(words, 0, 1, n) == int(bits.sum())
    if n > 70:
        # views: a bit offset that is not a word boundary, a strided run
        assert g[5:n - 3].count_true().extract() == orc.bit_count(words, 5, 1, n - 8)
        assert g[37:].count_false().extract() == orc.bit_count(words, 37, 1, n - 37, True)
        assert g[1::3].count_true().extract() == orc.bit_count(words, 1, 3, len(range(1, n, 3)))


def test_count_true_axes(xp_gpu):
    rng = np.random.default_rng(4)
    bits = rng.random((37, 5, 130)) < 0.5
    g = xp_gpu.Bit.from_numpy(bits)
    o = OracleXP.Bit.cast(bits)
    for axis in (0, 1, 2, [0, 1], [1, 2], [0, 2], None):
        same(g.count_true(axis=axis), o.count_true(axis=axis))
        same(g.count_false(axis=axis), o.count_false(axis=axis))
    same(g.count_true(axis=1, keepdims=True), o.count_true(axis=1, keepdims=True))


# ---- mulsum ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("tname", list(NP))
def test_mulsum(xp_gpu, tname):
    rng = np.random.default_rng(12)
    ha, hb = rng_array(rng, tname, 100_003, -30, 30), rng_array(rng, tname, 100_003, -30, 30)
    ga, oa = both(xp_gpu, tname, ha)
    gb, ob = both(xp_gpu, tname, hb)
    got = ga.mulsum(gb).to_numpy()
    if tname in INTS:
        assert got == orc.mulsum_1d(ha, hb)
    else:
        ref = float(np.dot(ha.astype(np.float64), hb.astype(np.float64)))
        scale = float(np.abs(ha.astype(np.float64) * hb.astype(np.float64)).sum())
        assert abs(float(got) - ref) <= (FP32_SUM_TOL if tname == "SFloat" else FP64_SUM_TOL) * scale
    hm, hv = rng_array(rng, tname, (33, 65), -9, 9), rng_array(rng, tname, (65,), -9, 9)
    gm, om = both(xp_gpu, tname, hm)
    gv, ov = both(xp_gpu, tname, hv)
    for axis in (0, 1):
        same(gm.mulsum(gv, axis=axis), om.mulsum(ov, axis=axis), exact=tname in INTS, rtol=1e-4, atol=1e-3)


# ---- casts ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("src", list(NP))
@pytest.mark.parametrize("dst", list(NP))
def test_store_cast(xp_gpu, src, dst):
    rng = np.random.default_rng(2)
    host = rng_array(rng, src, (70, 33), -1000, 1000)
    g, o = both(xp_gpu, src, host)
    same(getattr(xp_gpu, dst).cast(g), getattr(OracleXP, dst).cast(o))
    same(getattr(xp_gpu, dst).cast(g.transpose()), getattr(OracleXP, dst).cast(o.transpose()))


def test_mixed_type_operands_upcast(xp_gpu):
    rng = np.random.default_rng(8)
    hi, hf = rng_array(rng, "Int32", (40, 50)), rng_array(rng, "SFloat", (40, 50))
    gi, oi = both(xp_gpu, "Int32", hi)
    gf, of = both(xp_gpu, "SFloat", hf)
    same(gi + gf, oi + of)
    same(gf * gi, of * oi)
    hd = rng_array(rng, "DFloat", (50,))
    gd, od = both(xp_gpu, "DFloat", hd)
    same(gf - gd, of - od)
    hl = rng_array(rng, "Int64", (40, 1))
    gl, ol = both(xp_gpu, "Int64", hl)
    same(gi * gl, oi * ol)


def test_shape_mismatch_raises(xp_gpu):
    a = xp_gpu.SFloat.zeros(3, 4)
    b = xp_gpu.SFloat.zeros(3, 5)
    with pytest.raises(xp_gpu.ShapeError):
        a + b


def test_empty_arrays(xp_gpu):
    a = xp_gpu.SFloat.zeros(0)
    assert (a + a).shape == (0,)
    assert (a > 0).shape == (0,)
    assert a.sum().extract() == 0.0
    assert xp_gpu.Bit.from_numpy(np.zeros(0, bool)).count_true().extract() == 0
