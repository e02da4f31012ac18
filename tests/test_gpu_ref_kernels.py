"""libcumo_b200 against the reference's OWN CUDA kernels on the same GPU.

oracle/_ref/libcumo_ref_kernels.so holds the reference's kernel templates expanded for sfloat, dfloat, int32,
int64 and bit and compiled with the same nvcc (oracle/build_ref_kernels.py).  Its launch functions have the names
and argument lists of libcumo_b200's, so every case builds ONE set of descriptors and hands it to both libraries.
Both run the same CUDA math library, so elementwise results, comparisons, integer work, min/max and every index
reduction are held to bit-for-bit equality; floating-point sums, products and moments, which the two engines add
up in different orders, to the stated tolerances (fp32 1e-5, fp64 1e-12 of the sum of magnitudes).
Skipped where the reference kernels were never built (no reference checkout was available to build them from).
"""
import ctypes
from ctypes import byref, c_int, c_int32, c_size_t, c_ssize_t, c_uint64, c_void_p

import numpy as np
import pytest

from oracle import ref_kernels

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_kernels.available(), reason="oracle/_ref/libcumo_ref_kernels.so not built")]

TYPES = ("sfloat", "dfloat", "int32", "int64")
FLOATS = ("sfloat", "dfloat")
SUM_TOL = {"sfloat": 1e-5, "dfloat": 1e-12}


@pytest.fixture(scope="module")
def libs():
    import torch  # noqa: F401
    from cumo_b200 import _lib

    ours, ref = _lib.load(), ref_kernels.lib()
    yield ours, ref
    assert ref.refk_last_error() == 0


def run_both(libs, run):
    """run(L) launches on library L and returns the output tensors; returns (ours, ref) after a sync and error check."""
    import torch

    ours, ref = libs
    a = run(ours)
    torch.cuda.synchronize()
    msg = ctypes.c_char_p()
    assert ours.cb200_last_error(byref(msg)) == 0, msg.value
    b = run(ref)
    torch.cuda.synchronize()
    assert ref.refk_last_error() == 0
    return a, b


def values(tname, shape, g, kind="normal"):
    import torch
    import abi_call as ac

    dt = ac.torch_dtype(tname)
    if tname in FLOATS:
        if kind == "unit":
            return (torch.rand(shape, device="cuda", generator=g, dtype=torch.float64) * 0.5 + 0.75).to(dt)
        return (torch.randn(shape, device="cuda", generator=g, dtype=torch.float64) * 3).to(dt)
    if kind == "small":
        return torch.randint(0, 6, shape, device="cuda", generator=g, dtype=dt)
    if kind == "unit":
        return torch.randint(1, 3, shape, device="cuda", generator=g, dtype=dt)
    return torch.randint(-50, 50, shape, device="cuda", generator=g, dtype=dt)


LAYOUTS = ["flat", "rowcol", "outer", "transposed", "view3d", "reversed"]


def operands(tname, layout, g, kind2="normal"):
    """(x view, y view, logical shape); `reversed` is returned as a flat pair whose descriptors the caller flips."""
    if layout in ("flat", "reversed"):
        n = 100_003
        return values(tname, (n,), g), values(tname, (n,), g, kind2), (n,)
    if layout == "rowcol":
        return values(tname, (301, 1030), g), values(tname, (301, 1), g, kind2), (301, 1030)
    if layout == "outer":
        return values(tname, (301, 1), g), values(tname, (1, 1030), g, kind2), (301, 1030)
    if layout == "transposed":
        return values(tname, (1030, 301), g).t(), values(tname, (301, 1030), g, kind2), (301, 1030)
    x = values(tname, (7, 66, 130), g)[:, ::2, 3:99]
    y = values(tname, (7, 33, 96), g, kind2)
    return x, y, (7, 33, 96)


def flip(desc, t):
    """Walk a flat tensor backwards: pointer at the last element, negative step (`x.reverse` in the reference)."""
    desc.ptr = t.data_ptr() + (t.numel() - 1) * t.element_size()
    desc.step[0] = -t.element_size()
    return desc


BINARY = {"sfloat": ["add", "sub", "mul", "div", "mod", "pow", "copysign"], "int32": ["add", "sub", "mul", "div", "mod", "pow", "bit_and", "bit_or", "bit_xor", "left_shift", "right_shift"]}
BINARY["dfloat"], BINARY["int64"] = BINARY["sfloat"], BINARY["int32"]


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("tname", TYPES)
def test_binary_ops_bit_for_bit(libs, tname, layout):
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(sum(map(ord, tname + layout)))
    for op in BINARY[tname]:
        kind2 = "small" if op in ("pow", "left_shift", "right_shift") and tname not in FLOATS else "normal"
        x, y, shape = operands(tname, layout, g, kind2)
        flag_o, flag_r = torch.zeros(1, dtype=torch.int32, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda")
        flags = {}

        def run(L):
            out = torch.full(shape, 77, device="cuda", dtype=x.dtype)
            dx, dy, do = ac.iarray(x, shape), ac.iarray(y, shape), ac.iarray(out)
            if layout == "reversed":
                flip(dx, x)
            flag = flag_o if not flags else flag_r
            flags[len(flags)] = flag
            if op == "pow":
                ac.fn(L, f"cumo_iter_{tname}_pow_kernel_launch")(byref(dx), byref(dy), byref(do), byref(ac.indexer(shape)))
            else:
                ac.fn(L, f"cumo_iter_{tname}_{op}_kernel_launch")(byref(dx), byref(dy), byref(do), byref(ac.indexer(shape)), c_void_p(flag.data_ptr()))
            return [out]
        (a,), (b,) = run_both(libs, run)
        assert ac.bits_equal(a, b), f"{tname} {op} {layout}"
        assert flag_o.item() == flag_r.item(), f"{tname} {op} {layout}: division-by-zero flag"


@pytest.mark.parametrize("tname", TYPES)
def test_scalar_forms_bit_for_bit(libs, tname):
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(5)
    x = values(tname, (257, 515), g)
    view = x[:, 1:514]
    ops = ["add", "sub", "mul", "div", "mod"] + (["copysign"] if tname in FLOATS else ["bit_and", "bit_or", "bit_xor", "left_shift", "right_shift"])
    for op in ops:
        for left in (0, 1):
            for src in (x, view):
                sv = 3 if op in ("left_shift", "right_shift") else 7

                def run(L):
                    out = torch.full(src.shape, 9, device="cuda", dtype=x.dtype)
                    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
                    ac.fn(L, f"cumo_iter_{tname}_{op}_s_kernel_launch")(byref(ac.iarray(src)), ac.scalar(tname, sv), byref(ac.iarray(out)),
                                                                          byref(ac.indexer(src.shape)), c_void_p(flag.data_ptr()), c_int(left))
                    return [out, flag]
                (a, fa), (b, fb) = run_both(libs, run)
                assert ac.bits_equal(a, b) and fa.item() == fb.item(), f"{tname} {op}_s left={left}"
    # pow with a host numeric on either side
    base = values(tname, x.shape, g, "small") if tname not in FLOATS else x
    for left in (0, 1):
        def run(L):
            out = torch.empty_like(x)
            ac.fn(L, f"cumo_iter_{tname}_pow_s_kernel_launch")(byref(ac.iarray(base)), ac.scalar(tname, 2), byref(ac.iarray(out)), byref(ac.indexer(x.shape)), c_int(left))
            return [out]
        (a,), (b,) = run_both(libs, run)
        assert ac.bits_equal(a, b), f"{tname} pow_s left={left}"


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("tname", TYPES)
def test_clip_fill_seq_divmod_modf_frexp_bit_for_bit(libs, tname, layout):
    """The operations with three inputs, two outputs or a position-dependent value, on every layout: outputs that
    an operation refuses to write (an empty clip range, an integer zero divisor) must stay untouched in both."""
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(sum(map(ord, tname + layout)) + 1)
    x, y, shape = operands(tname, layout, g)
    z = values(tname, shape, g)

    def put(t, every, value, first=0):
        """value into every `every`-th element of t (any view), counted row-major from `first`"""
        pos = torch.arange(t.numel(), device="cuda").reshape(t.shape)
        t[(pos % every == first % every) & (pos >= first)] = value
    if tname in FLOATS:                                     # NaN on either side of a comparison
        put(z, 97, float("nan"))
        put(y, 89, float("nan"))
    ix = ac.indexer(shape)

    def descs(out_list):
        dx, dy, dz = ac.iarray(x, shape), ac.iarray(y, shape), ac.iarray(z, shape)
        if layout == "reversed":
            flip(dx, x)
        return dx, dy, dz, [ac.iarray(o) for o in out_list]

    def fresh(n=1, dtype=None):
        return [torch.full(shape, 77, device="cuda", dtype=dtype or x.dtype) for _ in range(n)]

    def clip_arrays(L):
        out, flag = fresh(), torch.zeros(1, dtype=torch.int32, device="cuda")
        dx, dy, dz, (do,) = descs(out)
        ac.fn(L, f"cumo_iter_{tname}_clip_kernel_launch")(byref(dx), byref(dy), byref(dz), byref(do), byref(ix), c_void_p(flag.data_ptr()))
        return out + [flag]
    (a, fa), (b, fb) = run_both(libs, clip_arrays)
    assert ac.bits_equal(a, b) and fa.item() == fb.item() == 1, f"{tname} clip {layout}"

    for name in ("clip_min", "clip_max"):
        def one_bound(L):
            out = fresh()
            dx, dy, _, (do,) = descs(out)
            ac.fn(L, f"cumo_iter_{tname}_{name}_kernel_launch")(byref(dx), byref(dy), byref(do), byref(ix))
            return out
        (a,), (b,) = run_both(libs, one_bound)
        assert ac.bits_equal(a, b), f"{tname} {name} {layout}"

        def one_bound_s(L):
            out = fresh()
            dx, _, _, (do,) = descs(out)
            ac.fn(L, f"cumo_iter_{tname}_{name}_s_kernel_launch")(byref(dx), ac.scalar(tname, 2), byref(do), byref(ix))
            return out
        (a,), (b,) = run_both(libs, one_bound_s)
        assert ac.bits_equal(a, b), f"{tname} {name}_s {layout}"

    def clip_s(L):
        out = fresh()
        dx, _, _, (do,) = descs(out)
        ac.fn(L, f"cumo_iter_{tname}_clip_s_kernel_launch")(byref(dx), ac.scalar(tname, -4), ac.scalar(tname, 5), byref(do), byref(ix))
        return out
    (a,), (b,) = run_both(libs, clip_s)
    assert ac.bits_equal(a, b), f"{tname} clip_s {layout}"

    def divmod_(L):
        out, flag = fresh(2), torch.zeros(1, dtype=torch.int32, device="cuda")
        dx, dy, _, (dq, dr) = descs(out)
        ac.fn(L, f"cumo_iter_{tname}_divmod_kernel_launch")(byref(dx), byref(dy), byref(dq), byref(dr), byref(ix), c_void_p(flag.data_ptr()))
        return out + [flag]
    (q1, r1, fa), (q2, r2, fb) = run_both(libs, divmod_)
    assert ac.bits_equal(q1, q2) and ac.bits_equal(r1, r2) and fa.item() == fb.item(), f"{tname} divmod {layout}"

    # fill and seq write THROUGH a layout; what lies outside the window must stay
    from ctypes import c_double, c_float
    D = c_float if tname == "sfloat" else c_double

    def window(base):
        if layout == "view3d":
            return base[:, ::2, 3:99]
        if layout == "transposed":
            return base[1].t()
        if layout in ("rowcol", "outer"):
            return base[2:5]
        return base.view(-1)

    for what in ("fill", "seq"):
        def write(L):
            base = torch.full((7, 66, 130), 77, device="cuda", dtype=x.dtype)
            target = window(base)
            d = ac.iarray(target)
            if layout == "reversed":
                flip(d, target)
            if what == "fill":
                ac.fn(L, f"cumo_iter_{tname}_fill_kernel_launch")(byref(d), byref(ac.indexer(target.shape)), ac.scalar(tname, 3))
            else:
                ac.fn(L, f"cumo_iter_{tname}_seq_kernel_launch")(byref(d), byref(ac.indexer(target.shape)), D(-1.7), D(0.37), c_double(5.0))
            return [base]
        (a,), (b,) = run_both(libs, write)
        assert ac.bits_equal(a, b), f"{tname} {what} {layout}"
        if what == "fill":
            assert (a == 3).sum().item() == window(a).numel() and (a == 77).sum().item() == a.numel() - window(a).numel()

    if tname in FLOATS:
        w = x
        for k, v in enumerate((float("nan"), float("inf"), -float("inf"), -0.0, 0.0, 1e-40)):
            put(w, w.numel() + 1, v, first=k)
        for name, second in ((f"cumo_iter_{tname}_modf_kernel_launch", None), (f"cumo_iter_{tname}_math_s_frexp_kernel_launch", torch.int32)):
            def two(L):
                o1, o2 = fresh()[0], fresh(dtype=second)[0]
                dw = ac.iarray(w, shape)
                if layout == "reversed":
                    flip(dw, w)
                ac.fn(L, name)(byref(dw), byref(ac.iarray(o1)), byref(ac.iarray(o2)), byref(ix))
                return [o1, o2]
            (a1, a2), (b1, b2) = run_both(libs, two)
            assert ac.bits_equal(a1, b1) and ac.bits_equal(a2, b2), f"{name} {layout}"


UNARY = {"sfloat": ["minus", "reciprocal", "sign", "square", "abs", "floor", "round", "ceil", "trunc", "rint"], "int32": ["minus", "reciprocal", "sign", "square", "abs", "bit_not"]}
UNARY["dfloat"], UNARY["int64"] = UNARY["sfloat"], UNARY["int32"]
MATH = ["sqrt", "cbrt", "log", "log2", "log10", "exp", "exp2", "exp10", "sin", "cos", "tan", "asin", "acos", "atan", "sinh", "cosh", "tanh",
        "asinh", "acosh", "atanh", "sinc", "erf", "erfc", "log1p", "expm1"]


def special_mix(tname, n, g):
    """Ordinary magnitudes, values inside (-1, 1), large arguments, and the special values."""
    import torch
    import abi_call as ac

    dt = ac.torch_dtype(tname)
    v = torch.randn(n, device="cuda", generator=g, dtype=torch.float64) * 3
    v[: n // 4] = torch.rand(n // 4, device="cuda", generator=g, dtype=torch.float64) * 2 - 1
    v[n // 4: n // 4 + 1000] = torch.randn(1000, device="cuda", generator=g, dtype=torch.float64) * 1e5
    v[-8:] = torch.tensor([0.0, -0.0, float("inf"), float("-inf"), float("nan"), 1.0, -1.0, 1e-30], device="cuda", dtype=torch.float64)
    return v.to(dt)


@pytest.mark.parametrize("tname", TYPES)
def test_unary_and_math_bit_for_bit(libs, tname):
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(6)
    n = 200_003
    x = special_mix(tname, n, g) if tname in FLOATS else values(tname, (n,), g)
    t2 = x[: 300 * 600].view(300, 600).t()                      # a transposed operand as well
    for src in (x, t2):
        for op in UNARY[tname]:
            def run(L):
                out = torch.full(src.shape, 5, device="cuda", dtype=x.dtype)
                flag = torch.zeros(1, dtype=torch.int32, device="cuda")
                ac.fn(L, f"cumo_iter_{tname}_{op}_kernel_launch")(byref(ac.iarray(src)), byref(ac.iarray(out)), byref(ac.indexer(src.shape)), c_void_p(flag.data_ptr()))
                return [out, flag]
            (a, fa), (b, fb) = run_both(libs, run)
            assert ac.bits_equal(a, b) and fa.item() == fb.item(), f"{tname} {op}"
        if tname not in FLOATS:
            continue
        for op in MATH:
            def run(L):
                out = torch.empty(src.shape, device="cuda", dtype=x.dtype)
                ac.fn(L, f"cumo_iter_{tname}_math_s_{op}_kernel_launch")(byref(ac.iarray(src)), byref(ac.iarray(out)), byref(ac.indexer(src.shape)))
                return [out]
            (a,), (b,) = run_both(libs, run)
            bad = (a.view(torch.int32 if tname == "sfloat" else torch.int64) != b.view(torch.int32 if tname == "sfloat" else torch.int64)).sum().item()
            assert bad == 0, f"{tname} {op}: {bad} of {a.numel()} elements differ from the reference kernel"


@pytest.mark.parametrize("tname", FLOATS)
def test_two_argument_math_bit_for_bit(libs, tname):
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(7)
    x, y = special_mix(tname, 100_001, g), special_mix(tname, 100_001, g)
    e = torch.randint(-20, 20, (100_001,), device="cuda", generator=g).to(x.dtype)
    for op, second in (("atan2", y), ("hypot", y), ("ldexp", e)):
        def run(L):
            out = torch.empty_like(x)
            ac.fn(L, f"cumo_iter_{tname}_math_s_{op}_kernel_launch")(byref(ac.iarray(x)), byref(ac.iarray(second)), byref(ac.iarray(out)), byref(ac.indexer(x.shape)))
            return [out]
        (a,), (b,) = run_both(libs, run)
        assert ac.bits_equal(a, b), f"{tname} {op}"
        for left in (0, 1):
            def run_s(L):
                out = torch.empty_like(x)
                ac.fn(L, f"cumo_iter_{tname}_math_s_{op}_s_kernel_launch")(byref(ac.iarray(e if op == "ldexp" and not left else x)), byref(ac.iarray(out)),
                                                                            byref(ac.indexer(x.shape)), ac.scalar(tname, 3.0), c_int(left))
                return [out]
            (a,), (b,) = run_both(libs, run_s)
            assert ac.bits_equal(a, b), f"{tname} {op}_s left={left}"
    for op in ("maximum", "minimum", "maximum_nan", "minimum_nan"):
        def run(L):
            out = torch.empty_like(x)
            ac.fn(L, f"cumo_{tname}_{op}_kernel_launch")(byref(ac.iarray(x)), byref(ac.iarray(y)), byref(ac.iarray(out)), byref(ac.indexer(x.shape)))
            return [out]
        (a,), (b,) = run_both(libs, run)
        assert ac.same_values(a, b), f"{tname} {op}"


@pytest.mark.parametrize("tname", TYPES)
def test_comparisons_to_bit_words(libs, tname):
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(8)
    n = 100_003
    x, y = values(tname, (n,), g), values(tname, (n,), g)
    y[::3] = x[::3]
    ops = ["eq", "ne", "gt", "ge", "lt", "le"] + (["nearly_eq"] if tname in FLOATS else [])
    for op in ops:
        for pos in (0, 37):
            def run(L):
                words = torch.zeros((n + pos + 31) // 32 + 1, device="cuda", dtype=torch.int32)
                ac.fn(L, f"cumo_iter_{tname}_{op}_kernel_launch")(byref(ac.iarray(x)), byref(ac.iarray(y)), byref(ac.bit_iarray(words, pos)), byref(ac.indexer((n,))))
                w2 = torch.zeros_like(words)
                ac.fn(L, f"cumo_iter_{tname}_{op}_s_kernel_launch")(byref(ac.iarray(x)), ac.scalar(tname, 1), byref(ac.bit_iarray(w2, pos)), byref(ac.indexer((n,))), c_int(pos != 0))
                return [words, w2]
            (a, a2), (b, b2) = run_both(libs, run)
            assert torch.equal(a, b) and torch.equal(a2, b2), f"{tname} {op} pos={pos}"
    # two dimensions, a broadcast operand, Bit output with a row step that leaves gaps
    r, c = 130, 257
    m, col = values(tname, (r, c), g), values(tname, (r, 1), g)

    def run2(L):
        words = torch.zeros((r * 300 + 31) // 32, device="cuda", dtype=torch.int32)
        ac.fn(L, f"cumo_iter_{tname}_gt_kernel_launch")(byref(ac.iarray(m)), byref(ac.iarray(col, (r, c))), byref(ac.bit_iarray(words, 3, (300, 1))), byref(ac.indexer((r, c))))
        return [words]
    (a,), (b,) = run_both(libs, run2)
    assert torch.equal(a, b)
    if tname in FLOATS:
        s = special_mix(tname, n, g)
        for op in ("isnan", "isinf", "isposinf", "isneginf", "isfinite", "signbit"):
            def run3(L):
                words = torch.zeros((n + 31) // 32, device="cuda", dtype=torch.int32)
                ac.fn(L, f"cumo_iter_{tname}_{op}_kernel_launch")(byref(ac.iarray(s)), byref(ac.bit_iarray(words)), byref(ac.indexer((n,))))
                return [words]
            (a,), (b,) = run_both(libs, run3)
            assert torch.equal(a, b), f"{tname} {op}"


RED_CASES = [((513, 4100), (1,)), ((513, 4100), (0,)), ((513, 4100), (0, 1)), ((37, 50, 61), (0, 2)), ((37, 50, 61), (1,)), (((1 << 20) + 7,), (0,)), ((3000, 33), (0,))]


def out_shape_of(shape, axes):
    return tuple(n for d, n in enumerate(shape) if d not in axes)


@pytest.mark.parametrize("shape,axes", RED_CASES)
@pytest.mark.parametrize("tname", TYPES)
def test_value_reductions(libs, tname, shape, axes):
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(9)
    x = values(tname, shape, g)
    xn = x.clone()
    if tname in FLOATS:
        xn.view(-1)[::97] = float("nan")
    osh = out_shape_of(shape, axes)
    is_f = tname in FLOATS
    acc_dt = x.dtype if is_f else torch.int64
    scale = x.abs().double().sum(dim=axes) if axes != tuple(range(len(shape))) else x.abs().double().sum()
    exact = ["min", "max", "ptp"] + ([] if is_f else ["sum"])
    tol = (["sum", "mean", "rms", "var", "stddev"] if is_f else [])
    for op in exact + tol:
        for nan in ((False, True) if is_f else (False,)):
            src = xn if nan else x
            name = f"cumo_{tname}_{op}{'_nan' if nan else ''}_kernel_launch"

            def run(L):
                out = torch.zeros(osh, device="cuda", dtype=acc_dt if op in ("sum", "prod") else x.dtype)
                ac.fn(L, name)(byref(ac.reduction_arg(src, out, axes)))
                return [out]
            (a,), (b,) = run_both(libs, run)
            if op in exact:
                assert ac.same_values(a, b), name
            elif op in ("sum", "mean"):
                n_red = x.numel() // max(1, a.numel())
                bound = SUM_TOL[tname] * scale / (n_red if op == "mean" else 1)
                assert torch.all((a.double() - b.double()).abs() <= bound), name
            else:
                assert torch.allclose(a.double(), b.double(), rtol=200 * SUM_TOL[tname], atol=0, equal_nan=True), name
    # prod on values close to one (no overflow), integers exact
    u = values(tname, shape, g, "unit")

    def runp(L):
        out = torch.zeros(osh, device="cuda", dtype=acc_dt)
        ac.fn(L, f"cumo_{tname}_prod_kernel_launch")(byref(ac.reduction_arg(u, out, axes)))
        return [out]
    (a,), (b,) = run_both(libs, runp)
    if is_f:
        assert torch.allclose(a.double(), b.double(), rtol=1e-3 if tname == "sfloat" else 1e-9, equal_nan=True)
    else:
        assert torch.equal(a, b)
    # minmax: two outputs
    for nan in ((False, True) if is_f else (False,)):
        src = xn if nan else x

        def runm(L):
            lo, hi = torch.zeros(osh, device="cuda", dtype=x.dtype), torch.zeros(osh, device="cuda", dtype=x.dtype)
            ac.fn(L, f"cumo_{tname}_minmax{'_nan' if nan else ''}_kernel_launch")(byref(ac.reduction_arg(src, lo, axes)), byref(ac.iarray(hi)))
            return [lo, hi]
        (a1, a2), (b1, b2) = run_both(libs, runm)
        assert ac.same_values(a1, b1) and ac.same_values(a2, b2)
    if tname == "dfloat":
        for nan in (False, True):
            src = xn if nan else x

            def runk(L):
                out = torch.zeros(osh, device="cuda", dtype=x.dtype)
                ac.fn(L, f"cumo_dfloat_kahan_sum{'_nan' if nan else ''}_kernel_launch")(byref(ac.reduction_arg(src, out, axes)))
                return [out]
            (a,), (b,) = run_both(libs, runk)
            assert torch.all((a - b).abs() <= 1e-12 * scale)


@pytest.mark.parametrize("shape,axes", RED_CASES)
@pytest.mark.parametrize("tname", TYPES)
def test_index_reductions_bit_for_bit(libs, tname, shape, axes):
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(10)
    x = values(tname, shape, g)
    if tname in FLOATS:
        x = torch.round(x)                      # many exact ties: first occurrence must win in both
    xn = x.clone()
    if tname in FLOATS:
        xn.view(-1)[5::101] = float("nan")
    osh = out_shape_of(shape, axes)
    for op in ("max_index", "min_index", "argmax", "argmin"):
        for nan in ((False, True) if tname in FLOATS else (False,)):
            for width, dt in ((32, torch.int32), (64, torch.int64)):
                src = xn if nan else x
                name = f"cumo_{tname}_{op}{'_nan' if nan else ''}_int{width}_kernel_launch"

                def run(L):
                    out = torch.full(osh, -1, device="cuda", dtype=dt)
                    ac.fn(L, name)(byref(ac.reduction_arg(src, out, axes)))
                    return [out]
                (a,), (b,) = run_both(libs, run)
                assert torch.equal(a, b), name


@pytest.mark.parametrize("tname", TYPES)
def test_pow_int32_forms_and_mulsum(libs, tname):
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(11)
    n = 70_001
    x = values(tname, (n,), g, "unit") if tname in FLOATS else values(tname, (n,), g, "small")
    e = torch.randint(0, 7, (n,), device="cuda", generator=g, dtype=torch.int32)

    def run(L):
        o1, o2, o3 = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
        ac.fn(L, f"cumo_iter_{tname}_pow_int32_kernel_launch")(byref(ac.iarray(x)), byref(ac.iarray(e)), byref(ac.iarray(o1)), byref(ac.indexer((n,))))
        ac.fn(L, f"cumo_iter_{tname}_pow_int32_s_kernel_launch")(byref(ac.iarray(x)), c_int32(5), byref(ac.iarray(o2)), byref(ac.indexer((n,))))
        ac.fn(L, f"cumo_iter_{tname}_pow_int32_s_left_kernel_launch")(ac.scalar(tname, 2), byref(ac.iarray(e)), byref(ac.iarray(o3)), byref(ac.indexer((n,))))
        return [o1, o2, o3]
    a, b = run_both(libs, run)
    for i in range(3):
        assert ac.bits_equal(a[i], b[i]), f"{tname} pow_int32 form {i}"
    # mulsum: the reducing form adds into *p3, the plain form into p3[i]
    y = values(tname, (n,), g, "unit")
    for nan in ((False, True) if tname in FLOATS else (False,)):
        sfx = "_nan" if nan else ""

        def runm(L):
            acc = torch.ones(1, device="cuda", dtype=x.dtype)
            es = x.element_size()
            ac.fn(L, f"cumo_{tname}_mulsum{sfx}_reduce_kernel_launch")(c_void_p(x.data_ptr()), c_void_p(y.data_ptr()), c_void_p(acc.data_ptr()), c_ssize_t(es), c_ssize_t(es), c_uint64(n))
            each = torch.ones(n // 2, device="cuda", dtype=x.dtype)
            ac.fn(L, f"cumo_{tname}_mulsum{sfx}_kernel_launch")(c_void_p(x.data_ptr()), c_void_p(y.data_ptr()), c_void_p(each.data_ptr()), c_ssize_t(2 * es), c_ssize_t(es), c_ssize_t(es), c_uint64(n // 2))
            return [acc, each]
        (a1, a2), (b1, b2) = run_both(libs, runm)
        assert ac.bits_equal(a2, b2)
        if tname in FLOATS:
            assert abs(a1.item() - b1.item()) <= SUM_TOL[tname] * (x.abs().double() * y.abs().double()).sum().item()
        else:
            assert a1.item() == b1.item()


SOURCES = {"sfloat": "float32", "dfloat": "float64", "int64": "int64", "int32": "int32", "int16": "int16", "int8": "int8",
           "uint64": "uint64", "uint32": "uint32", "uint16": "uint16", "uint8": "uint8"}


@pytest.mark.parametrize("dst", TYPES)
def test_store_from_every_source_class(libs, dst):
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(12)
    r, c = 257, 130
    for sname, sdt in SOURCES.items():
        dt = getattr(torch, sdt)
        if dt.is_floating_point:
            src = (torch.randn(c, r, device="cuda", generator=g, dtype=torch.float64) * 100).to(dt)
        else:
            lo = 0 if sdt.startswith("u") else -100
            src = torch.randint(lo, 100, (c, r), device="cuda", generator=g, dtype=torch.int64).to(dt)
        for view in (src.t(), src.t().contiguous()):
            def run(L):
                out = torch.zeros((r, c), device="cuda", dtype=ac.torch_dtype(dst))
                ac.fn(L, f"cumo_iter_{dst}_store_{sname}_kernel_launch")(byref(ac.iarray(out)), byref(ac.iarray(view)), byref(ac.indexer((r, c))))
                return [out]
            (a,), (b,) = run_both(libs, run)
            assert ac.bits_equal(a, b), f"{dst} <- {sname}"


@pytest.mark.parametrize("tname", TYPES)
def test_store_through_index_arrays(libs, tname):
    """cumo_iter_T_store_T_stridx_kernel_launch: a gather (source rows picked by an index array), a scatter, and plain steps."""
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(13)
    src = values(tname, (500, 37), g)
    es = src.element_size()
    pick = torch.randint(0, 500, (211,), device="cuda", generator=g, dtype=torch.int64)
    row_off = pick * (37 * es)                                    # byte offsets of the picked rows
    perm = torch.randperm(211, device="cuda", generator=g).to(torch.int64) * (37 * es)

    def run(L):
        gathered = torch.zeros((211, 37), device="cuda", dtype=src.dtype)
        f = ac.fn(L, f"cumo_iter_{tname}_store_{tname}_stridx_kernel_launch")
        f(byref(ac.stridx_iarray(gathered)), byref(ac.stridx_iarray(src[:211], {0: row_off})), byref(ac.indexer((211, 37))))
        scattered = torch.zeros((211, 37), device="cuda", dtype=src.dtype)
        f(byref(ac.stridx_iarray(scattered, {0: perm})), byref(ac.stridx_iarray(src[:211].t().contiguous().t())), byref(ac.indexer((211, 37))))
        return [gathered, scattered]
    (a1, a2), (b1, b2) = run_both(libs, run)
    assert ac.bits_equal(a1, b1) and ac.bits_equal(a2, b2)
    assert ac.bits_equal(a1, src[pick])


def test_bit_counts_all_four_forms(libs):
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(14)
    n = 50_021
    words = torch.randint(-(1 << 31), 1 << 31, ((3 * n + 40) // 32 + 2,), device="cuda", generator=g, dtype=torch.int64).to(torch.int32)
    idx = (torch.randperm(3 * n, device="cuda", generator=g)[:n]).to(torch.int64)
    for which in ("count_true", "count_false"):
        def run(L):
            total = torch.zeros(2, device="cuda", dtype=torch.int64)
            ac.fn(L, f"cumo_iter_bit_{which}_stride_kernel_launch")(c_size_t(7), c_void_p(total.data_ptr()), c_void_p(words.data_ptr()), c_ssize_t(3), c_uint64(n))
            ac.fn(L, f"cumo_iter_bit_{which}_index_kernel_launch")(c_size_t(7), c_void_p(total.data_ptr() + 8), c_void_p(words.data_ptr()), c_void_p(idx.data_ptr()), c_uint64(n))
            each = torch.zeros(2, n, device="cuda", dtype=torch.int64)
            ac.fn(L, f"cumo_iter_bit_{which}_stride_stride_kernel_launch")(c_size_t(7), c_void_p(each.data_ptr()), c_void_p(words.data_ptr()), c_ssize_t(3), c_ssize_t(8), c_uint64(n))
            ac.fn(L, f"cumo_iter_bit_{which}_index_stride_kernel_launch")(c_size_t(7), c_void_p(each[1].data_ptr()), c_void_p(words.data_ptr()), c_void_p(idx.data_ptr()), c_ssize_t(8), c_uint64(n))
            return [total, each]
        (a1, a2), (b1, b2) = run_both(libs, run)
        assert torch.equal(a1, b1) and torch.equal(a2, b2), which


@pytest.mark.parametrize("tname", ("int32", "int64"))
def test_bincount_forms(libs, tname):
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(15)
    n, bins = 90_001, 700
    items = torch.randint(0, bins, (n,), device="cuda", generator=g, dtype=ac.torch_dtype(tname))
    es = items.element_size()
    byte_idx = torch.randperm(n, device="cuda", generator=g).to(torch.int64) * es          # visit the items in another order
    w32 = torch.randint(0, 8, (n,), device="cuda", generator=g).float()                     # small integers: sums exact in any order
    w64 = w32.double()
    for bits, cdt in (("32", torch.int32), ("64", torch.int64)):
        for use_idx in (False, True):
            def run(L):
                counts = torch.full((bins,), 5, device="cuda", dtype=cdt)
                oor, item = torch.zeros(1, device="cuda", dtype=torch.int32), torch.zeros(1, device="cuda", dtype=torch.int64)
                ac.fn(L, f"cumo_iter_{tname}_bincount_{bits}_kernel_launch")(c_void_p(items.data_ptr()), c_ssize_t(es), c_void_p(byte_idx.data_ptr() if use_idx else None), c_uint64(n),
                                                                              c_void_p(counts.data_ptr()), c_ssize_t(counts.element_size()), c_uint64(bins), c_void_p(oor.data_ptr()), c_void_p(item.data_ptr()))
                return [counts, oor]
            (a, fa), (b, fb) = run_both(libs, run)
            assert torch.equal(a, b) and fa.item() == fb.item() == 0
    for fn_sfx, w in (("sf", w32), ("df", w64)):
        def run(L):
            sums = torch.full((bins,), 5, device="cuda", dtype=w.dtype)
            oor, item = torch.zeros(1, device="cuda", dtype=torch.int32), torch.zeros(1, device="cuda", dtype=torch.int64)
            ac.fn(L, f"cumo_iter_{tname}_bincount_{fn_sfx}_kernel_launch")(c_void_p(items.data_ptr()), c_ssize_t(es), c_void_p(w.data_ptr()), c_ssize_t(w.element_size()), c_uint64(n),
                                                                            c_void_p(sums.data_ptr()), c_ssize_t(w.element_size()), c_uint64(bins), c_void_p(oor.data_ptr()), c_void_p(item.data_ptr()))
            return [sums]
        (a,), (b,) = run_both(libs, run)
        assert torch.equal(a, b)


@pytest.mark.parametrize("tname", TYPES)
def test_cumulative_ops(libs, tname):
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(16)
    n = 150_001
    x = values(tname, (2 * n,), g)
    u = values(tname, (2 * n,), g, "unit")
    es = x.element_size()
    for op, src in (("cumsum", x), ("cumprod", u)):
        for nan in ((False, True) if tname in FLOATS else (False,)):
            s2 = src.clone()
            if nan:
                s2[::50] = float("nan")
            if op == "cumprod" and tname not in FLOATS:
                s2 = torch.ones_like(s2)
                s2[::7] = 2
                s2 = s2[: 2 * 60]

            def run(L):
                m = s2.numel() // 2
                out = torch.zeros(m, device="cuda", dtype=x.dtype)
                rc = ac.fn(L, f"cumo_{tname}_{op}{'_nan' if nan else ''}_kernel_launch", c_int)(c_void_p(s2.data_ptr()), c_void_p(out.data_ptr()), c_ssize_t(2 * es), c_ssize_t(es), c_uint64(m))
                assert rc == 0
                return [out]
            (a,), (b,) = run_both(libs, run)
            if tname in FLOATS:
                if op == "cumsum":
                    scale = s2[::2].nan_to_num().abs().double().cumsum(0)
                    both_nan = torch.isnan(a) & torch.isnan(b)          # a leading NaN stays NaN in the plain scan, and at position 0
                    assert torch.all(((a.double() - b.double()).abs() <= SUM_TOL[tname] * scale + 1e-30) | both_nan), f"{op} nan={nan}"
                else:
                    assert torch.allclose(a.double(), b.double(), rtol=1e-3 if tname == "sfloat" else 1e-9, equal_nan=True)
            else:
                assert torch.equal(a, b)


def test_where_and_mask(libs):
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(17)
    n = 200_017
    words = torch.randint(-(1 << 31), 1 << 31, ((2 * n + 70) // 32 + 2,), device="cuda", generator=g, dtype=torch.int64).to(torch.int32)
    bit_idx = torch.randperm(2 * n, device="cuda", generator=g)[:n].to(torch.int64)
    byte_idx = torch.randperm(n, device="cuda", generator=g).to(torch.int64) * 8

    def run(L):
        new = ac.fn(L, "cumo_bit_where_scratch_new", c_void_p)
        free = ac.fn(L, "cumo_cuda_runtime_free")
        where = ac.fn(L, "cumo_bit_where_kernel_launch")
        mask = ac.fn(L, "cumo_bit_mask_kernel_launch")
        outs = []
        for p, s, idx in ((0, 1, None), (27, 1, None), (5, 2, None), (3, 0, bit_idx)):
            for invert in (0, 1):
                for elmsz, dt in ((4, torch.int32), (8, torch.int64)):
                    scratch = new()
                    out = torch.full((n + 1,), -7, device="cuda", dtype=dt)
                    half = (n // 3) // 32 * 32
                    # two launches continue one result: the cursor lives in the scratch.  The second run starts `half * s`
                    # bits further on, given as a word pointer moved on by whole words with the same small bit position:
                    # the reference's contiguous path shifts a word by the full position (types/bit_kernel.h:45-52 with
                    # where_kernel.cu:69), so it only serves positions inside the first word, and the comparison stays there;
                    # positions beyond it are checked against the host-loop semantics in test_gpu_abi_more.py.
                    where(c_void_p(words.data_ptr()), c_size_t(p), c_ssize_t(s), c_void_p(idx.data_ptr() if idx is not None else None), c_uint64(half), c_int(invert),
                          c_void_p(out.data_ptr()), c_size_t(elmsz), c_uint64(0), c_void_p(scratch))
                    if idx is None:
                        where(c_void_p(words.data_ptr() + 4 * (half * s // 32)), c_size_t(p), c_ssize_t(s), None, c_uint64(n - half), c_int(invert),
                              c_void_p(out.data_ptr()), c_size_t(elmsz), c_uint64(half), c_void_p(scratch))
                    torch.cuda.synchronize()
                    free(c_void_p(scratch))
                    outs.append(out)
        for p, s, idx, p2, s2, idx2 in ((0, 1, None, 16, 8, None), (27, 1, None, 0, -8, None), (3, 0, bit_idx, 0, 0, byte_idx), (5, 2, None, 24, 0, byte_idx)):
            scratch = new()
            out = torch.full((n + 1,), -7, device="cuda", dtype=torch.int64)
            base = 8 * n if s2 < 0 else p2
            mask(c_void_p(words.data_ptr()), c_size_t(p), c_ssize_t(s), c_void_p(idx.data_ptr() if idx is not None else None), c_uint64(n),
                 c_void_p(out.data_ptr()), c_size_t(base), c_ssize_t(s2), c_void_p(idx2.data_ptr() if idx2 is not None else None), c_void_p(scratch))
            torch.cuda.synchronize()
            free(c_void_p(scratch))
            outs.append(out)
        return outs
    a, b = run_both(libs, run)
    for i, (u, v) in enumerate(zip(a, b)):
        if not torch.equal(u, v):
            bad = torch.nonzero(u != v).view(-1)
            k = int(bad[0])
            raise AssertionError(f"case {i}: {bad.numel()} of {u.numel()} differ, first at {k}: ours {u[max(0, k - 2):k + 3].tolist()} reference {v[max(0, k - 2):k + 3].tolist()}")


class _BitStridx(ctypes.Structure):
    """cumo_na_bit_iarray_stridx_t (include/cumo/indexer.h:57-61)."""
    import abi_call as _ac
    _fields_ = [("ptr", c_void_p), ("pos", c_size_t), ("stridx", _ac.Stridx * _ac.MAX_DIM)]


def _bit_stridx(words, pos, steps, index_arrays=None):
    v = _BitStridx()
    v.ptr, v.pos = words.data_ptr(), pos
    for d, s in enumerate(steps):
        ia = (index_arrays or {}).get(d)
        if ia is not None:
            v.stridx[d].index = ia.data_ptr()
        else:
            v.stridx[d].stride = (s << 1) | 1
    return v


def test_bit_operators_and_reductions_word_for_word(libs):
    """Bit o Bit and all? / any? through both launch forms, against the reference's own kernels: contiguous runs at every
    combination of bit offsets around a word boundary, strided / reversed / 2-d / index-array views, the three reduce forms."""
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(21)

    def words(n_words):
        return torch.randint(-(1 << 31), 1 << 31, (n_words,), device="cuda", generator=g, dtype=torch.int64).to(torch.int32)

    n = 70_001
    w1, w2 = words(n // 32 + 4), words(n // 32 + 4)
    base3 = words(n // 32 + 4)
    for op in ("and", "or", "xor", "eq"):
        for p1, p2, p3 in ((0, 0, 0), (5, 5, 5), (0, 7, 31), (31, 0, 1), (13, 29, 2)):
            def run(L):
                out = base3.clone()                     # the bits outside the run must come back untouched
                ac.fn(L, f"cumo_iter_bit_{op}_contiguous_kernel_launch")(c_void_p(w1.data_ptr()), c_size_t(p1), c_void_p(w2.data_ptr()), c_size_t(p2),
                                                                          c_void_p(out.data_ptr()), c_size_t(p3), c_uint64(n))
                return out
            a, b = run_both(libs, run)
            assert torch.equal(a, b), (op, p1, p2, p3)
    for op in ("copy", "not", "store_bit"):
        for p1, p3 in ((0, 0), (9, 9), (3, 30), (30, 3)):
            def run(L):
                out = base3.clone()
                ac.fn(L, f"cumo_iter_bit_{op}_contiguous_kernel_launch")(c_void_p(w1.data_ptr()), c_size_t(p1), c_void_p(out.data_ptr()), c_size_t(p3), c_uint64(n))
                return out
            a, b = run_both(libs, run)
            assert torch.equal(a, b), (op, p1, p3)
    # general views: (rows, cols) with a reversed first operand, a column-strided second one, an index array on the output rows
    rows, cols = 37, 301
    big1, big2 = words(rows * cols * 3 // 32 + 8), words(rows * cols * 3 // 32 + 8)
    row_index = (torch.randperm(rows, device="cuda", generator=g) * (cols + 11)).to(torch.int64)        # bit offsets of the output rows
    shape = (rows, cols)
    for op in ("and", "or", "xor", "eq", "copy", "not", "store_bit"):
        def run(L):
            out = words((rows + 1) * (cols + 11) // 32 + 8)
            v1 = _bit_stridx(big1, 17 + (rows * cols - 1), (-cols, -1))                                  # walks backwards from its last element
            v2 = _bit_stridx(big2, 3, (2 * cols + 5, 2))
            v3 = _bit_stridx(out, 6, (0, 1), {0: row_index})
            ix = ac.indexer(shape)
            if op in ("copy", "not", "store_bit"):
                ac.fn(L, f"cumo_iter_bit_{op}_kernel_launch")(byref(v1), byref(v3), byref(ix))
            else:
                ac.fn(L, f"cumo_iter_bit_{op}_kernel_launch")(byref(v1), byref(v2), byref(v3), byref(ix))
            return out
        # the output's untouched bits differ between the two runs (fresh random words), so compare what was written
        ours, ref = libs
        torch.manual_seed(0)
        state = g.get_state()
        a = run(ours)
        torch.cuda.synchronize()
        g.set_state(state)
        b = run(ref)
        torch.cuda.synchronize()
        assert ref.refk_last_error() == 0
        assert torch.equal(a, b), op
    # all? / any?: one flipping bit at the start, in the middle, at the end, nowhere; the three launch forms
    m = 50_003
    idx = (torch.randperm(3 * m, device="cuda", generator=g)[:m]).to(torch.int64)
    for name, init in (("all_p", 1), ("any_p", 0)):
        for flip_at in (None, 0, m // 2, m - 1):
            src = torch.full((3 * m // 32 + 4,), -1 if init else 0, device="cuda", dtype=torch.int32)
            if flip_at is not None:
                for q in (11 + flip_at, 11 + 3 * flip_at, 11 + int(idx[flip_at])):                     # the contiguous, the strided and the indexed run
                    src[q // 32] ^= (1 << (q % 32)) if q % 32 != 31 else -(1 << 31)

            def run(L):
                out = torch.full((4,), -1 if init else 0, device="cuda", dtype=torch.int32)
                ac.fn(L, f"cumo_iter_bit_{name}_contiguous_reduce_kernel_launch")(c_void_p(src.data_ptr()), c_size_t(11), c_void_p(out.data_ptr()), c_size_t(3), c_uint64(m))
                ac.fn(L, f"cumo_iter_bit_{name}_reduce_kernel_launch")(c_void_p(src.data_ptr()), c_size_t(11), c_ssize_t(3), None, c_void_p(out.data_ptr()), c_size_t(40), c_uint64(m))
                ac.fn(L, f"cumo_iter_bit_{name}_reduce_kernel_launch")(c_void_p(src.data_ptr()), c_size_t(11), c_ssize_t(0), c_void_p(idx.data_ptr()), c_void_p(out.data_ptr()), c_size_t(70), c_uint64(m))
                each = torch.full((m // 32 + 2,), -1 if init else 0, device="cuda", dtype=torch.int32)
                ac.fn(L, f"cumo_iter_bit_{name}_elementwise_kernel_launch")(c_void_p(src.data_ptr()), c_size_t(11), c_ssize_t(3), None, c_void_p(each.data_ptr()), c_size_t(5), c_ssize_t(1), None, c_uint64(m))
                return [out, each]
            (a1, a2), (b1, b2) = run_both(libs, run)
            assert torch.equal(a1, b1) and torch.equal(a2, b2), (name, flip_at)


BIT_SOURCES = {"dfloat": "float64", "sfloat": "float32", "int64": "int64", "int32": "int32", "int16": "int16", "int8": "int8",
               "uint64": "uint64", "uint32": "uint32", "uint16": "uint16", "uint8": "uint8"}


def test_bit_value_conversions_and_fill_word_for_word(libs):
    """value <- Bit, Bit <- value (all ten source classes) and Bit#fill against the reference's own kernels: runs laid end
    to end at several bit offsets (the other bits of the end words must come back untouched), strided and reversed views,
    index arrays on either side."""
    import torch
    import abi_call as ac

    g = torch.Generator(device="cuda").manual_seed(33)

    def words(n_words):
        return torch.randint(-(1 << 31), 1 << 31, (n_words,), device="cuda", generator=g, dtype=torch.int64).to(torch.int32)

    def source(name, shape):
        dt = getattr(torch, BIT_SOURCES[name])
        v = torch.randint(-2, 3, shape, device="cuda", generator=g, dtype=torch.int64)
        if name.startswith("uint"):
            v = v.abs()
        if dt.is_floating_point:
            v = v.to(dt) * 0.5
            flat = v.view(-1)
            flat[3], flat[4], flat[5] = float("nan"), -0.0, float("inf")
            return v
        return v.to(dt)

    n = 70_001
    mask = words(n // 32 + 4)
    ix1 = ac.indexer((n,))
    # value <- Bit
    for tname in TYPES:
        for pos in (0, 5, 31, 37):
            def run(L):
                out = torch.full((n,), 77, device="cuda", dtype=ac.torch_dtype(tname))
                ac.fn(L, f"cumo_iter_{tname}_store_bit_kernel_launch")(byref(ac.stridx_iarray(out)), byref(_bit_stridx(mask, pos, (1,))), byref(ix1))
                return [out]
            (a,), (b,) = run_both(libs, run)
            assert ac.bits_equal(a, b), (tname, pos)
        rows, cols = 37, 301
        big = words(rows * cols * 3 // 32 + 8)
        pick = (torch.randperm(rows, device="cuda", generator=g) * cols * 3).to(torch.int64)              # bit offsets of the rows

        def run(L):
            out = torch.full((rows, 2 * cols), 77, device="cuda", dtype=ac.torch_dtype(tname))
            view = out[:, ::2]
            ac.fn(L, f"cumo_iter_{tname}_store_bit_kernel_launch")(byref(ac.stridx_iarray(view)), byref(_bit_stridx(big, 9, (0, 3), {0: pick})), byref(ac.indexer((rows, cols))))
            rev = torch.full((n,), 77, device="cuda", dtype=ac.torch_dtype(tname))
            d = ac.stridx_iarray(rev)
            d.ptr = rev.data_ptr() + (n - 1) * rev.element_size()
            d.stridx[0].stride = ((-rev.element_size()) << 1) | 1
            ac.fn(L, f"cumo_iter_{tname}_store_bit_kernel_launch")(byref(d), byref(_bit_stridx(mask, 2, (1,))), byref(ix1))
            return [out, rev]
        (a1, a2), (b1, b2) = run_both(libs, run)
        assert ac.bits_equal(a1, b1) and ac.bits_equal(a2, b2), tname
    # Bit <- value
    base = words(n // 32 + 4)
    for sname in BIT_SOURCES:
        src = source(sname, (n,))
        for pos in (0, 5, 31, 37):
            def run(L):
                out = base.clone()
                ac.fn(L, f"cumo_iter_bit_store_{sname}_kernel_launch")(byref(_bit_stridx(out, pos, (1,))), byref(ac.stridx_iarray(src)), byref(ix1))
                return [out]
            (a,), (b,) = run_both(libs, run)
            assert torch.equal(a, b), (sname, pos)
        rows, cols = 37, 301
        src2 = source(sname, (rows, 2 * cols))
        rowpos = (torch.randperm(rows, device="cuda", generator=g) * (cols + 11)).to(torch.int64)

        def run(L):
            out = base.clone()
            ac.fn(L, f"cumo_iter_bit_store_{sname}_kernel_launch")(byref(_bit_stridx(out, 6, (0, 1), {0: rowpos})), byref(ac.stridx_iarray(src2[:, ::2])), byref(ac.indexer((rows, cols))))
            out2 = base.clone()
            ac.fn(L, f"cumo_iter_bit_store_{sname}_kernel_launch")(byref(_bit_stridx(out2, 3 + 2 * (cols - 1), (2 * cols + 5, -2))), byref(ac.stridx_iarray(src2.t()[:cols, :rows].t())), byref(ac.indexer((rows, cols))))
            return [out, out2]
        (a1, a2), (b1, b2) = run_both(libs, run)
        assert torch.equal(a1, b1) and torch.equal(a2, b2), sname
    # fill
    for y in (0, 1):
        for pos, m in ((0, n), (5, n), (31, 2), (37, 27), (3, 64), (0, 32)):
            def run(L):
                o1, o2 = base.clone(), base.clone()
                # the word-at-a-time form takes the run's first word and the offset inside it (tmpl_bit/fill.c calls it so)
                ac.fn(L, "cumo_iter_bit_fill_contiguous_kernel_launch")(c_void_p(o1.data_ptr() + 4 * (pos // 32)), c_size_t(pos % 32), c_uint64(m), ctypes.c_uint32(0xffffffff if y else 0))
                ac.fn(L, "cumo_iter_bit_fill_kernel_launch")(byref(_bit_stridx(o2, pos, (1,))), ctypes.c_uint32(y), byref(ac.indexer((m,))))
                return [o1, o2]
            (a1, a2), (b1, b2) = run_both(libs, run)
            assert torch.equal(a1, b1) and torch.equal(a2, b2) and torch.equal(a1, a2), (y, pos, m)
        rows, cols = 37, 301
        rowpos = (torch.randperm(rows, device="cuda", generator=g) * (cols * 2 + 11)).to(torch.int64)

        def run(L):
            out = base.clone()
            ac.fn(L, "cumo_iter_bit_fill_kernel_launch")(byref(_bit_stridx(out, 6, (0, 2), {0: rowpos})), ctypes.c_uint32(y), byref(ac.indexer((rows, cols))))
            return [out]
        (a,), (b,) = run_both(libs, run)
        assert torch.equal(a, b), y


@pytest.mark.parametrize("tname", TYPES)
def test_poly_and_eye_bit_for_bit(libs, tname):
    """Horner over array and repeated coefficients on several layouts, and the diagonal fill through a strided matrix."""
    import torch
    import abi_call as ac
    from cumo_b200 import _lib

    g = torch.Generator(device="cuda").manual_seed(77)
    kind = "unit" if tname not in FLOATS else "normal"
    for layout in ("flat", "transposed", "view3d"):
        x, c_full, shape = operands(tname, layout, g, kind)
        scalar_c = values(tname, (1,), g, kind)
        row_c = values(tname, (shape[-1],), g, kind)
        for ncoef in (0, 1, 2, 4):
            coefs = [c_full, scalar_c, row_c, scalar_c][:ncoef]

            def run(L):
                out = torch.full(shape, 77, device="cuda", dtype=x.dtype)
                arr = (_lib.NaIArray * max(1, ncoef))()
                for i, c in enumerate(coefs):
                    arr[i] = ac.iarray(c, shape)
                ac.fn(L, f"cumo_iter_{tname}_poly_kernel_launch")(byref(ac.iarray(x, shape)), arr, c_int(ncoef), byref(ac.iarray(out)), byref(ac.indexer(shape)))
                return [out]
            (a,), (b,) = run_both(libs, run)
            assert ac.bits_equal(a, b), (tname, layout, ncoef)
    for kofs in (0, 1, -2, 5):
        def run(L):
            base = torch.full((40, 2 * 37), 77, device="cuda", dtype=ac.torch_dtype(tname))
            m = base[3:33, ::2]                                             # 30 x 37, columns two elements apart
            es = base.element_size()
            ac.fn(L, f"cumo_iter_{tname}_eye_stride_kernel_launch")(c_void_p(m.data_ptr()), c_ssize_t(m.stride(0) * es), c_ssize_t(m.stride(1) * es),
                                                                      c_ssize_t(kofs), ac.scalar(tname, 3), c_uint64(30), c_uint64(37))
            return [base]
        (a,), (b,) = run_both(libs, run)
        assert ac.bits_equal(a, b), (tname, kofs)
