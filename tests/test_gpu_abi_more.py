"""Entry points of the C ABI that the method-level tests do not reach, called with hand-filled descriptors and
checked against the CPU oracle: kahan_sum, pow with an Int32 exponent array and with a host numeric base, ldexp,
the index forms of the Bit counts, bincount through an index array, where through an index array, Bit#mask,
the same-type store through index arrays, and the store from the narrow and unsigned integer classes.
"""
from ctypes import byref, c_int, c_int32, c_size_t, c_ssize_t, c_uint64, c_void_p

import numpy as np
import pytest

from oracle import cumo_oracle as orc

pytestmark = pytest.mark.gpu

NP = {"sfloat": np.float32, "dfloat": np.float64, "int32": np.int32, "int64": np.int64}


@pytest.fixture(scope="module")
def L():
    from cumo_b200 import _lib

    return _lib.load()


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_kahan_sum_against_the_oracle_and_float64(L):
    """cumo_dfloat_kahan_sum[_nan]_kernel_launch: the oracle's Kahan loop (types/real_accum.h f_kahan_sum) and a
    float64 pairwise sum bound it to 1e-12 of the sum of magnitudes; values of mixed magnitude make a plain sum lose digits."""
    import torch
    import abi_call as ac

    rng = np.random.default_rng(0)
    h = (rng.standard_normal((300, 5000)) * 10.0 ** rng.integers(-6, 7, (300, 5000))).astype(np.float64)
    hn = h.copy()
    hn[:, ::17] = np.nan
    for nan, host in ((False, h), (True, hn)):
        for axes in ((1,), (0,), (0, 1)):
            src = dev(host)
            out = torch.zeros([n for d, n in enumerate(host.shape) if d not in axes], device="cuda", dtype=torch.float64)
            ac.fn(L, f"cumo_dfloat_kahan_sum{'_nan' if nan else ''}_kernel_launch")(byref(ac.reduction_arg(src, out, axes)))
            torch.cuda.synchronize()
            want = orc.reduce("kahan_sum", host, axis=axes, nan=nan)
            scale = np.nansum(np.abs(host), axis=axes)
            assert np.all(np.abs(out.cpu().numpy() - want) <= 1e-12 * scale)
            ref = np.nansum(host, axis=axes) if nan else host.sum(axis=axes)
            assert np.all(np.abs(out.cpu().numpy() - ref) <= 1e-12 * scale)


@pytest.mark.parametrize("tname", list(NP))
def test_pow_with_an_int32_exponent(L, tname):
    """cumo_iter_T_pow_int32_kernel_launch (exponent array), _s (host exponent), _s_left (host base): repeated
    multiplication, bit for bit (float_macro_kernel.h:126-149 / xint_macro_kernel.h pow_int)."""
    import torch
    import abi_call as ac

    rng = np.random.default_rng(1)
    dt = NP[tname]
    shape = (123, 77)
    x = (rng.uniform(-2, 2, shape)).astype(dt) if tname.endswith("float") else rng.integers(-6, 7, shape).astype(dt)
    e = rng.integers(0, 9, shape).astype(np.int32)
    gx, ge = dev(x), dev(e)
    # a column-sliced base, an exponent that is one row repeated
    xv, ev = gx[:, 3:70], ge[5:6, 3:70]
    o = torch.zeros((123, 67), device="cuda", dtype=gx.dtype)
    ac.fn(L, f"cumo_iter_{tname}_pow_int32_kernel_launch")(byref(ac.iarray(xv)), byref(ac.iarray(ev, (123, 67))), byref(ac.iarray(o)), byref(ac.indexer((123, 67))))
    torch.cuda.synchronize()
    assert np.array_equal(o.cpu().numpy(), orc.pow_int32(x[:, 3:70], np.broadcast_to(e[5:6, 3:70], (123, 67))))
    o2 = torch.zeros(shape, device="cuda", dtype=gx.dtype)
    ac.fn(L, f"cumo_iter_{tname}_pow_int32_s_kernel_launch")(byref(ac.iarray(gx)), c_int32(3), byref(ac.iarray(o2)), byref(ac.indexer(shape)))
    o3 = torch.zeros(shape, device="cuda", dtype=gx.dtype)
    ac.fn(L, f"cumo_iter_{tname}_pow_int32_s_left_kernel_launch")(ac.scalar(tname, 3), byref(ac.iarray(ge)), byref(ac.iarray(o3)), byref(ac.indexer(shape)))
    torch.cuda.synchronize()
    assert np.array_equal(o2.cpu().numpy(), orc.pow_int32(x, 3))
    assert np.array_equal(o3.cpu().numpy(), orc.pow_int32(dt(3), e))


@pytest.mark.parametrize("tname", ("sfloat", "dfloat"))
def test_ldexp_array_and_scalar_forms(L, tname):
    """cumo_iter_T_math_s_ldexp[_s]_kernel_launch: x * 2**(int)y, exact in both precisions."""
    import torch
    import abi_call as ac

    rng = np.random.default_rng(2)
    dt = NP[tname]
    x = rng.standard_normal(50_001).astype(dt)
    y = rng.integers(-30, 31, 50_001).astype(dt)
    gx, gy = dev(x), dev(y)
    o = torch.zeros_like(gx)
    ac.fn(L, f"cumo_iter_{tname}_math_s_ldexp_kernel_launch")(byref(ac.iarray(gx)), byref(ac.iarray(gy)), byref(ac.iarray(o)), byref(ac.indexer(x.shape)))
    torch.cuda.synchronize()
    assert np.array_equal(o.cpu().numpy(), orc.binary("ldexp", x, y)[0])
    assert np.array_equal(o.cpu().numpy(), np.ldexp(x, y.astype(np.int32)).astype(dt))
    for left, want in ((0, np.ldexp(x, 5)), (1, np.ldexp(dt(5), y.astype(np.int32)))):
        o = torch.zeros_like(gx)
        ac.fn(L, f"cumo_iter_{tname}_math_s_ldexp_s_kernel_launch")(byref(ac.iarray(gy if left else gx)), byref(ac.iarray(o)), byref(ac.indexer(x.shape)), ac.scalar(tname, 5), c_int(left))
        torch.cuda.synchronize()
        assert np.array_equal(o.cpu().numpy(), want.astype(dt)), f"scalar_is_left={left}"


def test_bit_counts_through_an_index_array(L):
    """cumo_iter_bit_count_{true,false}_{index,index_stride,stride_stride}_kernel_launch against unpacked bits."""
    import torch
    import abi_call as ac

    rng = np.random.default_rng(3)
    nbits, n = 100_000, 31_007
    words = rng.integers(0, 2 ** 32, nbits // 32, dtype=np.uint64).astype(np.uint32)
    bits = np.unpackbits(words.view(np.uint8), bitorder="little")
    idx = rng.choice(nbits - 64, n, replace=False).astype(np.int64)
    gw, gi = dev(words.view(np.int32)), dev(idx)
    p1 = 11
    picked = bits[p1 + idx]
    strided = bits[p1 + 3 * np.arange(n)]
    for which, want_bit in (("count_true", 1), ("count_false", 0)):
        tot = torch.zeros(1, device="cuda", dtype=torch.int64)
        ac.fn(L, f"cumo_iter_bit_{which}_index_kernel_launch")(c_size_t(p1), c_void_p(tot.data_ptr()), c_void_p(gw.data_ptr()), c_void_p(gi.data_ptr()), c_uint64(n))
        each_i = torch.zeros(n, device="cuda", dtype=torch.int64)
        ac.fn(L, f"cumo_iter_bit_{which}_index_stride_kernel_launch")(c_size_t(p1), c_void_p(each_i.data_ptr()), c_void_p(gw.data_ptr()), c_void_p(gi.data_ptr()), c_ssize_t(8), c_uint64(n))
        each_s = torch.zeros(2 * n, device="cuda", dtype=torch.int64)
        ac.fn(L, f"cumo_iter_bit_{which}_stride_stride_kernel_launch")(c_size_t(p1), c_void_p(each_s.data_ptr()), c_void_p(gw.data_ptr()), c_ssize_t(3), c_ssize_t(16), c_uint64(n))
        torch.cuda.synchronize()
        assert tot.item() == int((picked == want_bit).sum())
        assert np.array_equal(each_i.cpu().numpy(), (picked == want_bit).astype(np.int64))
        assert np.array_equal(each_s.cpu().numpy()[::2], (strided == want_bit).astype(np.int64))
        assert not each_s.cpu().numpy()[1::2].any()


@pytest.mark.parametrize("tname", ("int32", "int64"))
def test_bincount_through_an_index_array(L, tname):
    """The idx1 != NULL form of cumo_iter_T_bincount_{32,64}_kernel_launch: items are read at byte offsets idx1[i]."""
    import torch
    import abi_call as ac

    rng = np.random.default_rng(4)
    dt = NP[tname]
    items = rng.integers(0, 500, 40_000).astype(dt)
    pick = rng.integers(0, 40_000, 25_001).astype(np.int64)
    gi, gp = dev(items), dev(pick * items.itemsize)
    for bits, cdt, tdt in (("32", np.uint32, "int32"), ("64", np.uint64, "int64")):
        counts = torch.full((500,), 3, device="cuda", dtype=getattr(torch, tdt))
        oor, item = torch.zeros(1, device="cuda", dtype=torch.int32), torch.zeros(1, device="cuda", dtype=torch.int64)
        ac.fn(L, f"cumo_iter_{tname}_bincount_{bits}_kernel_launch")(c_void_p(gi.data_ptr()), c_ssize_t(0), c_void_p(gp.data_ptr()), c_uint64(len(pick)), c_void_p(counts.data_ptr()),
                                                                      c_ssize_t(counts.element_size()), c_uint64(500), c_void_p(oor.data_ptr()), c_void_p(item.data_ptr()))
        torch.cuda.synchronize()
        assert oor.item() == 0
        assert np.array_equal(counts.cpu().numpy().astype(np.uint64), orc.bincount(items[pick], minlength=500).astype(np.uint64))


def test_where_through_an_index_array_and_mask(L):
    """cumo_bit_where_kernel_launch with idx != NULL (element i is bit p + idx[i]) and cumo_bit_mask_kernel_launch in its
    four addressing combinations (mask_kernel.cu:6-36): the byte positions of the masked array's kept elements."""
    import torch
    import abi_call as ac

    rng = np.random.default_rng(5)
    nbits, n = 400_000, 120_011
    words = rng.integers(0, 2 ** 32, nbits // 32, dtype=np.uint64).astype(np.uint32)
    bits = np.unpackbits(words.view(np.uint8), bitorder="little").astype(bool)
    idx = rng.choice(nbits - 40, n, replace=False).astype(np.int64)
    gw, gi = dev(words.view(np.int32)), dev(idx)
    new, free = ac.fn(L, "cumo_bit_where_scratch_new", c_void_p), ac.fn(L, "cumo_cuda_runtime_free")
    for invert in (0, 1):
        sel = bits[9 + idx] ^ bool(invert)
        scratch = new()
        out = torch.full((n,), -1, device="cuda", dtype=torch.int64)
        ac.fn(L, "cumo_bit_where_kernel_launch")(c_void_p(gw.data_ptr()), c_size_t(9), c_ssize_t(0), c_void_p(gi.data_ptr()), c_uint64(n), c_int(invert),
                                                 c_void_p(out.data_ptr()), c_size_t(8), c_uint64(1000), c_void_p(scratch))
        torch.cuda.synchronize()
        free(c_void_p(scratch))
        hits = int(sel.sum())
        assert np.array_equal(out.cpu().numpy()[:hits], 1000 + np.nonzero(sel)[0])
        assert (out.cpu().numpy()[hits:] == -1).all()
    byte_idx = rng.permutation(n).astype(np.int64) * 4
    gb = dev(byte_idx)
    e = np.arange(n)
    cases = [((5, 1, None), (64, 4, None), bits[5 + e], 64 + 4 * e),                      # contiguous mask over a contiguous array
             ((5, 3, None), (4 * n, -4, None), bits[5 + 3 * e], 4 * n - 4 * e),             # strided mask, array walked backwards
             ((9, 0, gi), (16, 0, gb), bits[9 + idx], 16 + byte_idx),                      # both through index arrays
             ((0, 2, None), (0, 0, gb), bits[2 * e], byte_idx)]
    for (p, s, ia), (p2, s2, ib), sel, pos in cases:
        scratch = new()
        out = torch.full((n,), -1, device="cuda", dtype=torch.int64)
        half = n // 2
        mask = ac.fn(L, "cumo_bit_mask_kernel_launch")
        if ia is None and ib is None:                                                       # two launches continue one result
            mask(c_void_p(gw.data_ptr()), c_size_t(p), c_ssize_t(s), None, c_uint64(half), c_void_p(out.data_ptr()), c_size_t(p2), c_ssize_t(s2), None, c_void_p(scratch))
            mask(c_void_p(gw.data_ptr()), c_size_t(p + half * s), c_ssize_t(s), None, c_uint64(n - half), c_void_p(out.data_ptr()), c_size_t(p2 + half * s2), c_ssize_t(s2), None, c_void_p(scratch))
        else:
            mask(c_void_p(gw.data_ptr()), c_size_t(p), c_ssize_t(s), c_void_p(ia.data_ptr() if ia is not None else None), c_uint64(n), c_void_p(out.data_ptr()),
                 c_size_t(p2), c_ssize_t(s2), c_void_p(ib.data_ptr() if ib is not None else None), c_void_p(scratch))
        torch.cuda.synchronize()
        free(c_void_p(scratch))
        hits = int(sel.sum())
        assert np.array_equal(out.cpu().numpy()[:hits], pos[sel])


@pytest.mark.parametrize("tname", list(NP))
def test_masked_gather_end_to_end(L, tname):
    """x[mask] materialised the way the extension does it: Bit#mask builds the index array of a 1-D view, the
    same-type stridx store copies the view out (gen/tmpl_bit/mask.c:95-140, store_from.c:82-89)."""
    import torch
    import abi_call as ac

    rng = np.random.default_rng(6)
    dt = NP[tname]
    h = rng.integers(-1000, 1000, (300, 217)).astype(dt)
    keep = rng.random((300, 217)) < 0.3
    words = np.packbits(keep.reshape(-1), bitorder="little")
    words = np.concatenate([words, np.zeros((-len(words)) % 4, np.uint8)]).view(np.int32)
    gx, gw = dev(h), dev(words)
    n, hits = h.size, int(keep.sum())
    new, free = ac.fn(L, "cumo_bit_where_scratch_new", c_void_p), ac.fn(L, "cumo_cuda_runtime_free")
    scratch = new()
    positions = torch.empty(hits, device="cuda", dtype=torch.int64)
    ac.fn(L, "cumo_bit_mask_kernel_launch")(c_void_p(gw.data_ptr()), c_size_t(0), c_ssize_t(1), None, c_uint64(n), c_void_p(positions.data_ptr()),
                                            c_size_t(0), c_ssize_t(h.itemsize), None, c_void_p(scratch))
    free(c_void_p(scratch))
    out = torch.zeros(hits, device="cuda", dtype=gx.dtype)
    ac.fn(L, f"cumo_iter_{tname}_store_{tname}_stridx_kernel_launch")(byref(ac.stridx_iarray(out)), byref(ac.stridx_iarray(gx.view(-1)[:hits], {0: positions})), byref(ac.indexer((hits,))))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), h[keep])
    # scatter back through the same index array into a zeroed array: x[mask] = values
    back = torch.zeros_like(gx)
    ac.fn(L, f"cumo_iter_{tname}_store_{tname}_stridx_kernel_launch")(byref(ac.stridx_iarray(back.view(-1)[:hits], {0: positions})), byref(ac.stridx_iarray(out)), byref(ac.indexer((hits,))))
    torch.cuda.synchronize()
    assert np.array_equal(back.cpu().numpy(), np.where(keep, h, 0))


@pytest.mark.parametrize("dst", list(NP))
def test_store_from_the_narrow_and_unsigned_classes(L, dst):
    """cumo_iter_T_store_{int8,int16,uint8,uint16,uint32,uint64}_kernel_launch: plain C conversions (m_from_sint,
    m_from_uint32, m_from_uint64), contiguous and transposed sources."""
    import torch
    import abi_call as ac

    rng = np.random.default_rng(7)
    for sname, sdt in (("int8", np.int8), ("int16", np.int16), ("uint8", np.uint8), ("uint16", np.uint16), ("uint32", np.uint32), ("uint64", np.uint64)):
        info = np.iinfo(sdt)
        hi = min(int(info.max), 2 ** 31 - 1)
        h = rng.integers(int(info.min), hi, (130, 61), endpoint=True).astype(sdt)
        g = dev(h.view(np.dtype(f"int{8 * h.itemsize}")))          # torch carries the bytes; the library is told the real type by the symbol
        for src, want_src in ((g, h), (g.t(), h.T)):
            out = torch.zeros(want_src.shape, device="cuda", dtype=getattr(torch, np.dtype(NP[dst]).name))
            ac.fn(L, f"cumo_iter_{dst}_store_{sname}_kernel_launch")(byref(ac.iarray(out)), byref(ac.iarray(src)), byref(ac.indexer(want_src.shape)))
            torch.cuda.synchronize()
            assert np.array_equal(out.cpu().numpy(), want_src.astype(NP[dst])), f"{dst} <- {sname}"
