"""k-means assignment step on device arrays, single GPU or row-sharded.

The reference expresses the step with array operations (bench/kmeans_bench.rb:108-126); this is the
fused form of the same arithmetic: labels = argmin_k(|c_k|^2 - 2 <x, c_k>), lowest index on ties,
and the population of every cluster.  Two kernels compute it: `cb200_kmeans_assign_sfloat_tc`
(tcgen05 tensor cores, split-TF32, for D a multiple of 32 and K <= 256 that fit shared memory) and
`cb200_kmeans_assign_sfloat` (fp32 FMA, any D multiple of 4).
"""
from __future__ import annotations

from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p, create_string_buffer

from . import _lib
from .narray import CumoError, Int32, SFloat, UInt64


def tensor_core_form_fits(d: int, k: int) -> bool:
    n_pad = (k + 15) // 16 * 16
    return d >= 32 and d % 32 == 0 and 1 <= k <= 256 and 2 * (d // 32) * n_pad * 128 + 3 * 32768 + 8 * n_pad + 104 <= 227 * 1024


def assign(x: SFloat, c: SFloat, want_min_dist: bool = False, algo: str = "auto"):
    """x (N, D), c (K, D), both SFloat -> (labels Int32[N], counts UInt64[K][, min_dist SFloat[N]]).
    algo: "tensor" (tcgen05), "cores" (fp32 FMA) or "auto" (tensor when the shape allows it)."""
    if not (isinstance(x, SFloat) and isinstance(c, SFloat) and x.ndim == 2 and c.ndim == 2 and x.shape[1] == c.shape[1]):
        raise TypeError("assign needs SFloat x (N, D) and c (K, D)")
    if not x.contiguous():
        x = x.dup()
    if not c.contiguous():
        c = c.dup()
    n, d = x.shape
    k = c.shape[0]
    if algo == "auto":
        algo = "tensor" if tensor_core_form_fits(d, k) else "cores"
    if algo not in ("tensor", "cores"):
        raise ValueError("algo must be 'auto', 'tensor' or 'cores'")
    lib = _lib.load()
    fn = lib.cb200_kmeans_assign_sfloat_tc if algo == "tensor" else lib.cb200_kmeans_assign_sfloat
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int64, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_char_p, c_size_t]
    labels = Int32(n)
    counts = UInt64.zeros(k)
    dist = SFloat(n) if want_min_dist else None
    err = create_string_buffer(256)
    if fn(x.data_ptr, n, d, c.data_ptr, k, labels.data_ptr, dist.data_ptr if dist is not None else None, counts.data_ptr, err, len(err)):
        raise CumoError(err.value.decode())
    return (labels, counts, dist) if want_min_dist else (labels, counts)


def assign_sharded(comm, x_local: SFloat, c: SFloat, algo: str = "auto"):
    """Points row-sharded over the ranks of `comm`, centroids replicated: local labels, global counts.
    The per-cluster counts are integers, so their all_reduce(SUM) is exact and order independent."""
    labels, counts = assign(x_local, c, algo=algo)
    return labels, comm.all_reduce_sum(counts)
