"""k-means assignment step on device arrays (`cb200_kmeans_assign_sfloat`), single GPU or row-sharded.

The reference expresses the step with array operations (bench/kmeans_bench.rb:108-126); this is the
fused form of the same arithmetic: labels = argmin_k(|c_k|^2 - 2 <x, c_k>), lowest index on ties,
and the population of every cluster.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p, create_string_buffer

from . import _lib
from .narray import Int32, NArray, SFloat, UInt64, CumoError


def assign(x: SFloat, c: SFloat, want_min_dist: bool = False):
    """x (N, D), c (K, D), both contiguous SFloat -> (labels Int32[N], counts UInt64[K][, min_dist SFloat[N]])."""
    if not (isinstance(x, SFloat) and isinstance(c, SFloat) and x.ndim == 2 and c.ndim == 2 and x.shape[1] == c.shape[1]):
        raise TypeError("assign needs SFloat x (N, D) and c (K, D)")
    if not (x.contiguous() and c.contiguous()):
        x, c = x.dup(), c.dup()
    lib = _lib.load()
    fn = lib.cb200_kmeans_assign_sfloat
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int64, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_char_p, c_size_t]
    n, d = x.shape
    k = c.shape[0]
    labels = Int32(n)
    counts = UInt64.zeros(k)
    dist = SFloat(n) if want_min_dist else None
    err = create_string_buffer(256)
    if fn(x.data_ptr, n, d, c.data_ptr, k, labels.data_ptr, dist.data_ptr if dist is not None else None, counts.data_ptr, err, len(err)):
        raise CumoError(err.value.decode())
    return (labels, counts, dist) if want_min_dist else (labels, counts)


def assign_sharded(comm, x_local: SFloat, c: SFloat):
    """Points row-sharded over the ranks of `comm`, centroids replicated: local labels, global counts.
    The per-cluster counts are integers, so their all_reduce(SUM) is exact and order independent."""
    labels, counts = assign(x_local, c)
    return labels, comm.all_reduce_sum(counts)
