"""Run one named kernel case on synthetic device data, a few launches, and print its timing.

    python -m cumo_b200.cases --case exp --mib 512 --reps 3

This is the small, self-ending command that profiler captures are taken on (one kernel,
a few launches, a few hundred MiB on the device) and a quick way to time a single kernel
outside bench.py.  `--mib` is the size of the main input array.
"""
from __future__ import annotations

import argparse

import numpy as np


def build_cases(xp, torch, mib: int):
    g = torch.Generator(device="cuda").manual_seed(0)
    n32 = mib * (1 << 20) // 4
    n64 = mib * (1 << 20) // 8
    cols = 4096
    rows32, rows64 = max(1, n32 // cols), max(1, n64 // cols)
    cache = {}

    def f32():
        if "f32" not in cache:
            cache["f32"] = xp.SFloat.from_torch(torch.rand(rows32 * cols, device="cuda", generator=g) * 2 - 1)
        return cache["f32"]

    def f64():
        if "f64" not in cache:
            cache["f64"] = xp.DFloat.from_torch(torch.rand(rows64 * cols, device="cuda", dtype=torch.float64, generator=g))
        return cache["f64"]

    def i32():
        if "i32" not in cache:
            cache["i32"] = xp.Int32.from_torch(torch.randint(-(1 << 20), 1 << 20, (rows32 * cols,), device="cuda", dtype=torch.int32, generator=g))
        return cache["i32"]

    def outer():
        r = max(1, n32 // 16384)
        x = xp.SFloat.from_torch(torch.randn(r, 1, device="cuda", generator=g))
        y = xp.SFloat.from_torch(torch.randn(1, 16384, device="cuda", generator=g))
        return x, y

    def col():
        a = f32().reshape(rows32, cols)
        return a, a.sum(axis=1).reshape(rows32, 1)

    def km():
        from . import kmeans
        n, d, k = n32 // 64, 64, 256
        cen = torch.randn(k, d, device="cuda", generator=g) * 4
        pts = cen[torch.randint(0, k, (n,), device="cuda", generator=g)] + torch.randn(n, d, device="cuda", generator=g)
        return kmeans, xp.SFloat.from_torch(pts), xp.SFloat.from_torch(cen)

    def gemm():
        from . import linalg
        m, k, n = max(128, n32 // 4096), 4096, 4096
        a = xp.SFloat.from_torch(torch.randn(m, k, device="cuda", generator=g))
        bt = xp.SFloat.from_torch(torch.randn(n, k, device="cuda", generator=g))
        return linalg, a, bt

    cases = {
        # name: (setup -> callable, algorithmic bytes)
        "exp": (lambda: (lambda a=f32(): xp.NMath.exp(a)), 2 * n32 * 4),
        "mul_scalar": (lambda: (lambda a=f32(): a * 0.5), 2 * n32 * 4),
        "mul": (lambda: (lambda a=f32(): a * a), 3 * n32 * 4),
        "outer_add": (lambda: (lambda xy=outer(): xy[0] + xy[1]), n32 * 4),
        "add_col": (lambda: (lambda ac=col(): ac[0] + ac[1]), 2 * n32 * 4),
        "sum_axis1_sq_f32": (lambda: (lambda a=f32()[0:(int((rows32 * cols) ** 0.5) // 64 * 64) ** 2].reshape(int((rows32 * cols) ** 0.5) // 64 * 64, -1): a.sum(axis=1)), (int((rows32 * cols) ** 0.5) // 64 * 64) ** 2 * 4),
        "mul_row": (lambda: (lambda a=f32().reshape(rows32, cols), w=f32()[0:cols].reshape(1, cols): a * w), 2 * n32 * 4),
        "sum_f32": (lambda: (lambda a=f32(): a.sum()), n32 * 4),
        "sum_f64": (lambda: (lambda a=f64(): a.sum()), n64 * 8),
        "max_f64": (lambda: (lambda a=f64(): a.max()), n64 * 8),
        "argmax_f32": (lambda: (lambda a=f32(): a.argmax()), n32 * 4),
        "sum_axis0_f32": (lambda: (lambda a=f32().reshape(rows32, cols): a.sum(axis=0)), n32 * 4),
        "sum_axis1_f32": (lambda: (lambda a=f32().reshape(rows32, cols): a.sum(axis=1)), n32 * 4),
        "max_index_axis1_f32": (lambda: (lambda a=f32().reshape(rows32, cols): a.max_index(axis=1)), n32 * 4),
        "argmax_axis0_f32": (lambda: (lambda a=f32().reshape(rows32, cols): a.argmax(axis=0)), n32 * 4),
        "gt_scalar_i32": (lambda: (lambda a=i32(): a > 0), n32 * 4 + n32 // 8),
        "count_true": (lambda: (lambda m=(i32() > 0): m.count_true()), n32 // 8),
        "mod_scalar_i32": (lambda: (lambda a=i32(): a % 7), 2 * n32 * 4),
        "cumsum_f32": (lambda: (lambda a=f32(): a.cumsum()), 2 * n32 * 4),
        "bincount_i32": (lambda: (lambda a=xp.Int32.from_torch(torch.randint(0, 256, (rows32 * cols,), device="cuda", dtype=torch.int32, generator=g)): a.bincount()), n32 * 4 + 1024),
        "where_bits": (lambda: (lambda m=(i32() > 0): m.where()), n32 // 8 + (n32 // 2) * 4),
        "gemm_tc": (lambda: (lambda m=gemm(): m[0].gemm_nt(m[1], m[2])), n32 * 4 + 4096 * 4096 * 4 + n32 * 4),
        "kmeans_tensor": (lambda: (lambda m=km(): m[0].assign(m[1], m[2], algo="tensor")), n32 * 4 + n32 // 16),
        "kmeans_cores": (lambda: (lambda m=km(): m[0].assign(m[1], m[2], algo="cores")), n32 * 4 + n32 // 16),
        "sum_i32": (lambda: (lambda a=i32(): a.sum()), n32 * 4),
    }
    return cases


def main():
    import torch

    import cumo_b200 as xp

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--case", required=True)
    ap.add_argument("--mib", type=int, default=512)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--warm", type=int, default=1)
    a = ap.parse_args()
    torch.cuda.set_device(0)
    cases = build_cases(xp, torch, a.mib)
    if a.case == "list":
        print(" ".join(cases))
        return
    setup, nbytes = cases[a.case]
    fn = setup()
    for _ in range(a.warm):
        fn()
    ts = []
    hold = getattr(torch.cuda, "_sleep", None)
    for _ in range(a.reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if hold is not None:
            hold(400_000)        # keeps the device busy ~0.2 ms so the call is enqueued before the first event fires
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    med = float(np.median(ts))
    print(f"{a.case}: {a.mib} MiB input, {nbytes} algorithmic bytes, median {med:.4f} ms over {a.reps} launches, {nbytes / (med * 1e-3) / 1e9:.1f} GB/s")


if __name__ == "__main__":
    main()
