"""Benchmark of the hot path: effective HBM GB/s of the broadcast-elementwise chain.

A step is one pass of BASELINE config 1 over one batch of synthetic input on each GPU:
    t = x(8192,1) + y(1,16384);  u = NMath.exp(t);  r = u * 0.5          (fp32, 512 MiB outputs)
i.e. three kernels of libcumo_b200 reached through the reference-facing API (cumo_b200.narray ->
host layer -> `cumo_iter_sfloat_*_kernel_launch`).  `value` is the algorithmic bytes of the three
kernels (each distinct input element once, each output element once) over all GPUs divided by
the device time of the timed steps, inputs resident in HBM.  `e2e` is the same chain with the
inputs coming from pinned host memory and the result read back to pinned host memory inside the
timed region.  With --gpus N (launched by torch.distributed.run) every rank runs the same workload
on its own GPU (weak scaling, no data-path collective: rows are independent), and rank 0 also
times the row-sharded full reduction that does need a collective and reports it under `sharded`.

`--impl reference` times the CPU restatement of the reference's host loops (oracle/, all host
threads) on a bounded sample of the same workload and prints the same line with impl=reference.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

R, C = 8192, 16384                      # BASELINE config 1
ES = 4
BYTES_ADD = R * C * ES + (R + C) * ES   # outer broadcast add: output + the two vectors
BYTES_EXP = 2 * R * C * ES
BYTES_MUL = 2 * R * C * ES
BYTES_STEP = BYTES_ADD + BYTES_EXP + BYTES_MUL
METRIC = "effective HBM GB/s, fp32 broadcast-elementwise chain x(8192,1)+y(1,16384) -> exp -> *0.5"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one ew_row_kernel<Exp<float>,4> launch on this workload, from one
# ncu capture of `bench.py --case exp --mib 512` (the same 512 MiB in / 512 MiB out launch); the line says so.
EXP_KERNEL_DRAM_TRAFFIC_BYTES = 536890624 + 485002240


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def oracle_chain(hx, hy, rows):
    """The chain on the first `rows` rows with the CPU oracle; returns seconds."""
    sys.path.insert(0, str(ROOT / "tests"))
    from oracle_narray import OracleXP as ox

    x, y = ox.SFloat.cast(hx[:rows]), ox.SFloat.cast(hy)
    t0 = time.perf_counter()
    r = ox.NMath.exp(x + y) * 0.5
    dt = time.perf_counter() - t0
    assert r.shape == (rows, C)
    return dt


def sample_bytes(rows):
    return (rows * C * ES + (rows + C) * ES) + 4 * rows * C * ES


def run_reference(args):
    """Reference arm: the reference's CPU algorithm (oracle port), all host threads, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import cumo_oracle as orc

    cores = os.cpu_count() or 1
    orc.set_threads(cores)
    rng = np.random.default_rng(1)
    hx = rng.standard_normal((R, 1)).astype(np.float32)
    hy = rng.standard_normal((1, C)).astype(np.float32)
    rows = 1024                                    # 1/8 of the workload per step
    for _ in range(args.warmup):
        oracle_chain(hx, hy, rows)
    t = [oracle_chain(hx, hy, rows) for _ in range(args.steps)]
    sec = float(np.sum(t))
    value = sample_bytes(rows) * args.steps / sec / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": sec / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "BASELINE config 1: x(8192,1)+y(1,16384), exp, *0.5 (fp32)", "sample": f"first {rows} of {R} rows per step"},
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": orc.threads(), "kind": "port",
                             "sample": f"{rows} of {R} rows per step, {args.steps} steps, CPU restatement of the reference's host loops (no Ruby here to run Numo)"},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def time_kernel(torch, fn, reps=10, warm=2):
    """Median / min device time (ms) of fn() measured launch by launch with CUDA events on the launch stream.
    A short busy-wait kernel is queued ahead of the first event so that the host has the call enqueued before
    the device reaches it: the interval is then the device time of the call, not the host's time to issue it."""
    for _ in range(warm):
        fn()
    hold = getattr(torch.cuda, "_sleep", None)
    ts = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if hold is not None:
            hold(400_000)                     # ~0.2 ms of device time on the same stream
        a.record()
        fn()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    return float(np.median(ts)), float(np.min(ts))


FULL_SIZES = {"t": 16384, "c1": (16384, 4096), "c2": (R, C), "c3_n": 1 << 28, "c3_m": (65536, 4096), "c4_n": 1 << 27, "c4_m": (32768, 4096), "c5": (1 << 24, 64, 256)}
# what the single-threaded CPU leg runs: the same kernels on arrays of a few MiB (the oracle streams at a few GB/s at best)
CPU_SAMPLE_SIZES = {"t": 1024, "c1": (1024, 512), "c2": (256, C), "c3_n": 1 << 22, "c3_m": (1024, 4096), "c4_n": 1 << 22, "c4_m": (1024, 4096), "c5": (4096, 64, 256)}


def kernel_rows(X, arr, S, copies=1):
    """Yield (config, kernel, algorithmic bytes, callable) for every per-kernel line of BASELINE's configs.
    X is the array module (device library or CPU oracle facade), arr(kind, shape) makes a seeded input in it,
    S the sizes.  `copies` > 1 rotates the small C1 operands among that many distinct buffers."""
    def rot(items):
        state = {"i": 0}

        def nxt():
            state["i"] = (state["i"] + 1) % len(items)
            return items[state["i"]]
        return nxt

    # C1 scaled (1 GiB at full size) and at its own 4096^2 (64 MiB: below the 256 MB bar, reported only)
    for n, tag in ((S["c1"][0], "C1x16"), (S["c1"][1], "C1")):
        k = copies if tag == "C1" else 1
        a = rot([arr("f32_pm1", (n, n)) for _ in range(k)])
        b = rot([arr("f32_pm1", (n, n)) for _ in range(k)])
        col = rot([arr("f32_pm1", (n, 1)) for _ in range(k)])
        s = n * n * 4
        yield tag, "a*b", 3 * s, lambda a=a, b=b: a() * b()
        yield tag, "a.sum(axis:1)", s + n * 4, lambda a=a: a().sum(axis=1)
        yield tag, "a + col(n,1)", 2 * s + n * 4, lambda a=a, col=col: a() + col()
        yield tag, "c.sum(axis:0)", s + n * 4, lambda a=a: a().sum(axis=0)
        yield tag, "c.max_index(axis:1)", s + n * 4, lambda a=a: a().max_index(axis=1)
        del a, b, col
    # C2
    r2, c2 = S["c2"]
    x, y = arr("f32_normal", (r2, 1)), arr("f32_normal", (1, c2))
    t = x + y
    yield "C2", "x(R,1)+y(1,C)", r2 * c2 * 4 + (r2 + c2) * 4, lambda: x + y
    yield "C2", "exp", 2 * r2 * c2 * 4, lambda: X.NMath.exp(t)
    yield "C2", "*0.5", 2 * r2 * c2 * 4, lambda: t * 0.5
    del t
    # C3
    n3, (mr, mc) = S["c3_n"], S["c3_m"]
    for kind, es, tag in (("f32_01", 4, "f32"), ("f64_01", 8, "f64")):
        v = arr(kind, (n3,))
        for op in ("sum", "mean", "max", "min", "argmax"):
            yield "C3", f"{tag} 1-D {op}", n3 * es + (4 if op == "argmax" else es), lambda op=op, v=v: getattr(v, op)()
        m = arr(kind, (mr, mc))
        for ax, n_out in ((0, mc), (1, mr)):
            for op in ("sum", "mean", "max", "min", "argmax"):
                yield "C3", f"{tag} 2-D {op}(axis:{ax})", mr * mc * es + n_out * (4 if op == "argmax" else es), lambda op=op, ax=ax, m=m: getattr(m, op)(axis=ax)
        del v, m
    # C4
    n4, (ir, ic) = S["c4_n"], S["c4_m"]
    ia, ib = arr("i32", (n4,)), arr("i32", (n4,))
    s = n4 * 4
    yield "C4", "a*3", 2 * s, lambda: ia * 3
    yield "C4", "+b", 3 * s, lambda: ia + ib
    yield "C4", "%7 (incl. the flag sync)", 2 * s, lambda: ia % 7
    yield "C4", "a>0 -> Bit", s + s // 32, lambda: ia > 0
    mask = ia > 0
    yield "C4", "count_true", s // 32 + 8, lambda: mask.count_true()
    im = arr("i32", (ir, ic))
    yield "C4", "max_index(axis:1)", ir * ic * 4 + ir * 4, lambda: im.max_index(axis=1)
    yield "C4", "Int32 sum -> Int64", s + 8, lambda: ia.sum()
    # T: operands whose contiguous axes differ (a transposed operand), 1 GiB per array at full size
    nt = S["t"]
    ta, tb, ti = arr("f32_pm1", (nt, nt)), arr("f32_pm1", (nt, nt)), arr("i32", (nt, nt))
    st = nt * nt * 4
    yield "T", "a + b.transpose", 3 * st, lambda: ta + tb.transpose()
    yield "T", "b.transpose.dup", 2 * st, lambda: tb.transpose().dup()
    yield "T", "SFloat.cast(i32.transpose)", 2 * st, lambda: X.SFloat.cast(ti.transpose())
    del ta, tb, ti
    # ... and with 8-byte elements and on a small plane, the shapes that take the copy-engine (TMA) form of the tile kernel
    nd = nt * 3 // 4 // 64 * 64
    td = arr("f64_01", (nd, nd))
    yield "T", "f64 a + a.transpose (TMA tile kernel)", 3 * nd * nd * 8, lambda: td + td.transpose()
    yield "T", "f64 a.transpose.dup (TMA tile kernel)", 2 * nd * nd * 8, lambda: td.transpose().dup()
    del td
    ns = max(64, nt // 4)
    tsm = arr("f32_pm1", (ns, ns))
    yield "T", "f32 b.transpose.dup, plane/16 (TMA tile kernel)", 2 * ns * ns * 4, lambda: tsm.transpose().dup()
    del tsm
    # F: the rows after the hot path (scan, histogram, compaction), same sizes
    v32 = arr("f32_01", (n3,))
    yield "F", "f32 1-D cumsum", 2 * n3 * 4, lambda: v32.cumsum()
    del v32
    # ... and the elementwise operations with a third operand, a second result or a position-dependent value
    c32 = arr("f32_01", (n3,))
    yield "F", "f32 clip(0.25, 0.75)", 2 * n3 * 4, lambda: c32.clip(0.25, 0.75)
    lo32 = c32 * 0.5
    hi32 = lo32 + 0.25
    yield "F", "f32 clip(lo array, hi array)", 4 * n3 * 4, lambda: c32.clip(lo32, hi32)
    yield "F", "f32 divmod(array)", 4 * n3 * 4, lambda: c32.divmod(hi32)
    del lo32, hi32
    yield "F", "f32 modf", 3 * n3 * 4, lambda: c32.modf()
    yield "F", "f32 fill", n3 * 4, lambda: c32.fill(0.5)
    yield "F", "f32 seq", n3 * 4, lambda: c32.seq(0.0, 1.0)
    del c32
    lab = arr("labels256", (n4,))
    yield "F", "Int32 bincount (256 bins)", n4 * 4 + 256 * 4, lambda: lab.bincount()
    yield "F", "Bit where (half set)", n4 // 8 + (n4 // 2) * 4, lambda: mask.where()


def kernel_table(torch, xp, peak):
    """Per-kernel effective GB/s at the BASELINE sizes (1 GPU, inputs resident, arrays >= 256 MB except C1), each beside
    the single-threaded CPU oracle running the same kernel on a sample of a few MiB."""
    g = torch.Generator(device="cuda").manual_seed(0)

    def dev_arr(kind, shape):
        if kind == "f32_pm1":
            return xp.SFloat.from_torch(torch.rand(*shape, device="cuda", generator=g) * 2 - 1)
        if kind == "f32_normal":
            return xp.SFloat.from_torch(torch.randn(*shape, device="cuda", generator=g))
        if kind == "f32_01":
            return xp.SFloat.from_torch(torch.rand(*shape, device="cuda", generator=g))
        if kind == "f64_01":
            return xp.DFloat.from_torch(torch.rand(*shape, device="cuda", dtype=torch.float64, generator=g))
        if kind == "labels256":
            return xp.Int32.from_torch(torch.randint(0, 256, shape, device="cuda", dtype=torch.int32, generator=g))
        return xp.Int32.from_torch(torch.randint(-(1 << 20), 1 << 20, shape, device="cuda", dtype=torch.int32, generator=g))

    sys.path.insert(0, str(ROOT / "tests"))
    from oracle_narray import OracleXP as ox
    from oracle import cumo_oracle as orc
    orc.set_threads(1)
    rng = np.random.default_rng(0)

    def cpu_arr(kind, shape):
        if kind == "f32_pm1":
            return ox.SFloat.cast(rng.uniform(-1, 1, shape).astype(np.float32))
        if kind == "f32_normal":
            return ox.SFloat.cast(rng.standard_normal(shape).astype(np.float32))
        if kind == "f32_01":
            return ox.SFloat.cast(rng.random(shape, dtype=np.float32))
        if kind == "f64_01":
            return ox.DFloat.cast(rng.random(shape))
        if kind == "labels256":
            return ox.Int32.cast(rng.integers(0, 256, shape, dtype=np.int32))
        return ox.Int32.cast(rng.integers(-(1 << 20), 1 << 20, shape, dtype=np.int32))

    cpu = {}
    for config, name, nbytes, fn in kernel_rows(ox, cpu_arr, CPU_SAMPLE_SIZES):
        fn()
        best = float("inf")
        for _ in range(2):
            t0 = time.perf_counter()
            fn()
            best = min(best, time.perf_counter() - t0)
        cpu[(config, name)] = round(nbytes / best / 1e9, 3)

    rows = []
    for config, name, nbytes, fn in kernel_rows(xp, dev_arr, FULL_SIZES, copies=8):
        med, best = time_kernel(torch, fn, reps=20)
        gbs = nbytes / (med * 1e-3) / 1e9
        rows.append({"config": config, "kernel": name, "bytes": int(nbytes), "ms": round(med, 4), "ms_min": round(best, 4),
                     "GBps": round(gbs, 1), "frac_of_measured": round(gbs / peak, 3), "frac_of_nominal": round(gbs / NOMINAL_HBM_GBS, 3),
                     "cpu_GBps_1thread_sample": cpu.get((config, name))})
    try:
        ref = ref_gpu_table(torch, FULL_SIZES)
    except Exception as e:                           # the baseline leg must never take the product's numbers down with it
        ref = {}
        print(f"reference-kernel leg skipped: {e}", file=sys.stderr)
    for row in rows:
        ms = ref.get((row["config"], row["kernel"]))
        if ms:
            row["ref_gpu_ms"] = ms
            row["ref_gpu_GBps"] = round(row["bytes"] / (ms * 1e-3) / 1e9, 1)
            row["speedup_vs_ref_gpu"] = round(ms / row["ms"], 2)

    # `%7` without the host's read-back of the division-by-zero flag: the launch function called directly, events around it
    try:
        sys.path.insert(0, str(ROOT / "tests"))
        import abi_call as ac
        from ctypes import byref, c_int, c_int32, c_void_p
        from cumo_b200 import _lib as _l
        n4 = FULL_SIZES["c4_n"]
        ia = torch.randint(-(1 << 20), 1 << 20, (n4,), device="cuda", dtype=torch.int32, generator=g)
        io = torch.empty_like(ia)
        flag = torch.zeros(1, device="cuda", dtype=torch.int32)
        ix = ac.indexer((n4,))
        fn = ac.fn(_l.load(), "cumo_iter_int32_mod_s_kernel_launch")
        med, best = time_kernel(torch, lambda: fn(byref(ac.iarray(ia)), c_int32(7), byref(ac.iarray(io)), byref(ix), c_void_p(flag.data_ptr()), c_int(0)), reps=20)
        nb = 2 * n4 * 4
        gbs = nb / (med * 1e-3) / 1e9
        rows.append({"config": "C4", "kernel": "%7 kernel alone (launch function, no flag read-back)", "bytes": nb, "ms": round(med, 4), "ms_min": round(best, 4),
                     "GBps": round(gbs, 1), "frac_of_measured": round(gbs / peak, 3), "frac_of_nominal": round(gbs / NOMINAL_HBM_GBS, 3)})
        del ia, io
    except Exception as e:
        print(f"%7 kernel-alone row skipped: {e}", file=sys.stderr)

    # managed memory, which is what every buffer of the reference is (its pool hands out cudaMallocManaged blocks):
    # exp and sum on buffers prefetched to the device, beside the cudaMalloc rows above
    try:
        rows += managed_rows(torch, xp, peak)
    except Exception as e:
        print(f"managed-memory rows skipped: {e}", file=sys.stderr)

    # C5 (BASELINE config 4): k-means assignment, 2^24 points x 64-D against 256 centres, fused
    from cumo_b200 import kmeans
    n, d, k = FULL_SIZES["c5"]
    cen = torch.randn(k, d, device="cuda", generator=g) * 4
    pts = cen[torch.randint(0, k, (n,), device="cuda", generator=g)] + torch.randn(n, d, device="cuda", generator=g)
    px, pc = xp.SFloat.from_torch(pts), xp.SFloat.from_torch(cen)
    ns = CPU_SAMPLE_SIZES["c5"][0]
    hx, hc = pts[:ns].cpu().numpy(), cen.cpu().numpy()
    t0 = time.perf_counter()
    orc.kmeans_assign(hx, hc)
    cpu_sec = time.perf_counter() - t0
    for algo, what in (("tensor", "fused, tcgen05 3xTF32"), ("cores", "fused, fp32 cores")):
        nbytes = n * d * 4 + k * d * 4 + n * 4 + k * 8
        med, best = time_kernel(torch, lambda algo=algo: kmeans.assign(px, pc, algo=algo), reps=20)
        gbs = nbytes / (med * 1e-3) / 1e9
        row = {"config": "C5", "kernel": f"kmeans assign 2^24x64 vs 256 ({what})", "bytes": int(nbytes), "ms": round(med, 4), "ms_min": round(best, 4),
               "GBps": round(gbs, 1), "frac_of_measured": round(gbs / peak, 3), "frac_of_nominal": round(gbs / NOMINAL_HBM_GBS, 3),
               "cpu_GBps_1thread_sample": round((ns * d * 4 + k * d * 4 + ns * 4 + k * 8) / cpu_sec / 1e9, 4),
               # useful flops of the (N, K, D) contraction; the tensor form issues three TF32 MMAs per product
               "TFLOPs": round(2.0 * n * k * d / (med * 1e-3) / 1e12, 2)}
        if algo == "tensor":
            row["TFLOPs_issued_tf32"] = round(3 * row["TFLOPs"], 1)
        rows.append(row)
    # single-precision matrix product on the tensor cores (`dot`): TFLOP/s, beside torch's fp32 (non-TF32) cuBLAS product
    from cumo_b200 import linalg
    del px, pc, pts
    gm = 8192
    ga = torch.randn(gm, gm, device="cuda", generator=g)
    gb = torch.randn(gm, gm, device="cuda", generator=g)
    xa, xb = xp.SFloat.from_torch(ga), xp.SFloat.from_torch(gb)
    med, best = time_kernel(torch, lambda: linalg.gemm_nt(xa, xb), reps=10)
    torch.backends.cuda.matmul.allow_tf32 = False
    med_lib, _ = time_kernel(torch, lambda: ga @ gb.T, reps=5)
    nbytes = 3 * gm * gm * 4
    rows.append({"config": "F", "kernel": "SFloat dot 8192^3 (tcgen05 3xTF32, K-chunked)", "bytes": nbytes, "ms": round(med, 4), "ms_min": round(best, 4),
                 "GBps": round(nbytes / (med * 1e-3) / 1e9, 1), "frac_of_measured": None, "frac_of_nominal": None,
                 "TFLOPs": round(2.0 * gm ** 3 / (med * 1e-3) / 1e12, 1),
                 "TFLOPs_issued_tf32": round(6.0 * gm ** 3 / (med * 1e-3) / 1e12, 1),
                 "cublas_fp32_ms": round(med_lib, 4), "cublas_fp32_TFLOPs": round(2.0 * gm ** 3 / (med_lib * 1e-3) / 1e12, 1)})
    # double-precision `dot` (CUDA-core tile kernel; the reference calls cublasDgemm) beside torch's fp64 cuBLAS product
    del xa, xb, ga, gb
    dm = 4096
    da = torch.randn(dm, dm, device="cuda", dtype=torch.float64, generator=g)
    db = torch.randn(dm, dm, device="cuda", dtype=torch.float64, generator=g)
    ya, yb = xp.DFloat.from_torch(da), xp.DFloat.from_torch(db)
    med, best = time_kernel(torch, lambda: linalg.dot(ya, yb), reps=5)
    med_lib, _ = time_kernel(torch, lambda: da @ db, reps=5)
    rows.append({"config": "F", "kernel": "DFloat dot 4096^3 (CUDA cores, FP64 FMA)", "bytes": 3 * dm * dm * 8, "ms": round(med, 4), "ms_min": round(best, 4),
                 "GBps": round(3 * dm * dm * 8 / (med * 1e-3) / 1e9, 1), "frac_of_measured": None, "frac_of_nominal": None,
                 "TFLOPs": round(2.0 * dm ** 3 / (med * 1e-3) / 1e12, 1), "cublas_fp64_ms": round(med_lib, 4),
                 "cublas_fp64_TFLOPs": round(2.0 * dm ** 3 / (med_lib * 1e-3) / 1e12, 1)})
    return rows


def managed_rows(torch, xp, peak):
    from cuda.bindings import runtime as rt

    n = 1 << 28
    nbytes = n * 4
    ptrs = []
    for _ in range(2):
        err, p = rt.cudaMallocManaged(nbytes, rt.cudaMemAttachGlobal)
        if err != rt.cudaError_t.cudaSuccess:
            raise RuntimeError(f"cudaMallocManaged: {err}")
        ptrs.append(int(p))
    try:
        loc = rt.cudaMemLocation()
        loc.type = rt.cudaMemLocationType.cudaMemLocationTypeDevice
        loc.id = torch.cuda.current_device()
        for p in ptrs:
            try:
                (err,) = rt.cudaMemPrefetchAsync(p, nbytes, loc, 0, 0)
            except TypeError:
                (err,) = rt.cudaMemPrefetchAsync(p, nbytes, loc.id, 0)
            if err != rt.cudaError_t.cudaSuccess:
                raise RuntimeError(f"cudaMemPrefetchAsync: {err}")
        torch.cuda.synchronize()
        a = xp.SFloat.from_device_pointer(ptrs[0], (n,))
        o = xp.SFloat.from_device_pointer(ptrs[1], (n,))
        a.fill(0.5)
        o.fill(0.0)
        xp.synchronize()
        out = []
        for name, fn, nb in (("exp, 2^28 f32 read from managed memory (prefetched)", lambda: xp.NMath.exp(a), 2 * nbytes),
                             ("sum, 2^28 f32 in managed memory (prefetched)", lambda: o.sum(), nbytes + 4)):
            med, best = time_kernel(torch, fn, reps=10)
            gbs = nb / (med * 1e-3) / 1e9
            out.append({"config": "M", "kernel": name, "bytes": int(nb), "ms": round(med, 4), "ms_min": round(best, 4), "GBps": round(gbs, 1),
                        "frac_of_measured": round(gbs / peak, 3), "frac_of_nominal": round(gbs / NOMINAL_HBM_GBS, 3)})
        del a, o
        xp.synchronize()
        return out
    finally:
        torch.cuda.synchronize()
        for p in ptrs:
            rt.cudaFree(p)


def ref_gpu_table(torch, S):
    """The reference's OWN kernels (oracle/_ref/libcumo_ref_kernels.so: its templates expanded and compiled with the
    same nvcc by oracle/build_ref_kernels.py) timed on this GPU with the descriptors its host code would build for the
    same rows: {(config, kernel): ms}.  Empty when that library was never built."""
    from oracle import ref_kernels

    L = ref_kernels.lib()
    if L is None:
        return {}
    sys.path.insert(0, str(ROOT / "tests"))
    import abi_call as ac
    from ctypes import byref, c_float, c_int, c_int32, c_size_t, c_ssize_t, c_uint64, c_void_p

    g = torch.Generator(device="cuda").manual_seed(0)
    out = {}

    def t(config, name, fn, reps=5):
        med, _ = time_kernel(torch, fn, reps=reps, warm=1)
        if L.refk_last_error():
            raise RuntimeError(f"reference kernel failed to launch: {config} {name}")
        out[(config, name)] = round(med, 4)

    def ew(sym, x, y, o, shape):
        ac.fn(L, sym)(byref(ac.iarray(x, shape)), byref(ac.iarray(y, shape)), byref(ac.iarray(o)), byref(ac.indexer(shape)), None)

    def red(sym, src, dst, axes):
        ac.fn(L, sym)(byref(ac.reduction_arg(src, dst, axes)))

    for n, tag in ((S["c1"][0], "C1x16"), (S["c1"][1], "C1")):
        a = torch.rand(n, n, device="cuda", generator=g) * 2 - 1
        b = torch.rand(n, n, device="cuda", generator=g) * 2 - 1
        col = torch.rand(n, 1, device="cuda", generator=g)
        o = torch.empty_like(a)
        vec = torch.empty(n, device="cuda")
        idx = torch.empty(n, device="cuda", dtype=torch.int32)
        t(tag, "a*b", lambda: ew("cumo_iter_sfloat_mul_kernel_launch", a.view(-1), b.view(-1), o.view(-1), (n * n,)))
        t(tag, "a.sum(axis:1)", lambda: red("cumo_sfloat_sum_kernel_launch", a, vec, (1,)))
        t(tag, "a + col(n,1)", lambda: ew("cumo_iter_sfloat_add_kernel_launch", a, col, o, (n, n)))
        t(tag, "c.sum(axis:0)", lambda: red("cumo_sfloat_sum_kernel_launch", a, vec, (0,)))
        t(tag, "c.max_index(axis:1)", lambda: red("cumo_sfloat_max_index_int32_kernel_launch", a, idx, (1,)))
        del a, b, col, o
    r2, c2 = S["c2"]
    x, y = torch.randn(r2, 1, device="cuda", generator=g), torch.randn(1, c2, device="cuda", generator=g)
    tt = x + y
    o2 = torch.empty_like(tt)
    t("C2", "x(R,1)+y(1,C)", lambda: ew("cumo_iter_sfloat_add_kernel_launch", x, y, o2, (r2, c2)))
    t("C2", "exp", lambda: ac.fn(L, "cumo_iter_sfloat_math_s_exp_kernel_launch")(byref(ac.iarray(tt.view(-1))), byref(ac.iarray(o2.view(-1))), byref(ac.indexer((r2 * c2,)))))
    t("C2", "*0.5", lambda: ac.fn(L, "cumo_iter_sfloat_mul_s_kernel_launch")(byref(ac.iarray(tt.view(-1))), c_float(0.5), byref(ac.iarray(o2.view(-1))), byref(ac.indexer((r2 * c2,))), None, c_int(0)))
    del tt, o2
    n3, (mr, mc) = S["c3_n"], S["c3_m"]
    for dt, tname, tag in ((torch.float32, "sfloat", "f32"), (torch.float64, "dfloat", "f64")):
        v = torch.rand(n3, device="cuda", generator=g, dtype=dt)
        m = v.view(mr, mc)
        for op in ("sum", "mean", "max", "min", "argmax"):
            sym = f"cumo_{tname}_{op}_int32_kernel_launch" if op == "argmax" else f"cumo_{tname}_{op}_kernel_launch"
            odt = torch.int32 if op == "argmax" else dt
            one = torch.empty((), device="cuda", dtype=odt)
            t("C3", f"{tag} 1-D {op}", lambda: red(sym, v, one, (0,)), reps=3)
            for ax, n_out in ((0, mc), (1, mr)):
                dst = torch.empty(n_out, device="cuda", dtype=odt)
                t("C3", f"{tag} 2-D {op}(axis:{ax})", lambda: red(sym, m, dst, (ax,)), reps=3)
        del v, m
    n4, (ir, ic) = S["c4_n"], S["c4_m"]
    ia = torch.randint(-(1 << 20), 1 << 20, (n4,), device="cuda", dtype=torch.int32, generator=g)
    ib = torch.randint(-(1 << 20), 1 << 20, (n4,), device="cuda", dtype=torch.int32, generator=g)
    io = torch.empty_like(ia)
    flag = torch.zeros(1, device="cuda", dtype=torch.int32)
    ix = ac.indexer((n4,))
    t("C4", "a*3", lambda: ac.fn(L, "cumo_iter_int32_mul_s_kernel_launch")(byref(ac.iarray(ia)), c_int32(3), byref(ac.iarray(io)), byref(ix), None, c_int(0)))
    t("C4", "+b", lambda: ew("cumo_iter_int32_add_kernel_launch", ia, ib, io, (n4,)))

    def mod7():                                       # the reference's host reads the division-by-zero flag back after the launch
        ac.fn(L, "cumo_iter_int32_mod_s_kernel_launch")(byref(ac.iarray(ia)), c_int32(7), byref(ac.iarray(io)), byref(ix), c_void_p(flag.data_ptr()), c_int(0))
        torch.cuda.synchronize()
    t("C4", "%7 (incl. the flag sync)", mod7)
    words = torch.zeros(n4 // 32, device="cuda", dtype=torch.int32)
    t("C4", "a>0 -> Bit", lambda: ac.fn(L, "cumo_iter_int32_gt_s_kernel_launch")(byref(ac.iarray(ia)), c_int32(0), byref(ac.bit_iarray(words)), byref(ix), c_int(0)), reps=3)
    cnt = torch.zeros(1, device="cuda", dtype=torch.int64)
    t("C4", "count_true", lambda: ac.fn(L, "cumo_iter_bit_count_true_stride_kernel_launch")(c_size_t(0), c_void_p(cnt.data_ptr()), c_void_p(words.data_ptr()), c_ssize_t(1), c_uint64(n4)), reps=3)
    im = ia.view(ir, ic)
    idx = torch.empty(ir, device="cuda", dtype=torch.int32)
    t("C4", "max_index(axis:1)", lambda: red("cumo_int32_max_index_int32_kernel_launch", im, idx, (1,)))
    s64 = torch.empty((), device="cuda", dtype=torch.int64)
    t("C4", "Int32 sum -> Int64", lambda: red("cumo_int32_sum_kernel_launch", ia, s64, (0,)))
    nt = S["t"]
    ta = torch.rand(nt, nt, device="cuda", generator=g)
    tb = torch.rand(nt, nt, device="cuda", generator=g)
    to = torch.empty_like(ta)
    t("T", "a + b.transpose", lambda: ew("cumo_iter_sfloat_add_kernel_launch", ta, tb.t(), to, (nt, nt)), reps=3)
    t("T", "b.transpose.dup", lambda: ac.fn(L, "cumo_iter_sfloat_store_sfloat_kernel_launch")(byref(ac.iarray(to)), byref(ac.iarray(tb.t())), byref(ac.indexer((nt, nt)))), reps=3)
    ti = ia.new_empty((nt, nt)).copy_(tb * 1000)
    t("T", "SFloat.cast(i32.transpose)", lambda: ac.fn(L, "cumo_iter_sfloat_store_int32_kernel_launch")(byref(ac.iarray(to)), byref(ac.iarray(ti.t())), byref(ac.indexer((nt, nt)))), reps=3)
    del ta, tb, to, ti
    # the rows after the hot path: thrust scan, global-atomic histogram, compaction
    v32 = torch.rand(n3, device="cuda", generator=g)
    o32 = torch.empty_like(v32)
    t("F", "f32 1-D cumsum", lambda: ac.fn(L, "cumo_sfloat_cumsum_kernel_launch", c_int)(c_void_p(v32.data_ptr()), c_void_p(o32.data_ptr()), c_ssize_t(4), c_ssize_t(4), c_uint64(n3)), reps=3)
    del v32, o32
    lab = torch.randint(0, 256, (n4,), device="cuda", dtype=torch.int32, generator=g)
    counts = torch.empty(256, device="cuda", dtype=torch.int32)
    oor, item = torch.zeros(1, device="cuda", dtype=torch.int32), torch.zeros(1, device="cuda", dtype=torch.int64)
    t("F", "Int32 bincount (256 bins)", lambda: ac.fn(L, "cumo_iter_int32_bincount_32_kernel_launch")(c_void_p(lab.data_ptr()), c_ssize_t(4), None, c_uint64(n4), c_void_p(counts.data_ptr()), c_ssize_t(4),
                                                                                                     c_uint64(256), c_void_p(oor.data_ptr()), c_void_p(item.data_ptr())), reps=3)
    ac.fn(L, "cumo_iter_int32_gt_s_kernel_launch")(byref(ac.iarray(ia)), c_int32(0), byref(ac.bit_iarray(words)), byref(ix), c_int(0))
    pos = torch.empty(n4, device="cuda", dtype=torch.int32)
    new, free = ac.fn(L, "cumo_bit_where_scratch_new", c_void_p), ac.fn(L, "cumo_cuda_runtime_free")

    def where():
        scratch = new()
        ac.fn(L, "cumo_bit_where_kernel_launch")(c_void_p(words.data_ptr()), c_size_t(0), c_ssize_t(1), None, c_uint64(n4), c_int(0), c_void_p(pos.data_ptr()), c_size_t(4), c_uint64(0), c_void_p(scratch))
        free(c_void_p(scratch))
    t("F", "Bit where (half set)", where, reps=3)
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: libcumo_b200 has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    import cumo_b200 as xp
    from cumo_b200 import _lib

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    rng = np.random.default_rng(1 + rank)
    hx = torch.from_numpy(rng.standard_normal((R, 1)).astype(np.float32)).pin_memory()
    hy = torch.from_numpy(rng.standard_normal((1, C)).astype(np.float32)).pin_memory()
    hout = torch.empty((R, C), dtype=torch.float32).pin_memory()

    def upload():
        return (xp.SFloat.from_host_pointer(hx.data_ptr(), (R, 1), R * ES), xp.SFloat.from_host_pointer(hy.data_ptr(), (1, C), C * ES))

    def chain(x, y):
        return xp.NMath.exp(x + y) * 0.5

    gx, gy = upload()
    xp.synchronize()
    for _ in range(args.warmup):
        chain(gx, gy)
    barrier()
    c0 = _lib.launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    block_ms = []
    with ClockSampler(local) as clocks:
        start.record()
        for _ in range(args.steps):
            chain(gx, gy)
        stop.record()
        barrier()
        launches = _lib.launch_count() - c0
        # the same K-step block again and again under the same clock sampling, so that the evidence spans some hundreds
        # of milliseconds instead of one block of a few: the line's `value` stays the first, contract-shaped block
        for _ in range(50):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(args.steps):
                chain(gx, gy)
            b.record()
            b.synchronize()
            block_ms.append(a.elapsed_time(b))
    ms = torch.tensor([start.elapsed_time(stop)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    value = BYTES_STEP * world * args.steps / (ms * 1e-3) / 1e9

    # end to end: host buffers in, host buffer out, copies inside the timed region.  The rows go in blocks: block k's
    # result travels to the host on a copy stream while block k+1's kernels run, so a step costs about what its
    # 512 MiB device->host copy costs (PCIe-bound by construction).
    n_blocks = 8
    rb = R // n_blocks
    copy_stream = torch.cuda.Stream()
    hx_blocks = [hx[b * rb:(b + 1) * rb] for b in range(n_blocks)]

    def e2e_step():
        y = xp.SFloat.from_host_pointer(hy.data_ptr(), (1, C), C * ES)
        keep = []
        for b in range(n_blocks):
            x = xp.SFloat.from_host_pointer(hx_blocks[b].data_ptr(), (rb, 1), rb * ES)
            r = chain(x, y)
            r.read_into_host_async(hout[b * rb:(b + 1) * rb].data_ptr(), rb * C * ES, copy_stream.cuda_stream)
            keep.append(r)
        copy_stream.synchronize()                    # the step's result is in host memory
        return keep

    for _ in range(min(2, args.warmup)):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_value = BYTES_STEP * world * args.steps / (float(e2e_ms.item()) * 1e-3) / 1e9
    # the device->host copy of one step's result alone, all ranks copying at the same time: the floor of e2e
    dres = torch.empty((R, C), dtype=torch.float32, device="cuda")
    barrier()
    c0e, c1e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0e.record()
    for _ in range(5):
        hout.copy_(dres, non_blocking=True)
    c1e.record()
    barrier()
    d2h_ms = torch.tensor([c0e.elapsed_time(c1e) / 5], device="cuda")
    if world > 1:
        dist.all_reduce(d2h_ms, op=dist.ReduceOp.MAX)
    d2h_ms = float(d2h_ms.item())
    del dres

    peak, peak_kind = measured_peak()
    line = None
    if rank == 0:
        # roofline of the dominant kernel (exp: 1 GiB algorithmic bytes per launch), timed launch by launch
        t = gx + gy
        med, _ = time_kernel(torch, lambda: xp.NMath.exp(t), reps=max(5, args.steps))
        achieved = BYTES_EXP / (med * 1e-3) / 1e9
        del t
        line = {"metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic",
                "config": {"workload": "BASELINE config 1: x(8192,1)+y(1,16384), exp, *0.5 (fp32), per GPU", "rows_per_gpu": R, "cols": C,
                           "algorithmic_bytes_per_step_per_gpu": BYTES_STEP, "l2": "every kernel streams >= 512 MiB, 4x the 126 MB L2; no flush",
                           "partition": "independent row blocks per GPU, no data-path collective"},
                "gpu_launches": int(launches) * world,
                "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": (R + C) * ES, "d2h_bytes_per_step": R * C * ES,
                        "ms_per_step": float(e2e_ms.item()) / args.steps, "row_blocks": n_blocks,
                        "d2h_copy_alone_ms": d2h_ms, "d2h_GBps_per_gpu": R * C * ES / (d2h_ms * 1e-3) / 1e9,
                        "note": "a step cannot be shorter than its 512 MiB device->host copy; copy_alone is that copy timed by itself with all ranks copying at once"},
                "roofline": {"bound": "hbm", "kernel": "ew_row_kernel<Exp<float>,4>", "achieved": achieved, "peak": peak, "peak_kind": peak_kind,
                             "unit": "GB/s", "frac": achieved / peak, "frac_of_nominal_8TBps": achieved / NOMINAL_HBM_GBS,
                             "traffic": EXP_KERNEL_DRAM_TRAFFIC_BYTES, "traffic_origin": "ncu dram__bytes_read.sum + dram__bytes_write.sum, one launch of `bench.py --case exp --mib 512`",
                             "algorithmic_bytes_per_launch": BYTES_EXP, "ms_per_launch": med},
                "chain_frac_of_peak": value / world / peak,
                "repeat_blocks": {"blocks": len(block_ms), "steps_per_block": args.steps, "ms_per_step_median": float(np.median(block_ms)) / args.steps,
                                  "ms_per_step_min": float(np.min(block_ms)) / args.steps, "ms_per_step_max": float(np.max(block_ms)) / args.steps,
                                  "GBps_median_this_rank": BYTES_STEP * args.steps / (float(np.median(block_ms)) * 1e-3) / 1e9},
                "clocks": clocks.summary()}
    if world > 1:
        sharded = sharded_section(torch, dist, xp, rank, world)
        if rank == 0:
            line["sharded"] = sharded
    if rank == 0 and world == 1:
        rows = 2048
        from oracle import cumo_oracle as orc
        orc.set_threads(1)
        sec = oracle_chain(hx.numpy(), hy.numpy(), rows)
        line["cpu_baseline"] = {"value": sample_bytes(rows) / sec / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                                "sample": f"first {rows} of {R} rows of the same workload, one pass, single thread like Numo ({os.cpu_count()} host cores present)"}
        if not args.no_kernels:
            line["kernels"] = kernel_table(torch, xp, peak)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def sharded_section(torch, dist, xp, rank, world):
    """Row-sharded reductions that need a collective: 2^28 fp32 elements per GPU, and a (65536,4096) block per GPU.
    Every result is checked on every rank (a planted maximum straddles each shard boundary; sums against float64
    sums that torch all-reduces), and every op is timed beside the same op on the local shard alone:
    efficiency = t_local / t_sharded."""
    from cumo_b200.sharded import Comm, ShardedArray
    from cumo_b200 import kmeans

    comm = Comm(xp)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    n = 1 << 28
    tv = torch.rand(n, device="cuda", generator=g)
    # the maximum twice across every shard boundary: last element of rank r-1 and first of rank r.  First occurrence
    # over the whole array is the last element of rank 0; per column of the matrix view it is row 65535 of rank 0.
    if rank > 0:
        tv[:4096] = 2.0
    if rank < world - 1:
        tv[-4096:] = 2.0
    v = xp.SFloat.from_torch(tv)
    sv = ShardedArray(comm, v, n * world, n * rank)
    m = v.reshape(65536, 4096)
    sm = ShardedArray(comm, m, 65536 * world, 65536 * rank)
    kn, kd, kk = 1 << 24, 64, 256                    # BASELINE config 4 per GPU: points sharded, centroids replicated, counts all-reduced
    gc = torch.Generator(device="cuda").manual_seed(4)
    cen = torch.randn(kk, kd, device="cuda", generator=gc) * 4
    pts = cen[torch.randint(0, kk, (kn,), device="cuda", generator=g)] + torch.randn(kn, kd, device="cuda", generator=g)
    px, pc = xp.SFloat.from_torch(pts), xp.SFloat.from_torch(cen)

    # ---- correctness, on every rank ----
    def allsum(t):
        t = t.clone()
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return t
    ref_sum = allsum(tv.sum(dtype=torch.float64).reshape(1)).item()
    got = float(sv.sum().extract())
    assert abs(got - ref_sum) <= 1e-5 * ref_sum, ("sharded sum", got, ref_sum)
    first_max = (n - 4096) if world > 1 else int(tv.argmax().item())
    assert int(sv.argmax().extract()) == first_max, ("sharded argmax", int(sv.argmax().extract()), first_max)
    ref_col = allsum(tv.view(65536, 4096).sum(dim=0, dtype=torch.float64))
    got_col = torch.as_tensor(sm.sum(axis=0), device="cuda").double()
    assert torch.all((got_col - ref_col).abs() <= 1e-5 * ref_col), "sharded sum(axis:0)"
    ref_max = tv.view(65536, 4096).max(dim=0).values.clone()
    dist.all_reduce(ref_max, op=dist.ReduceOp.MAX)
    assert torch.equal(torch.as_tensor(sm.max(axis=0), device="cuda"), ref_max), "sharded max(axis:0)"
    if world > 1:
        am = torch.as_tensor(sm.argmax(axis=0), device="cuda")
        assert bool((am == 65535).all()), "sharded argmax(axis:0): the first of the planted maxima is row 65535 (rank 0's last row)"
    _, counts = kmeans.assign_sharded(comm, px, pc)
    assert int(torch.as_tensor(counts, device="cuda").view(torch.int64).sum().item()) == kn * world, "k-means counts"

    # ---- timing: the sharded op, and the same op on the local shard alone ----
    def timed(fn, reps=20):
        for _ in range(3):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b) / reps], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    out = []
    for name, fn, local_fn, nbytes in (
            ("sum 1-D 2^28/GPU", lambda: sv.sum(), lambda: v.sum(), n * 4),
            ("argmax 1-D 2^28/GPU", lambda: sv.argmax(), lambda: v.argmax(), n * 4),
            ("sum(axis:0) (65536,4096)/GPU", lambda: sm.sum(axis=0), lambda: m.sum(axis=0), n * 4),
            ("max(axis:0) (65536,4096)/GPU", lambda: sm.max(axis=0), lambda: m.max(axis=0), n * 4),
            ("argmax(axis:0) (65536,4096)/GPU", lambda: sm.argmax(axis=0), lambda: m.argmax(axis=0), n * 4),
            ("kmeans assign 2^24x64 vs 256 /GPU (tcgen05) + counts all_reduce", lambda: kmeans.assign_sharded(comm, px, pc), lambda: kmeans.assign(px, pc), kn * kd * 4 + kn * 4)):
        ms, ms_local = timed(fn), timed(local_fn)
        out.append({"op": name, "ms": round(ms, 4), "ms_local_only": round(ms_local, 4), "efficiency": round(ms_local / ms, 3),
                    "aggregate_GBps": round(nbytes * world / (ms * 1e-3) / 1e9, 1), "checked": True,
                    "gather": "peer memory" if comm.peer is not None else "nccl all_gather"})
    comm.check()                                     # no bounded wait of a peer exchange ran out
    if comm.peer is not None:
        # the same reductions with NCCL's all_gather in place of the peer-memory exchange, for comparison
        comm_nccl = Comm(xp, peer_exchange=False)
        sv2, sm2 = ShardedArray(comm_nccl, v, n * world, n * rank), ShardedArray(comm_nccl, m, 65536 * world, 65536 * rank)
        for entry, fn in zip(out, (lambda: sv2.sum(), lambda: sv2.argmax(), lambda: sm2.sum(axis=0), lambda: sm2.max(axis=0), lambda: sm2.argmax(axis=0))):
            entry["ms_with_nccl_all_gather"] = round(timed(fn), 4)
    return out


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

    side = int((rows32 * cols) ** 0.5) // 64 * 64
    side64 = int((rows64 * cols) ** 0.5) // 64 * 64

    def sq():
        return f32()[0:side * side].reshape(side, side)

    def sq2():
        if "sq2" not in cache:
            cache["sq2"] = xp.SFloat.from_torch(torch.rand(side, side, device="cuda", generator=g))
        return cache["sq2"]

    def km():
        from cumo_b200 import kmeans
        n, d, k = n32 // 64, 64, 256
        cen = torch.randn(k, d, device="cuda", generator=g) * 4
        pts = cen[torch.randint(0, k, (n,), device="cuda", generator=g)] + torch.randn(n, d, device="cuda", generator=g)
        return kmeans, xp.SFloat.from_torch(pts), xp.SFloat.from_torch(cen)

    def gemm():
        from cumo_b200 import linalg
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
        "mulsum_axis1_f32": (lambda: (lambda a=f32().reshape(rows32, cols), b=(f32() * 0.5).reshape(rows32, cols): a.mulsum(b, axis=1)), 2 * n32 * 4),
        "mulsum_axis0_f32": (lambda: (lambda a=f32().reshape(rows32, cols), b=(f32() * 0.5).reshape(rows32, cols): a.mulsum(b, axis=0)), 2 * n32 * 4),
        "mulsum_axis1_short_f32": (lambda: (lambda a=f32().reshape(rows32 * cols // 16, 16), b=(f32() * 0.5).reshape(rows32 * cols // 16, 16): a.mulsum(b, axis=1)), 2 * n32 * 4 + n32 // 4),
        "sum_axis1_short_f32": (lambda: (lambda a=f32().reshape(rows32 * cols // 16, 16): a.sum(axis=1)), n32 * 4 + n32 // 4),
        "cumsum_axis1_short_f32": (lambda: (lambda a=f32().reshape(rows32 * cols // 64, 64): a.cumsum(axis=1)), 2 * n32 * 4),
        "cumsum_axis1_f32": (lambda: (lambda a=f32().reshape(rows32, cols): a.cumsum(axis=1)), 2 * n32 * 4),
        "cumsum_axis0_f32": (lambda: (lambda a=f32().reshape(rows32, cols): a.cumsum(axis=0)), 2 * n32 * 4),
        "count_true_axis1": (lambda: (lambda m=(i32().reshape(rows32, cols) > 0): m.count_true(axis=1)), n32 // 8 + rows32 * 8),
        "count_true_axis0": (lambda: (lambda m=(i32().reshape(rows32, cols) > 0): m.count_true(axis=0)), n32 // 8 + cols * 8),
        "bits_to_f32": (lambda: (lambda m=(i32() > 0): xp.SFloat.cast(m)), n32 // 8 + n32 * 4),
        "i32_to_bits": (lambda: (lambda a=i32(): xp.Bit.cast(a)), n32 * 4 + n32 // 8),
        "poly3_f32": (lambda: (lambda a=f32(): a.poly(1.0, 2.0, 3.0)), 2 * n32 * 4),
        "clip_scalars_f32": (lambda: (lambda a=f32(): a.clip(-0.5, 0.5)), 2 * n32 * 4),
        "clip_arrays_f32": (lambda: (lambda a=f32(), lo=f32() * 0.5 - 0.5, hi=f32() * 0.5 + 0.5: a.clip(lo, hi)), 4 * n32 * 4),
        "divmod_f32": (lambda: (lambda a=f32(), b=f32() * 0.5 + 1.0: a.divmod(b)), 4 * n32 * 4),
        "modf_f32": (lambda: (lambda a=f32(): a.modf()), 3 * n32 * 4),
        "fill_f32": (lambda: (lambda a=xp.SFloat.new(rows32 * cols): a.fill(0.5)), n32 * 4),
        "seq_f32": (lambda: (lambda a=xp.SFloat.new(rows32 * cols): a.seq(0.0, 1.0)), n32 * 4),
        # operands whose contiguous axes differ: the shared-memory tile kernel
        "add_transposed": (lambda: (lambda a=sq(), b=sq2(): a + b.transpose()), 3 * side * side * 4),
        "copy_transposed": (lambda: (lambda b=sq(): b.transpose().dup()), 2 * side * side * 4),
        "copy_transposed_f64": (lambda: (lambda b=f64()[0:side64 * side64].reshape(side64, side64): b.transpose().dup()), 2 * side64 * side64 * 8),
        "add_transposed_f64": (lambda: (lambda a=f64()[0:side64 * side64].reshape(side64, side64): a + a.transpose()), 3 * side64 * side64 * 8),
        "cast_transposed_i32": (lambda: (lambda b=i32()[0:side * side].reshape(side, side): xp.SFloat.cast(b.transpose())), 2 * side * side * 4),
    }
    return cases




def run_case(args):
    """`--case NAME`: one named kernel case on synthetic device data, a few launches, its timing printed.  This is the
    small, self-ending command that profiler captures are taken on (one kernel, a few launches, a few hundred MiB on
    the device) and a quick way to time a single kernel; `--mib` is the size of the main input array."""
    import torch

    import cumo_b200 as xp

    torch.cuda.set_device(0)
    cases = build_cases(xp, torch, args.mib)
    if args.case == "list":
        print(" ".join(cases))
        return
    setup, nbytes = cases[args.case]
    fn = setup()
    med, best = time_kernel(torch, fn, reps=args.reps, warm=args.warm)
    print(f"{args.case}: {args.mib} MiB input, {nbytes} algorithmic bytes, median {med:.4f} ms (min {best:.4f}) over {args.reps} launches, {nbytes / (med * 1e-3) / 1e9:.1f} GB/s")


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel table of the other BASELINE configs")
    ap.add_argument("--case", help="run ONE named kernel case instead of the benchmark (`--case list` names them); for profiler captures")
    ap.add_argument("--mib", type=int, default=512, help="--case: size of the main input array")
    ap.add_argument("--reps", type=int, default=3, help="--case: timed launches")
    ap.add_argument("--warm", type=int, default=1, help="--case: untimed launches first")
    args = ap.parse_args()
    if args.case:
        run_case(args)
        return
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
