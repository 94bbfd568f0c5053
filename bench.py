#!/usr/bin/env python
"""Benchmark of the mapreduce / scan / sort hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--detail 0|1]

Headline workload (one "step"): the single-GPU scan configuration the metric is quoted on —
inclusive `scan!(+)` over Float32 n=2^28 (x ~ U[0,1)) and over UInt32 n=2^28 (x ~ U{0..255}),
i.e. 2 * 8n = 4.29 GB of algorithmic traffic per GPU per step. With N > 1 every rank holds its own
2^28-element shard of one global array of N*2^28 elements (weak scaling); a step is the sharded
scan: local reduce, exchange of the shard totals (a kernel of the library over mapped peer memory), local
scan seeded with the totals of the shards before.

`value` is whole-job effective GB/s (algorithmic bytes / device time) with the inputs resident in
HBM; `e2e` is the same metric through the host-buffer API (pinned host arrays in, host arrays out,
copies inside the timed region). `roofline` describes the dominant kernel (the look-back scan
kernel) against the measured HBM copy peak; `cpu_baseline` is the Base-like CPU code of oracle/
timed on this host; `primitives` lists the other configurations (mapreduce, affine scan, sorts)
measured the same way after the timed region.

`--impl reference` times the reference's CPU path (Julia Base semantics restated in oracle/,
the reference itself being Julia, which this machine does not have) on the same step (n = 2^28 per
array) with all host threads, the 1-thread figure beside it; both arms print the same `metric` and
`config`. With N > 1 the GPU arm also reports the sharded mapreduce and the sample sort at 2^28 per
GPU under `primitives`.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_HEADLINE = 1 << 28
NOMINAL_HBM_GBS = 8000.0
# One string for both arms: the driver divides the two lines only when metric, unit and direction agree.
METRIC = "effective GB/s, inclusive scan(+), Float32 + UInt32 at n=2^28 per GPU"


def workload_config(world):
    """The `config` object of the JSON line, identical for the GPU arm and the reference arm."""
    n = N_HEADLINE
    return {"workload": "inclusive scan!(+, dst, x): Float32 x~U[0,1) n=2^28 and UInt32 x~U{0..255} n=2^28 "
                        "per GPU" + ("" if world == 1 else "; sharded over %d GPUs (global n=%d*2^28): local "
                                     "reduce, exchange of the shard totals over mapped peer memory, seeded local scan" % (world, world)),
            "n_per_gpu": n, "algorithmic_bytes_per_step": world * 2 * 8 * n,
            "l2": "inputs (1 GiB per array) are larger than the 126 MB L2; no flush needed"}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for p in self.samples:
            try:
                sm.append(float(p[0]))
                mx.append(float(p[1]))
            except ValueError:
                continue
            for name, v in zip(names, p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# CPU arm (oracle/: the Base-like restatement)
# ---------------------------------------------------------------------------------------------
def host_threads():
    """Host threads this process may use: its CPU affinity, not OMP_NUM_THREADS (torchrun sets that to 1)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


class CpuScanWorkload:
    """Host arrays of the headline step (Float32 U[0,1) and UInt32 U{0..255}, n elements each) and the
    Base-like accumulate over both, timed with the wall clock."""

    def __init__(self, n, seed=0):
        import numpy as np
        from oracle import oracle as O
        self.O, self.n = O, n
        rng = np.random.default_rng(seed)
        self.xf = rng.random(n, dtype=np.float32)
        self.xu = np.frombuffer(rng.bytes(n), dtype=np.uint8).astype(np.uint32)  # uniform over {0..255}
        self.of, self.ou = np.empty_like(self.xf), np.empty_like(self.xu)
        self.nbytes = 2 * 8 * n

    def step(self, threads):
        t0 = time.perf_counter()
        self.O.base_accumulate(self.xf, self.of, threads)
        self.O.base_accumulate(self.xu, self.ou, threads)
        return time.perf_counter() - t0

    def best_gbs(self, threads, repeats):
        self.step(threads)  # warm the pages
        return self.nbytes / min(self.step(threads) for _ in range(repeats)) / 1e9


def cpu_baseline_object(work, threads):
    gbs = work.best_gbs(threads, 3)
    gbs1 = work.best_gbs(1, 2) if threads > 1 else gbs
    return {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port",
            "value_1_thread": round(gbs1, 3),
            "sample": "one full step: accumulate(+) over the Float32 and the UInt32 array of n=2^%d each, best of 3 "
                      "(1 thread: best of 2), C restatement of Base.accumulate (oracle/kf_oracle.c); the 1-thread figure "
                      "is the faithful stand-in for Julia's single-threaded Base.accumulate" % (work.n.bit_length() - 1)}


def cpu_primitive_legs(work, threads):
    """CPU figures for the other primitives (Base-like C code of oracle/, 1 thread and all cores)."""
    import numpy as np
    O = work.O
    out = {}

    def both(fn, nbytes):
        res = {}
        for name, t in (("cpu_1_thread", 1), ("cpu_all_cores", threads)):
            best = float("inf")
            for _ in range(2):
                t0 = time.perf_counter()
                fn(t)
                best = min(best, time.perf_counter() - t0)
            res[name] = {"GB/s": round(nbytes / best / 1e9, 2), "ms": round(best * 1e3, 2)}
        res["cores"] = threads
        return res

    n = work.n
    out["mapreduce_f32_sum_2p28"] = both(lambda t: O.base_mapreduce_add_f32(O.MAP_IDENTITY, work.xf, t), 4 * n)
    ns = 1 << 26
    rng = np.random.default_rng(1)
    keys = rng.integers(0, 1 << 32, ns, dtype=np.uint64).astype(np.uint32)
    kk, tk = np.empty_like(keys), np.empty_like(keys)
    vals, tv = np.empty(ns, dtype=np.uint32), np.empty(ns, dtype=np.uint32)

    def sort_keys(t):
        np.copyto(kk, keys)
        O.base_sort_k32(kk, None, tk, None, t)

    def sort_pairs(t):
        np.copyto(kk, keys)
        vals[:] = np.arange(ns, dtype=np.uint32)
        O.base_sort_k32(kk, vals, tk, tv, t)

    r = both(sort_keys, 36 * ns)
    r["sample"] = "n=2^26 keys (1/4 of the GPU case; the timed call includes the copy that restores the unsorted keys)"
    out["sort_u32_keys_2p28"] = r
    r = both(sort_pairs, 68 * ns)
    r["sample"] = "n=2^26 pairs (1/4 of the GPU case; includes restoring keys and payload)"
    out["sort_u32_keys_u32_payload_2p28"] = r
    return out


def run_reference_arm(args):
    """The reference's CPU path for the headline step (Base.accumulate restated in oracle/kf_oracle.c:
    KernelForge.jl itself is Julia, which this machine does not have), on the full n = 2^28 per array,
    with all host threads as `value` and the 1-thread figure beside it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    threads = host_threads()
    work = CpuScanWorkload(N_HEADLINE)
    for _ in range(args.warmup):
        work.step(threads)
    t0 = time.perf_counter()
    secs = sum(work.step(threads) for _ in range(args.steps))
    wall = time.perf_counter() - t0
    gbs = args.steps * work.nbytes / secs / 1e9
    gbs1 = work.best_gbs(1, 2) if threads > 1 else gbs
    sample = ("each step = the Float32 and the UInt32 array of n=2^28 (one GPU's share of the workload: 2 GiB in, "
              "2 GiB out), all %d host threads; KernelForge.jl is Julia (not installed here), so the CPU path is the C "
              "restatement of Base.accumulate in oracle/kf_oracle.c" % threads)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * secs / args.steps, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32+u32", "data": "synthetic",
        "config": workload_config(world),
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port",
                         "value_1_thread": round(gbs1, 3), "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": round(wall, 2),
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def time_gpu(fn, iters, torch, sync_each=False):
    """Average milliseconds per call of fn(), CUDA events on the current stream."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(iters):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters


CSV_COLUMNS = ["n", "type", "method", "mean_kernel_us", "std_kernel_us", "mean_total_us", "std_total_us",
               "bytes_algorithmic", "gbps", "pct_roofline", "gpus"]


def primitives_csv_rows(primitives, gpus, peak):
    """The `primitives` table as rows of the reference's benchmark CSV
    (`n,type,method,mean_kernel_us,std_kernel_us,mean_total_us,std_total_us`, perfs/julia/bench_utils.jl:7-22 of
    KernelForge.jl) with `bytes_algorithmic,gbps,pct_roofline,gpus` added. `mean_total_us` is the device time of
    one library call (its workspace clear included); the kernel-only and spread columns stay empty, this
    bench does not measure them. `n` and `type` are read from the entry's name (`..._f32_..._2p28...`)."""
    import re
    rows = []
    for name, v in primitives.items():
        m = re.search(r"_2p(\d+)", name)
        t = re.search(r"_(f32x2|f32|f64|u8|i8|u16|i16|u32|i32|u64|i64)(?=_|$)", name)
        gbps = float(v["GB/s"])
        rows.append({"n": (1 << int(m.group(1))) if m else "", "type": t.group(1) if t else "", "method": "kf_b200:" + name,
                     "mean_kernel_us": "", "std_kernel_us": "", "mean_total_us": round(float(v["ms"]) * 1e3, 3), "std_total_us": "",
                     "bytes_algorithmic": v.get("algorithmic_bytes", ""), "gbps": gbps,
                     "pct_roofline": round(100.0 * gbps / (peak * gpus), 2), "gpus": gpus})
    return rows


def write_primitives_csv(path, primitives, gpus, peak):
    import csv
    with open(path, "w", newline="") as fh:
        w = csv.DictWriter(fh, fieldnames=CSV_COLUMNS)
        w.writeheader()
        w.writerows(primitives_csv_rows(primitives, gpus, peak))


def primitives_table(kf, torch, peak, iters=10):
    """Effective GB/s of every other configuration of the path at its full size, one GPU."""
    out = {}
    n = N_HEADLINE
    g = torch.Generator(device="cuda").manual_seed(0)

    def add(name, nbytes, ms, launches):
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": round(ms, 4), "GB/s": round(gbs, 1), "frac_of_measured_peak": round(gbs / peak, 4),
                     "frac_of_nominal_8TBs": round(gbs / NOMINAL_HBM_GBS, 4), "algorithmic_bytes": nbytes,
                     "kernel_launches": launches}

    xf = torch.rand(n, dtype=torch.float32, device="cuda", generator=g)
    dst1 = torch.empty(1, dtype=torch.float32, device="cuda")
    tmp = kf.get_allocation(kf.MapReduce1D, kf.identity, "+", xf)
    fn = lambda: kf.mapreduce_(kf.identity, "+", dst1, xf, tmp=tmp)
    for _ in range(3):
        fn()
    add("mapreduce_f32_sum_2p28", 4 * n, time_gpu(fn, iters * 2, torch), 2)
    # BASELINE config 1 (n = 2^20, launch-bound): the bare C-ABI call, as a Julia `ccall` would issue it
    from kernelforge_jl_b200 import _cabi as C
    small, st = xf[: 1 << 20], torch.cuda.current_stream().cuda_stream
    args1 = (C.MAP_ABS2, C.OP_ADD, C.POST_IDENTITY, C.F32, small.data_ptr(), 1 << 20, dst1.data_ptr(), tmp.ptr(), tmp.nbytes, None, st)

    def fn():
        if kf.lib.kf_mapreduce(*args1) != 0:
            raise SystemExit("bench: kf_mapreduce failed")
    for _ in range(20):
        fn()
    add("mapreduce_f32_abs2_2p20", 4 << 20, time_gpu(fn, 1000, torch), 2)
    out["mapreduce_f32_abs2_2p20"]["note"] = ("per call of kf_mapreduce through ctypes, 1000 back-to-back calls: a kernel that clears "
                                              "the 256-byte header and the reduction chained behind it; launch-bound")
    yf = torch.rand(n, dtype=torch.float32, device="cuda", generator=g)
    fn = lambda: kf.mapreduce_(kf.prod, "+", dst1, (xf, yf), tmp=tmp)
    for _ in range(3):
        fn()
    add("mapreduce_dot_f32_2p28", 8 * n, time_gpu(fn, iters * 2, torch), 1)
    del yf

    na = 1 << 26
    a = 0.5 + 0.5 * torch.rand(na, dtype=torch.float32, device="cuda", generator=g)
    b = 2.0 * torch.rand(na, dtype=torch.float32, device="cuda", generator=g) - 1.0
    da, db = torch.empty_like(a), torch.empty_like(b)
    tmpa = kf.get_allocation(kf.Scan1D, kf.identity, kf.AffineCompose(), (a, b))
    fn = lambda: kf.scan_(kf.AffineCompose(), (da, db), (a, b), tmp=tmpa)
    for _ in range(3):
        fn()
    add("scan_affine_f32x2_2p26", 16 * na, time_gpu(fn, iters * 2, torch), 1)
    del a, b, da, db, tmpa

    def rand_u32():
        return torch.randint(0, 1 << 32, (n,), dtype=torch.int64, device="cuda", generator=g).to(torch.int32).view(torch.uint32)

    keys = rand_u32()
    work = torch.empty_like(keys)
    tmps = kf.get_allocation(kf.Sort1D, keys)

    def sort_once(src, ws):
        # out of place: the unsorted input is read again every iteration, nothing to restore
        kf.sort_(work.view(src.dtype), src, tmp=ws)

    for _ in range(2):
        sort_once(keys, tmps)
    add("sort_u32_keys_2p28", 36 * n, time_gpu(lambda: sort_once(keys, tmps), iters, torch), 6)
    kfl = torch.randn(n, dtype=torch.float32, device="cuda", generator=g)
    for _ in range(2):
        sort_once(kfl, tmps)
    add("sort_f32_keys_2p28", 36 * n, time_gpu(lambda: sort_once(kfl, tmps), iters, torch), 6)
    del kfl, tmps
    k16 = torch.randint(-32768, 32768, (n,), dtype=torch.int16, device="cuda", generator=g)
    w16 = torch.empty_like(k16)
    tmp16 = kf.get_allocation(kf.Sort1D, k16)
    f16 = lambda: kf.sort_(w16, k16, tmp=tmp16)
    for _ in range(2):
        f16()
    add("sort_i16_keys_2p28", (2 * 2 + 1) * 2 * n, time_gpu(f16, iters, torch), 3)
    out["sort_i16_keys_2p28"]["note"] = ("keys without payload: 65536-bin histogram, scan and fill (no key moves); bytes counted "
                                         "as for two 8-bit passes, the DRAM traffic is 4n")
    del k16, w16, tmp16
    k8 = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda", generator=g)
    w8 = torch.empty_like(k8)
    tmp8 = kf.get_allocation(kf.Sort1D, k8)
    f8 = lambda: kf.sort_(w8, k8, tmp=tmp8)
    for _ in range(2):
        f8()
    add("sort_u8_keys_2p28", 3 * n, time_gpu(f8, iters * 2, torch), 3)
    out["sort_u8_keys_2p28"]["note"] = "keys without payload: histogram, scan and fill; bytes counted as for one 8-bit pass, the DRAM traffic is 2n"
    tmps8 = kf.get_allocation(kf.Scan1D, kf.identity, "+", k8)
    fs8 = lambda: kf.scan_("+", w8, k8, tmp=tmps8)
    for _ in range(3):
        fs8()
    add("scan_u8_sum_2p28", 2 * n, time_gpu(fs8, iters * 2, torch), 1)
    del k8, w8, tmp8, tmps8
    # the callers one step out: argmax, findfirst (no element matches: the whole array is read), vcopy!
    from kernelforge_jl_b200.search import gt
    ws_am = torch.empty(kf.lib.kf_argmax_workspace_bytes(C.F32, n), dtype=torch.uint8, device="cuda")
    fam = lambda: kf.argmax1d(kf.identity, ">", xf, to_cpu=False, tmp=ws_am)
    for _ in range(3):
        fam()
    add("argmax_f32_2p28", 4 * n, time_gpu(fam, iters * 2, torch), 1)
    import ctypes
    import numpy as np
    two = np.array([2.0], dtype=np.float32)
    found = torch.empty(1, dtype=torch.int64, device="cuda")

    def ffind():
        if kf.lib.kf_find(gt(0).code, 0, C.F32, xf.data_ptr(), n, two.ctypes.data_as(ctypes.c_void_p), found.data_ptr(), st) != 0:
            raise SystemExit("bench: kf_find failed")
    for _ in range(3):
        ffind()
    add("findfirst_f32_2p28_no_match", 4 * n, time_gpu(ffind, iters * 2, torch), 1)
    cp = torch.empty_like(xf)
    fcp = lambda: kf.vcopy_(cp, xf)
    for _ in range(3):
        fcp()
    add("vcopy_f32_2p28", 8 * n, time_gpu(fcp, iters * 2, torch), 1)
    del cp, ws_am
    idx = torch.arange(n, dtype=torch.int32, device="cuda").view(torch.uint32)
    vout = torch.empty_like(idx)
    tmpp = kf.get_allocation(kf.Sort1D, idx, keys=keys)
    fnp = lambda: kf.sort_(vout, idx, keys=keys, keys_dst=work, tmp=tmpp)
    for _ in range(2):
        fnp()
    add("sort_u32_keys_u32_payload_2p28", 68 * n, time_gpu(fnp, iters, torch), 6)
    return out


def run_case(args):
    """One primitive, `--steps` calls at n = 2^log2n on cuda:0, timed with CUDA events. Meant to be run
    under a profiler on a small case (inputs larger than L2, a few hundred MB on the device)."""
    import torch
    from __graft_entry__ import load_package
    kf = load_package()
    torch.cuda.set_device(0)
    n = args.n if args.n else 1 << args.log2n
    g = torch.Generator(device="cuda").manual_seed(0)
    case = args.case
    if case in ("scan_u32", "scan_f32", "scan_f64", "scan_u8", "mapreduce_f32"):
        if case == "scan_u32":
            x = torch.randint(0, 256, (n,), dtype=torch.int32, device="cuda", generator=g).view(torch.uint32)
        elif case == "scan_u8":
            x = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda", generator=g)
        else:
            x = torch.rand(n, dtype=torch.float64 if case == "scan_f64" else torch.float32, device="cuda", generator=g)
        if case == "mapreduce_f32":
            dst = torch.empty(1, dtype=torch.float32, device="cuda")
            tmp = kf.get_allocation(kf.MapReduce1D, kf.identity, "+", x)
            fn, nbytes = (lambda: kf.mapreduce_(kf.identity, "+", dst, x, tmp=tmp)), 4 * n
        else:
            dst = torch.empty_like(x)
            tmp = kf.get_allocation(kf.Scan1D, kf.identity, "+", x)
            fn, nbytes = (lambda: kf.scan_("+", dst, x, tmp=tmp)), 2 * x.element_size() * n
    elif case == "scan_affine":
        a = 0.5 + 0.5 * torch.rand(n, dtype=torch.float32, device="cuda", generator=g)
        b = 2.0 * torch.rand(n, dtype=torch.float32, device="cuda", generator=g) - 1.0
        da, db = torch.empty_like(a), torch.empty_like(b)
        tmp = kf.get_allocation(kf.Scan1D, kf.identity, kf.AffineCompose(), (a, b))
        fn, nbytes = (lambda: kf.scan_(kf.AffineCompose(), (da, db), (a, b), tmp=tmp)), 16 * n
    elif case in ("sort_u32", "sort_f32", "sort_pairs", "sort_u64", "sort_u8", "sort_i16"):
        if case == "sort_u8":
            keys = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda", generator=g)
        elif case == "sort_i16":
            keys = torch.randint(-32768, 32768, (n,), dtype=torch.int16, device="cuda", generator=g)
        elif case == "sort_f32":
            keys = torch.randn(n, dtype=torch.float32, device="cuda", generator=g)
        elif case == "sort_u64":
            keys = torch.randint(-2**63, 2**63 - 1, (n,), dtype=torch.int64, device="cuda", generator=g).view(torch.uint64)
        else:
            keys = torch.randint(0, 1 << 32, (n,), dtype=torch.int64, device="cuda", generator=g).to(torch.int32).view(torch.uint32)
        out = torch.empty_like(keys)
        if case == "sort_pairs":
            idx = torch.arange(n, dtype=torch.int32, device="cuda").view(torch.uint32)
            vout = torch.empty_like(idx)
            tmp = kf.get_allocation(kf.Sort1D, idx, keys=keys)
            fn, nbytes = (lambda: kf.sort_(vout, idx, keys=keys, keys_dst=out, tmp=tmp)), 68 * n
        else:
            tmp = kf.get_allocation(kf.Sort1D, keys)
            fn, nbytes = (lambda: kf.sort_(out, keys, tmp=tmp)), {"sort_u64": 136, "sort_u8": 3, "sort_i16": 10}.get(case, 36) * n
    elif case in ("argmax_f32", "findfirst_f32", "vcopy_f32"):
        x = torch.rand(n, dtype=torch.float32, device="cuda", generator=g)
        tmp = kf.get_allocation(kf.MapReduce1D, kf.identity, "+", x)  # (only so that the common status check below has a workspace)
        kf.mapreduce_(kf.identity, "+", torch.empty(1, dtype=torch.float32, device="cuda"), x, tmp=tmp)
        if case == "argmax_f32":
            from kernelforge_jl_b200 import _cabi as C
            ws = torch.empty(kf.lib.kf_argmax_workspace_bytes(C.F32, n), dtype=torch.uint8, device="cuda")
            fn, nbytes = (lambda: kf.argmax1d(kf.identity, ">", x, to_cpu=False, tmp=ws)), 4 * n
        elif case == "findfirst_f32":  # no element matches: the whole array is read
            import ctypes
            import numpy as np
            from kernelforge_jl_b200 import _cabi as C
            two = np.array([2.0], dtype=np.float32)
            found = torch.empty(1, dtype=torch.int64, device="cuda")
            st = torch.cuda.current_stream().cuda_stream
            fn = lambda: kf.lib.kf_find(C.PRED_GT, 0, C.F32, x.data_ptr(), n, two.ctypes.data_as(ctypes.c_void_p), found.data_ptr(), st)
            nbytes = 4 * n
        else:
            y = torch.empty_like(x)
            fn, nbytes = (lambda: kf.vcopy_(y, x)), 8 * n
    else:
        raise SystemExit("unknown --case %r" % case)
    fn()
    ms = time_gpu(fn, max(1, args.steps), torch)
    rc = kf.lib.kf_check(tmp.ptr(), None)
    print(json.dumps({"case": case, "n": n, "ms": round(ms, 4), "GB/s": round(nbytes / ms / 1e6, 1), "device_status": rc}))
    return 0 if rc == 0 else 1


def run_sharded(args):
    """Global n = 2^global_log2n split into equal contiguous shards: mapreduce(+) over Float32 U[0,1),
    inclusive scan over UInt32 U{0..255}, sample sort of uniform UInt32 keys (1024 samples per GPU,
    NCCL all-to-all). Device-timed, max over ranks; results are verified with size-independent checks."""
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    kf = load_package()
    from kernelforge_jl_b200 import distributed as kfd
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", local))
    peak, _ = measured_peak()
    n = 1 << args.global_log2n
    n_per = n // world
    g = torch.Generator(device="cuda").manual_seed(7000 + rank)
    group = kfd.ShardGroup()

    def fill_u32(full_range):
        out = torch.empty(n_per, dtype=torch.int32, device="cuda")
        step = 1 << 26
        for lo in range(0, n_per, step):
            hi = min(n_per, lo + step)
            hi_val = (1 << 32) if full_range else 256
            out[lo:hi] = torch.randint(0, hi_val, (hi - lo,), dtype=torch.int64, device="cuda", generator=g).to(torch.int32)
        return out.view(torch.uint32)

    def timed(fn, iters):
        for _ in range(2):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / iters], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    res = {}
    xf = torch.rand(n_per, dtype=torch.float32, device="cuda", generator=g)
    ms = timed(lambda: kfd.mapreduce(group, kf.identity, "+", xf, to_cpu=False), args.steps)
    got = kfd.mapreduce(group, kf.identity, "+", xf)
    ref = xf.sum(dtype=torch.float64)
    dist.all_reduce(ref)
    assert abs(got - ref.item()) <= 1e-5 * args.global_log2n * ref.item(), (got, ref.item())
    res["mapreduce_f32"] = (4 * n, ms)
    del xf

    xu = fill_u32(False)
    du = torch.empty_like(xu)
    tmp = kf.get_allocation(kf.Scan1D, kf.identity, "+", xu)
    ms = timed(lambda: kfd.scan_(group, "+", du, xu, tmp=tmp), args.steps)
    d32, x32 = du.view(torch.int32), xu.view(torch.int32)
    assert bool(((d32[1:] - d32[:-1]) == x32[1:]).all().item())
    tot = x32.sum(dtype=torch.int64).reshape(1)
    tots = [torch.zeros_like(tot) for _ in range(world)]
    dist.all_gather(tots, tot)
    expect_last = int(sum(int(t.item()) for t in tots[: rank + 1])) & 0xFFFFFFFF
    assert (int(d32[-1].item()) & 0xFFFFFFFF) == expect_last
    res["scan_u32"] = (8 * n, ms)
    del xu, du, tmp, d32, x32

    keys = fill_u32(True)
    k64 = keys.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    chk = torch.stack([k64.sum(), (k64 * k64 + 7 * k64).sum()])
    del k64
    dist.all_reduce(chk)
    out_holder = {}

    def do_sort():
        out_holder["r"] = kfd.sort(group, keys)
    ms = timed(do_sort, max(1, args.steps // 2))
    chunk, counts = out_holder["r"]
    assert sum(counts) == n
    c64 = chunk.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    assert bool((c64[1:] >= c64[:-1]).all().item())
    chk2 = torch.stack([c64.sum(), (c64 * c64 + 7 * c64).sum()])
    dist.all_reduce(chk2)
    assert torch.equal(chk, chk2)
    edge = torch.stack([c64[0], c64[-1]])
    edges = [torch.zeros_like(edge) for _ in range(world)]
    dist.all_gather(edges, edge)
    for r in range(1, world):
        assert int(edges[r][0].item()) >= int(edges[r - 1][1].item())
    res["sample_sort_u32"] = (36 * n, ms)
    imbalance = max(counts) / (n / world)

    if rank == 0:
        line = {"metric": "effective GB/s (single-device algorithmic bytes on the global n / max device time over ranks)",
                "n_gpus": world, "scaling": "strong", "data": "synthetic", "global_n": n, "steps": args.steps,
                "config": {"workload": "sharded: mapreduce(+) Float32, inclusive scan UInt32, sample sort UInt32 keys; "
                                       "global n=2^%d in %d contiguous shards" % (args.global_log2n, world),
                           "sort_max_piece_over_mean": round(imbalance, 4)},
                "results": {k: {"ms": round(ms_, 4), "GB/s": round(b / ms_ / 1e6, 1),
                                "frac_of_measured_peak_x_gpus": round(b / ms_ / 1e6 / (peak * world), 4),
                                "frac_of_nominal_8TBs_x_gpus": round(b / ms_ / 1e6 / (NOMINAL_HBM_GBS * world), 4)}
                            for k, (b, ms_) in res.items()}}
        print(json.dumps(line))
    group.close()
    dist.barrier()
    dist.destroy_process_group()
    return 0


def pin_rank_to_core_slice(local, world):
    """Gives each rank its own slice of the visible cores (before any pinned allocation, so that the
    pinned pages and the copy threads of a rank stay on one socket's cores)."""
    try:
        cores = sorted(os.sched_getaffinity(0))
        if world > 1 and len(cores) >= world:
            per = len(cores) // world
            os.sched_setaffinity(0, cores[local * per:(local + 1) * per])
        return len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        return None


def sharded_primitives(kf, kfd, torch, dist, group, peak, iters):
    """The other two primitives on the sharded layout, 2^28 elements per GPU (weak scaling): mapreduce(+)
    over Float32 (local kernel + NCCL allreduce) and the sample sort of uniform UInt32 keys (partition
    pass, NCCL all-to-all, local onesweep). Device-timed, max over ranks, checked by size-independent
    properties. Returns {name: {...}} on every rank."""
    world, rank = group.world, group.rank
    n = N_HEADLINE
    g = torch.Generator(device="cuda").manual_seed(5000 + rank)

    def timed(fn, k):
        for _ in range(2):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(k):
            fn()
        b.record()
        dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / k], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out = {}

    def add(name, nbytes, ms, note):
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": round(ms, 4), "GB/s": round(gbs, 1), "frac_of_measured_peak_x_gpus": round(gbs / (peak * world), 4),
                     "frac_of_nominal_8TBs_x_gpus": round(gbs / (NOMINAL_HBM_GBS * world), 4),
                     "algorithmic_bytes": nbytes, "note": note}

    xf = torch.rand(n, dtype=torch.float32, device="cuda", generator=g)
    ms = timed(lambda: kfd.mapreduce(group, kf.identity, "+", xf, to_cpu=False), iters)
    got = kfd.mapreduce(group, kf.identity, "+", xf)
    ref = xf.sum(dtype=torch.float64)
    dist.all_reduce(ref)
    if abs(got - ref.item()) > 1e-5 * 32 * ref.item():
        raise SystemExit("bench: sharded mapreduce is off: %r vs %r" % (got, ref.item()))
    add("sharded_mapreduce_f32_sum_2p28_per_gpu", 4 * n * world, ms, "local mapreduce + NCCL allreduce of one partial per rank")
    del xf

    keys = torch.randint(0, 1 << 32, (n,), dtype=torch.int64, device="cuda", generator=g).to(torch.int32).view(torch.uint32)
    k64 = keys.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    chk = torch.stack([k64.sum(), (k64 * k64 + 7 * k64).sum()])
    del k64
    dist.all_reduce(chk)
    holder = {}

    def do_sort():
        holder["r"] = kfd.sort(group, keys)
    ms = timed(do_sort, max(2, iters // 4))
    chunk, counts = holder["r"]
    c64 = chunk.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    ok = sum(counts) == n * world and bool((c64[1:] >= c64[:-1]).all().item())
    chk2 = torch.stack([c64.sum(), (c64 * c64 + 7 * c64).sum()])
    dist.all_reduce(chk2)
    edge = torch.stack([c64[0], c64[-1]])
    edges = [torch.zeros_like(edge) for _ in range(world)]
    dist.all_gather(edges, edge)
    ok = ok and torch.equal(chk, chk2) and all(int(edges[r][0]) >= int(edges[r - 1][1]) for r in range(1, world))
    if not ok:
        raise SystemExit("bench: sample sort failed its checks (sortedness, checksums, piece boundaries)")
    add("sample_sort_u32_keys_2p28_per_gpu", 36 * n * world, ms,
        "4096 stratified samples per GPU, one partition pass, NCCL all-to-all, local onesweep; largest piece / mean = %.4f"
        % (max(counts) / n))
    return out


def run_gpu_arm(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    cores_of_rank = pin_rank_to_core_slice(local, world)
    torch.cuda.set_device(local)
    kf = load_package()
    from kernelforge_jl_b200 import distributed as kfd
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peak, peak_kind = measured_peak()
    n = N_HEADLINE
    warm = max(args.warmup, 3)

    # Each rank owns shard `rank` of a global array of world*n elements (seeded per shard).
    g = torch.Generator(device="cuda").manual_seed(1000 + rank)
    xf = torch.rand(n, dtype=torch.float32, device="cuda", generator=g)
    xu = torch.randint(0, 256, (n,), dtype=torch.int32, device="cuda", generator=g).view(torch.uint32)
    df, du = torch.empty_like(xf), torch.empty_like(xu)
    tmp_f = kf.get_allocation(kf.Scan1D, kf.identity, "+", xf)
    tmp_u = kf.get_allocation(kf.Scan1D, kf.identity, "+", xu)
    group = kfd.ShardGroup() if world > 1 else None

    def two_scans():
        kf.scan_("+", df, xf, tmp=tmp_f)
        kf.scan_("+", du, xu, tmp=tmp_u)

    # One GPU: the two scan calls (two workspace memsets, two kernels) are recorded once into a CUDA
    # graph and a step replays it, which removes the gaps between the four operations. The sharded step
    # is issued call by call (its exchange kernel takes a new epoch every call).
    captured = None
    if world == 1 and not os.environ.get("KF_BENCH_NO_GRAPH"):
        try:
            captured = kf.CapturedStep(two_scans)
        except Exception as exc:  # noqa: BLE001 - any capture failure falls back to plain calls, and the line says so
            print("bench: CUDA graph capture failed (%s); issuing the calls one by one" % exc, file=sys.stderr)
            captured = None
            torch.cuda.synchronize()

    def step():
        if captured is not None:
            captured.replay()
        elif world == 1:
            two_scans()
        else:  # 2 reductions, 2 seeded scans; each array's allgather runs behind the other array's kernels
            kfd.scan_many_(group, [("+", df, xf, tmp_f), ("+", du, xu, tmp_u)])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warm):
        step()
    barrier()
    # The timed region (K steps of < 1 ms) is shorter than one nvidia-smi sampling period, so the
    # sampler runs over a window of the SAME load around it: untimed steps before and after, a fixed
    # number on every rank (the sharded step contains collectives), sized from the warm-up.
    t0 = time.perf_counter()
    for _ in range(3):
        step()
    barrier()
    per_step_s = max((time.perf_counter() - t0) / 3, 1e-5)
    lead = int(0.6 / per_step_s) + 1
    tail = int(0.25 / per_step_s) + 1
    if world > 1:
        t = torch.tensor([lead, tail], dtype=torch.int64, device="cuda")
        dist.broadcast(t, 0)
        lead, tail = int(t[0].item()), int(t[1].item())
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(lead):
        step()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches0 = int(kf.lib.kf_launch_count())
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    barrier()
    launches = int(kf.lib.kf_launch_count()) - launches0  # kernels of libkf_b200.so launched by this rank in the timed region
    if captured is not None:  # replays do not pass through the library's host code: count what one replay holds
        launches = captured.launches * args.steps
    ms = start.elapsed_time(stop)
    for _ in range(tail):
        step()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = "sampled every 100 ms while %d + %d + %d identical steps ran (before, timed, after)" % (lead, args.steps, tail)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    step_bytes = world * 2 * 8 * n
    value = step_bytes / (ms_per_step * 1e-3) / 1e9

    # Device-side sanity of the timed outputs: wrapping first differences reproduce the input inside the
    # shard, and the shard's first output equals the carry of the shards before it plus its first input
    # (so a wrong carry across a shard boundary cannot pass).
    d32, x32 = du.view(torch.int32), xu.view(torch.int32)
    ok = bool(((d32[1:] - d32[:-1]) == x32[1:]).all().item())
    if world > 1:
        tot = x32.sum(dtype=torch.int64).reshape(1)
        tots = [torch.zeros_like(tot) for _ in range(world)]
        dist.all_gather(tots, tot)
        carry = sum(int(t.item()) for t in tots[:rank])
        ok = ok and ((int(d32[0].item()) - int(x32[0].item()) - carry) & 0xFFFFFFFF) == 0
        fl = xf.sum(dtype=torch.float64).reshape(1)
        fls = [torch.zeros_like(fl) for _ in range(world)]
        dist.all_gather(fls, fl)
        want = sum(float(t.item()) for t in fls[: rank + 1])
        ok = ok and abs(float(df[-1].item()) - want) <= 1e-5 * 32 * want
    if not ok:
        raise SystemExit("bench: scan output failed its difference / shard-boundary check")

    # ---- roofline of the dominant kernel: the UInt32/Float32 look-back scan kernel, single GPU view
    kern_ms = time_gpu(lambda: kf.scan_("+", du, xu, tmp=tmp_u), 20, torch)
    achieved = 8 * n / (kern_ms * 1e-3) / 1e9
    traffic = traffic_how = None
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as fh:
            tj = json.load(fh)
        # DRAM reads grow with n (measured ratio to the input at n = 2^26); the output is written once.
        # (Scaling the small case's WRITE counter would undercount: about 58 MB of the output are still
        # in L2 when the kernel ends, a constant, not a share of n.)
        traffic = int(round(tj["scan_kernel_roles_u32_read_ratio"] * 4 * n + 4 * n))
        traffic_how = tj["_how"]
    except Exception:
        pass
    # The same kernel and a plain copy under SUSTAINED load (0.5 s of back-to-back launches first: the
    # 1 kW power cap then lowers the SM clock), and the headline steps timed as a burst after an idle
    # pause: the two regimes MEASURED_PEAKS.json distinguishes.
    def sustained_ms(fn, iters):
        t_end = time.perf_counter() + 0.5
        while time.perf_counter() < t_end:
            for _ in range(50):
                fn()
            torch.cuda.synchronize()
        return time_gpu(fn, iters, torch)
    k_ms = sustained_ms(lambda: kf.scan_("+", du, xu, tmp=tmp_u), 20)
    c_ms = sustained_ms(lambda: du.copy_(xu), 20)
    sustained = {"achieved": round(8 * n / (k_ms * 1e-3) / 1e9, 1), "copy_measured_here": round(8 * n / (c_ms * 1e-3) / 1e9, 1),
                 "frac_of_copy": round(c_ms / k_ms, 4), "unit": "GB/s"}
    burst = None
    if world == 1:
        torch.cuda.synchronize()
        time.sleep(0.5)
        b_ms = time_gpu(step, args.steps, torch)
        burst = {"value": round(step_bytes / (b_ms * 1e-3) / 1e9, 1), "ms_per_step": round(b_ms, 4),
                 "note": "the same K steps timed right after 0.5 s of idle (no power capping yet); `value` is timed inside the sustained window"}
    roofline = {"bound": "hbm", "kernel": "scan_kernel_roles<uint32, +, 384x8, 2 buffers, reduction 3 tiles ahead>", "achieved": round(achieved, 1),
                "peak": peak, "peak_kind": peak_kind + " (STREAM-style copy)", "unit": "GB/s",
                "frac": round(achieved / peak, 4), "frac_of_nominal_8TBs": round(achieved / NOMINAL_HBM_GBS, 4),
                "algorithmic_bytes_per_launch": 8 * n, "kernel_ms": round(kern_ms, 4), "traffic": traffic,
                "traffic_how": traffic_how, "sustained": sustained}

    # ---- end to end through the host-buffer API: pinned host arrays in, host arrays out
    hf = torch.empty(n, dtype=torch.float32).pin_memory()
    hu = torch.empty(n, dtype=torch.int32).pin_memory()
    hf.copy_(xf)
    hu.copy_(xu.view(torch.int32))
    of = torch.empty(n, dtype=torch.float32).pin_memory()
    ou = torch.empty(n, dtype=torch.int32).pin_memory()
    pipe = kfd.HostScanPipeline(kf, n, chunk_bytes=args.e2e_chunk_mb << 20, slots=4)

    def e2e_step():
        pipe.scan_host_many([("+", of, hf), ("+", ou.view(torch.uint32), hu.view(torch.uint32))])

    def timed_host(fn, k):
        for _ in range(2):
            fn()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(k):
            fn()
        b.record()
        barrier()
        v = a.elapsed_time(b) / k
        if world > 1:
            t = torch.tensor([v], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            v = float(t.item())
        return v

    e_steps = max(2, min(args.steps, 5))
    e_ms = timed_host(e2e_step, e_steps)
    if not bool((ou[1:] - ou[:-1] == hu[1:]).all().item()):
        raise SystemExit("bench: host-pipeline scan output failed its difference check")

    # The ceiling of that number: the same bytes as plain pinned copies in both directions at once (no
    # kernel), on all ranks at the same time.
    s_up, s_down = torch.cuda.Stream(), torch.cuda.Stream()

    def copy_only():
        cur = torch.cuda.current_stream()
        s_up.wait_stream(cur)
        s_down.wait_stream(cur)
        with torch.cuda.stream(s_up):
            df.copy_(hf, non_blocking=True)
            du.view(torch.int32).copy_(hu, non_blocking=True)
        with torch.cuda.stream(s_down):
            of.copy_(xf, non_blocking=True)
            ou.copy_(xu.view(torch.int32), non_blocking=True)
        cur.wait_stream(s_up)
        cur.wait_stream(s_down)
    c_host_ms = timed_host(copy_only, e_steps)
    e2e = {"value": round(world * 2 * 8 * n / (e_ms * 1e-3) / 1e9, 2), "unit": "GB/s",
           "h2d_bytes_per_step": 2 * 4 * n, "d2h_bytes_per_step": 2 * 4 * n, "ms_per_step": round(e_ms, 3),
           "copy_ceiling": {"value": round(world * 2 * 8 * n / (c_host_ms * 1e-3) / 1e9, 2), "unit": "GB/s",
                            "ms_per_step": round(c_host_ms, 3),
                            "what": "the same 2 GiB up and 2 GiB down per rank as plain pinned-memory copies on two "
                                    "streams, all %d ranks at once, no kernel: what the host side of the box delivers" % world},
           "frac_of_copy_ceiling": round(c_host_ms / e_ms, 4), "host_cores_of_this_rank": cores_of_rank,
           "note": "independent per-rank host arrays; %d MiB chunks through a 4-slot device ring: H2D / scan(init=carry) / D2H on three streams" % args.e2e_chunk_mb}
    del hf, hu, of, ou, pipe

    prim = None
    if args.detail:
        if world == 1:
            prim = primitives_table(kf, torch, peak)
        else:
            prim = sharded_primitives(kf, kfd, torch, dist, group, peak, max(4, args.steps // 2))

    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 1),
            "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "warmup_run": warm,
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32+u32", "data": "synthetic",
            "frac_of_measured_peak": round(value / (peak * world), 4),
            "frac_of_nominal_8TBs": round(value / (NOMINAL_HBM_GBS * world), 4),
            "config": workload_config(world),
            "roofline": roofline, "e2e": e2e, "gpu_launches": launches,
            "gpu_launches_how": ("kernels of libkf_b200.so in one replay of the captured step (kf_launch_count() around the capture) "
                                 "x steps: 2 scan kernels per step" if captured is not None else
                                 "kf_launch_count() of libkf_b200.so before and after the timed region on rank 0 (%s per step)"
                                 % ("2 scan kernels" if world == 1 else "2 reductions, 2 exchange kernels, 2 seeded scans")),
            "step_launch": "one CUDA graph replay per step (the two kf_scan calls recorded once)" if captured is not None
                           else "library calls issued one by one on the stream",
            "clocks": clocks, "burst": burst,
        }
        if world == 1:
            work = CpuScanWorkload(n)
            threads = host_threads()
            line["cpu_baseline"] = cpu_baseline_object(work, threads)
            if prim is not None:
                for k, v in cpu_primitive_legs(work, threads).items():
                    if k in prim:
                        prim[k]["cpu"] = v
        if prim is not None:
            line["primitives"] = prim
        if args.csv:
            write_primitives_csv(args.csv, prim, world, peak)
        print(json.dumps(line))
    if world > 1:
        group.close()
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--detail", type=int, default=1, help="1: also measure the other primitives (single GPU)")
    ap.add_argument("--case", default=None,
                    help="run ONE primitive a few times at n=2^log2n and exit (small case for profiler captures): "
                         "scan_u32, scan_f32, scan_f64, scan_u8, scan_affine, mapreduce_f32, sort_u32, sort_f32, sort_u64, sort_u8, sort_i16, sort_pairs, argmax_f32, findfirst_f32, vcopy_f32")
    ap.add_argument("--log2n", type=int, default=26)
    ap.add_argument("--n", type=int, default=0, help="with --case: an exact element count instead of 2^log2n")
    ap.add_argument("--sharded", action="store_true",
                    help="measure the sharded configuration instead (mapreduce, scan and sample sort over one global "
                         "array of 2^--global-log2n elements split across the ranks; strong scaling)")
    ap.add_argument("--global-log2n", type=int, default=32)
    ap.add_argument("--e2e-chunk-mb", type=int, default=32, help="chunk size of the host-buffer pipeline (MiB)")
    ap.add_argument("--csv", default=None, help="also write the primitives table to this file in the reference's benchmark CSV schema")
    args = ap.parse_args()
    if args.case:
        return run_case(args)
    if args.sharded:
        return run_sharded(args)
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
