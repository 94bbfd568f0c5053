#!/usr/bin/env python
"""Runs the reference's CUB / Thrust comparator harnesses (built by baseline/Makefile into
baseline/_ref/) on the current GPU and prints one table.

The harnesses are the reference's own files (perfs/cuda_cpp/cub_nvcc/*.cu of KernelForge.jl),
compiled unmodified; this script only calls them with the command lines the reference's comparison
scripts use (`-n N -t TYPE -i ITER -w WARMUP_MS -j`, e.g. perfs/julia/benchmarks/scan_perf_comparison.jl)
and recomputes GB/s from their `mean_ms` with the byte counts this repository uses everywhere:
reduce n*sizeof(T), scan 2*n*sizeof(T), 8-bit-digit radix sort (2P+1)*n*sizeof(K). (The harnesses'
own `throughput_gb_s` uses other conventions: GiB, and 2*N*sizeof(T) for sorts.)

    python baseline/run_cub.py [--log2n 28 | --n 100000000] [--iters 20] [--out FILE]
"""
import argparse
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

# (binary, extra args, label, algorithmic bytes per element)
CASES = [
    ("cub_memcpy_benchmark", ["-t", "float"], "cudaMemcpy D2D Float32", 8),
    ("cub_sum_benchmark", ["-t", "float"], "cub::DeviceReduce::Sum Float32", 4),
    ("cub_scan_benchmark", ["-t", "float", "-m", "inclusive"], "cub::DeviceScan::InclusiveSum Float32", 8),
    ("cub_scan_benchmark", ["-t", "int", "-m", "inclusive"], "cub::DeviceScan::InclusiveSum Int32 (4-byte integer stand-in for UInt32)", 8),
    ("cub_scan_benchmark", ["-t", "double", "-m", "inclusive"], "cub::DeviceScan::InclusiveSum Float64", 16),
    ("cub_sort_benchmark", ["-t", "uint32"], "cub::DeviceRadixSort::SortKeys UInt32", 36),
    ("cub_sort_benchmark", ["-t", "float"], "cub::DeviceRadixSort::SortKeys Float32", 36),
    ("cub_sort_benchmark", ["-t", "uint64"], "cub::DeviceRadixSort::SortKeys UInt64", 136),
    ("thrust_sort_benchmark", ["-t", "uint32"], "thrust::sort UInt32", 36),
]


def first_json_object(text):
    """The harnesses print one JSON object (possibly after other lines)."""
    start = text.find("{")
    while start >= 0:
        depth = 0
        for i in range(start, len(text)):
            if text[i] == "{":
                depth += 1
            elif text[i] == "}":
                depth -= 1
                if depth == 0:
                    try:
                        return json.loads(text[start:i + 1])
                    except ValueError:
                        break
        start = text.find("{", start + 1)
    return None


def find_mean_ms(obj):
    if isinstance(obj, dict):
        if "mean_ms" in obj:
            return float(obj["mean_ms"])
        for v in obj.values():
            r = find_mean_ms(v)
            if r is not None:
                return r
    if isinstance(obj, list):
        for v in obj:
            r = find_mean_ms(v)
            if r is not None:
                return r
    return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--log2n", type=int, default=28)
    ap.add_argument("--n", type=int, default=0, help="an exact element count instead of 2^log2n (the reference publishes 10^6, 10^7, 10^8)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup-ms", type=int, default=200)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    n = args.n if args.n else 1 << args.log2n
    rows = []
    for binary, extra, label, bpe in CASES:
        exe = os.path.join(REF, binary)
        if not os.path.exists(exe):
            rows.append({"case": label, "error": "not built: run `make -C baseline` where the reference checkout is present"})
            continue
        cmd = [exe, "-n", str(n), "-i", str(args.iters), "-w", str(args.warmup_ms), "-j"] + extra
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        except subprocess.TimeoutExpired:
            rows.append({"case": label, "error": "timed out"})
            continue
        obj = first_json_object(r.stdout)
        ms = find_mean_ms(obj) if obj is not None else None
        if r.returncode != 0 or ms is None:
            rows.append({"case": label, "error": "rc=%d %s" % (r.returncode, (r.stderr or r.stdout)[-200:].strip())})
            continue
        rows.append({"case": label, "cmd": " ".join([binary] + cmd[1:]), "n": n, "mean_ms": round(ms, 4),
                     "bytes_per_element": bpe, "GB/s": round(bpe * n / ms / 1e6, 1)})
    print("| harness call | mean ms | algorithmic bytes / element | GB/s |\n|---|---|---|---|")
    for r in rows:
        if "error" in r:
            print("| %s | %s | | |" % (r["case"], r["error"]))
        else:
            print("| %s | %.4f | %d | %.0f |" % (r["case"], r["mean_ms"], r["bytes_per_element"], r["GB/s"]))
    if args.out:
        with open(args.out, "w") as fh:
            json.dump(rows, fh, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
