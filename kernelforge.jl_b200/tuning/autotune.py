"""Builds the B200 launch table from measurements, the way the reference's autotuners build its
per-architecture tuning files (data/tuning/{mapreduce1d,scan,sort}/autotune.jl of KernelForge.jl).

    python kernelforge.jl_b200/tuning/autotune.py sweep  [--out FILE] [--log2n 16,18,...] [--only scan,sort_keys]
    python kernelforge.jl_b200/tuning/autotune.py choose [--in FILE]  [--write]

`sweep` times every compiled launch variant of every primitive on the current GPU for each cell
(primitive, element bytes, log2 n) and appends one JSON line per measurement to FILE. It is
resumable per cell: cells already in FILE are skipped, so an interrupted run continues where it
stopped. Every variant is measured in two interleaved rounds and the faster round counts.

`choose` turns the measurements into table rows with the reference's rules:
  * the current table entry is always one of the candidates
    (data/tuning/mapreduce1d/autotune.jl:162-179);
  * it is only replaced where another variant wins by more than 6 % (data/tuning/sort/autotune.jl:
    143-147,236-253);
  * the boundary between two regimes lies at the geometric midpoint of the neighbouring measured
    sizes (data/tuning/mapreduce1d/autotune.jl:184-214).
It prints the table (markdown) and, with --write, rewrites launch_table.json (every row cites the cells
that chose it) and regenerates csrc/launch_table.h.
"""
import argparse
import ctypes
import importlib.util
import json
import math
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG_DIR = os.path.dirname(HERE)
DEFAULT_OUT = os.path.join(HERE, "sweep_b200.jsonl")
WIN = 0.06  # a variant must beat the current table entry by more than this to replace it

MR_VARIANTS = [(256, 4), (512, 4), (256, 8)]
MR_BLOCKS_PER_SM = [1, 2, 4, 8]
SCAN_VARIANTS = [(256, 4), (512, 4), (256, 8), (128, 8), (768, 4), (384, 8), (512, 8)]
SORT_VARIANTS = [(256, 16), (512, 16), (512, 24), (384, 24)]


def load_package():
    name = "kernelforge_jl_b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(PKG_DIR, "__init__.py"),
                                                  submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


# ---- measuring -------------------------------------------------------------------------------------
def time_call(torch, fn, target_ms=25.0):
    """Milliseconds per call: warm up, size the batch for about `target_ms`, CUDA events."""
    for _ in range(3):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    fn()
    b.record()
    torch.cuda.synchronize()
    one = max(a.elapsed_time(b), 1e-3)
    iters = int(min(400, max(3, target_ms / one)))
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def cells(args):
    log2s = [int(x) for x in args.log2n.split(",")]
    only = set(args.only.split(",")) if args.only else None
    out = []
    for prim, widths in (("mapreduce", (1, 2, 4, 8)), ("scan", (1, 2, 4, 8)), ("scan_affine", (8,)),
                         ("sort_keys", (1, 2, 4, 8)), ("sort_pairs", (8, 16))):
        if only and prim not in only:
            continue
        for w in widths:
            for l in log2s:
                if prim == "scan_affine" and l > 28:
                    continue
                out.append((prim, w, l))
    return out


def run_cell(kf, torch, C, prim, width, log2n):
    """Yields (variant label, threads, items, blocks_per_sm, ms) for every variant of the cell."""
    lib = kf.lib
    n = 1 << log2n
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(log2n * 16 + width)
    int_dt = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}
    code = {1: C.U8, 2: C.I16, 4: C.F32, 8: C.F64}
    key_code = {1: C.U8, 2: C.I16, 4: C.U32, 8: C.U64}
    sms = lib.kf_num_sms()

    def rand_float(dt):
        return torch.rand(n, dtype=dt, device="cuda", generator=g)

    def rand_bits(w):
        lo, hi = {1: (0, 256), 2: (-2**15, 2**15), 4: (-2**31, 2**31), 8: (-2**62, 2**62)}[w]
        return torch.randint(lo, hi, (n,), dtype=int_dt[w], device="cuda", generator=g)

    jobs = []
    if prim == "mapreduce":
        x = rand_bits(width) if width < 4 else rand_float(torch.float32 if width == 4 else torch.float64)
        dst = torch.empty(1, dtype=x.dtype, device="cuda")
        ws = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
        for (t, v) in MR_VARIANTS:
            for per in MR_BLOCKS_PER_SM:
                cfg = ctypes.pointer(C.LaunchCfg(t, v, per * sms, 0))
                if lib.kf_mapreduce_workspace_bytes(code[width], n, cfg) == 0:
                    continue
                jobs.append(("%dx%d, %d CTAs/SM" % (t, v, per), t, v, per,
                             lambda cfg=cfg: lib.kf_mapreduce(0, 0, 0, code[width], x.data_ptr(), n, dst.data_ptr(), ws.data_ptr(),
                                                              ws.numel(), cfg, st)))
    elif prim == "scan":
        x = rand_bits(width) if width < 4 else rand_float(torch.float32 if width == 4 else torch.float64)
        dst = torch.empty_like(x)
        for (t, v) in SCAN_VARIANTS:
            cfg = ctypes.pointer(C.LaunchCfg(t, v, 0, 0))
            need = lib.kf_scan_workspace_bytes(code[width], 0, n, cfg)
            if need == 0:
                continue
            ws = torch.empty(need, dtype=torch.uint8, device="cuda")
            jobs.append(("%dx%d" % (t, v), t, v, 0,
                         lambda cfg=cfg, ws=ws: lib.kf_scan(0, 0, 0, code[width], x.data_ptr(), dst.data_ptr(), n, None, 0,
                                                            ws.data_ptr(), ws.numel(), cfg, st)))
    elif prim == "scan_affine":
        a = 0.5 + 0.5 * rand_float(torch.float32)
        b = 2.0 * rand_float(torch.float32) - 1.0
        da, db = torch.empty_like(a), torch.empty_like(b)
        for (t, v) in SCAN_VARIANTS:
            cfg = ctypes.pointer(C.LaunchCfg(t, v, 0, 0))
            need = lib.kf_scan_workspace_bytes(C.F32, 1, n, cfg)
            if need == 0:
                continue
            ws = torch.empty(need, dtype=torch.uint8, device="cuda")
            jobs.append(("%dx%d" % (t, v), t, v, 0,
                         lambda cfg=cfg, ws=ws: lib.kf_scan_affine_soa(a.data_ptr(), b.data_ptr(), da.data_ptr(), db.data_ptr(), n,
                                                                       None, 0, ws.data_ptr(), ws.numel(), cfg, st)))
    else:
        pairs = prim == "sort_pairs"
        kw = width // 2 if pairs else width   # sort_pairs cells: 4+4 and 8+8 bytes
        keys = rand_bits(kw)
        kout = torch.empty_like(keys)
        vals = torch.arange(n, dtype=int_dt[kw], device="cuda") if pairs else None
        vout = torch.empty_like(vals) if pairs else None
        for (t, v) in SORT_VARIANTS:
            cfg = ctypes.pointer(C.LaunchCfg(t, v, 0, 0))
            need = lib.kf_sort_workspace_bytes(key_code[kw], kw if pairs else 0, n, cfg)
            if need == 0:
                continue
            ws = torch.empty(need, dtype=torch.uint8, device="cuda")
            if pairs:
                fn = lambda cfg=cfg, ws=ws: lib.kf_sort_pairs(key_code[kw], keys.data_ptr(), kout.data_ptr(), kw, vals.data_ptr(),
                                                              vout.data_ptr(), n, ws.data_ptr(), ws.numel(), cfg, st)
            else:
                fn = lambda cfg=cfg, ws=ws: lib.kf_sort_keys(key_code[kw], keys.data_ptr(), kout.data_ptr(), n, ws.data_ptr(),
                                                             ws.numel(), cfg, st)
            jobs.append(("%dx%d" % (t, v), t, v, 0, fn))

    best = {}
    for rnd in range(2):  # two interleaved rounds: a win has to show in both orders
        for label, t, v, per, fn in (jobs if rnd == 0 else reversed(jobs)):
            def call(fn=fn):
                rc = fn()
                if rc != 0:
                    raise RuntimeError("%s %s: kf_status %d" % (prim, label, rc))
            ms = time_call(torch, call)
            best[label] = min(best.get(label, float("inf")), ms)
    for label, t, v, per, _ in jobs:
        yield label, t, v, per, best[label]


def cmd_sweep(args):
    import torch
    kf = load_package()
    from kernelforge_jl_b200 import _cabi as C
    done = set()
    if os.path.exists(args.out):
        with open(args.out) as fh:
            for line in fh:
                r = json.loads(line)
                done.add((r["primitive"], r["elem_bytes"], r["log2n"]))
    todo = [c for c in cells(args) if c not in done]
    print("%d cells to measure (%d already in %s)" % (len(todo), len(done), args.out), flush=True)
    with open(args.out, "a") as fh:
        for prim, width, log2n in todo:
            try:
                rows = list(run_cell(kf, torch, C, prim, width, log2n))
            except torch.cuda.OutOfMemoryError:
                print("skip %s w=%d 2^%d: not enough device memory" % (prim, width, log2n), flush=True)
                torch.cuda.empty_cache()
                continue
            for label, t, v, per, ms in rows:
                fh.write(json.dumps({"primitive": prim, "elem_bytes": width, "log2n": log2n, "variant": label, "threads": t,
                                     "items": v, "blocks_per_sm": per, "ms": round(ms, 6)}) + "\n")
            fh.flush()
            b = min(rows, key=lambda r: r[4])
            print("%-12s w=%-2d n=2^%-2d best %-18s %.4f ms" % (prim, width, log2n, b[0], b[4]), flush=True)
            torch.cuda.empty_cache()
    return 0


# ---- choosing --------------------------------------------------------------------------------------
TABLE_PRIM = {"mapreduce": "mapreduce", "scan": "scan", "scan_affine": "scan", "sort_keys": "sort_keys", "sort_pairs": "sort_pairs"}


def table_lookup(rows, prim, eb, nbytes):
    for r in rows:
        if r["primitive"] != prim or (r["elem_bytes"] not in (0, eb)):
            continue
        if r["max_bytes"] is None or nbytes <= r["max_bytes"]:
            return r
    return None


def choose_rows(measurements, table_rows):
    """The chooser as a pure function: `measurements` are the sweep's records (dicts), `table_rows` the
    current table. Returns (new rows, report lines)."""
    meas = {}
    for r in measurements:
        meas.setdefault((r["primitive"], r["elem_bytes"]), {}).setdefault(r["log2n"], []).append(r)
    new_rows, report = [], []
    for (prim, eb), by_size in sorted(meas.items()):
        if prim == "scan_affine":
            continue  # the pair shares the 8-byte scan rows; it is listed in the report only
        tprim = TABLE_PRIM[prim]
        picks = []
        for log2n in sorted(by_size):
            cands = by_size[log2n]
            nbytes = (1 << log2n) * eb
            cur = table_lookup(table_rows, tprim, eb, nbytes)
            cur_m = [c for c in cands if cur and c["threads"] == cur["threads"] and c["items"] == cur["items"] and
                     (prim != "mapreduce" or c["blocks_per_sm"] == max(cur["blocks_per_sm"], 1))]
            best = min(cands, key=lambda c: c["ms"])
            keep = cur_m[0] if cur_m else best
            gain = keep["ms"] / best["ms"] - 1.0
            chosen = best if (not cur_m or gain > WIN) else keep
            picks.append((log2n, chosen, keep, best, gain))
            report.append((prim, eb, log2n, keep["variant"], keep["ms"], best["variant"], best["ms"], gain, chosen["variant"]))
        # merge neighbouring sizes with the same choice into regimes
        regimes = []
        for log2n, chosen, keep, best, gain in picks:
            key = (chosen["threads"], chosen["items"], chosen["blocks_per_sm"])
            if regimes and regimes[-1]["key"] == key:
                regimes[-1]["sizes"].append(log2n)
            else:
                regimes.append({"key": key, "sizes": [log2n]})
        for i, rg in enumerate(regimes):
            if i + 1 < len(regimes):  # geometric midpoint between the neighbouring measured sizes
                n1, n2 = 1 << rg["sizes"][-1], 1 << regimes[i + 1]["sizes"][0]
                max_bytes = int(math.sqrt(float(n1) * float(n2))) * eb
            else:
                max_bytes = None
            t, v, per = rg["key"]
            new_rows.append({"primitive": tprim, "elem_bytes": eb, "max_bytes": max_bytes, "threads": t, "items": v,
                             "blocks_per_sm": per,
                             "from": "sweep cells %s w=%d, log2 n = %s" % (prim, eb, ",".join(str(s) for s in rg["sizes"]))})
    return new_rows, report


def cmd_choose(args):
    with open(os.path.join(HERE, "launch_table.json")) as fh:
        table = json.load(fh)
    with open(args.inp) as fh:
        measurements = [json.loads(line) for line in fh if line.strip()]
    new_rows, report = choose_rows(measurements, table["rows"])
    print("| primitive | bytes | log2 n | table entry | ms | fastest | ms | gain of fastest | chosen |\n|---|---|---|---|---|---|---|---|---|")
    for r in report:
        print("| %s | %d | %d | %s | %.4f | %s | %.4f | %.1f %% | %s |" % (r[0], r[1], r[2], r[3], r[4], r[5], r[6], 100 * r[7], r[8]))
    if args.write:
        # catch-all rows (element sizes that were not swept) stay behind the measured ones
        tail = [r for r in table["rows"] if r["elem_bytes"] == 0 and r["max_bytes"] is None]
        table["rows"] = new_rows + tail
        with open(os.path.join(HERE, "launch_table.json"), "w") as fh:
            json.dump(table, fh, indent=1)
        spec = importlib.util.spec_from_file_location("gen_launch_table", os.path.join(HERE, "gen_launch_table.py"))
        gen = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(gen)
        gen.main()
    return 0


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("sweep")
    s.add_argument("--out", default=DEFAULT_OUT)
    s.add_argument("--log2n", default="16,18,20,22,24,26,28,30")
    s.add_argument("--only", default=None)
    c = sub.add_parser("choose")
    c.add_argument("--in", dest="inp", default=DEFAULT_OUT)
    c.add_argument("--write", action="store_true")
    args = ap.parse_args()
    return cmd_sweep(args) if args.cmd == "sweep" else cmd_choose(args)


if __name__ == "__main__":
    sys.exit(main())
