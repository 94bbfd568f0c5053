"""Sweeps every compiled launch variant of the three primitives on the current GPU and prints a
table (GB/s of algorithmic bytes, CUDA-event timed, inputs larger than L2). The launch table
(tuning/launch_table.json) is edited from this output: a row is only changed when a variant beats
the current default by more than 6 % in a repeated run, the rule the reference's autotuner uses
(data/tuning/sort/autotune.jl:143-147,236-253).

    python kernelforge.jl_b200/tuning/sweep.py [scan] [sort] [mapreduce] [--log2n 28]
"""
import ctypes
import importlib.util
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
PKG_DIR = os.path.dirname(HERE)


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


def timeit(fn, iters=10, warm=3):
    for _ in range(warm):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def main():
    kf = load_package()
    from kernelforge_jl_b200 import _cabi as C
    lib = kf.lib
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    what = args or ["scan", "sort", "mapreduce"]
    log2n = int(sys.argv[sys.argv.index("--log2n") + 1]) if "--log2n" in sys.argv else 28
    n = 1 << log2n
    g = torch.Generator(device="cuda").manual_seed(0)
    st = torch.cuda.current_stream().cuda_stream
    xf = torch.rand(n, dtype=torch.float32, device="cuda", generator=g)
    out = torch.empty_like(xf)
    ms = timeit(lambda: out.copy_(xf))
    print("| primitive | variant | ms | GB/s |\n|---|---|---|---|")
    print("| copy (torch, yardstick) | - | %.3f | %.0f |" % (ms, 8 * n / ms / 1e6))
    if "scan" in what:
        ws = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
        for (t, v) in [(256, 4), (512, 4), (256, 8), (128, 8), (768, 4), (384, 8), (512, 8)]:
            cfg = ctypes.pointer(C.LaunchCfg(t, v, 0, 0))

            def f():
                rc = lib.kf_scan(0, 0, 0, C.F32, xf.data_ptr(), out.data_ptr(), n, None, 0, ws.data_ptr(), ws.numel(), cfg, st)
                assert rc == 0, rc
            ms = timeit(f)
            kind = "persistent" if (t, v) in ((768, 4), (384, 8), (512, 8)) else "direct"
            print("| scan f32 + | %s %dx%d | %.3f | %.0f |" % (kind, t, v, ms, 8 * n / ms / 1e6), flush=True)
        assert lib.kf_check(ws.data_ptr(), st) == 0
    if "sort" in what:
        keys = torch.randint(0, 1 << 32, (n,), dtype=torch.int64, device="cuda", generator=g).to(torch.int32)
        dst = torch.empty_like(keys)
        for (t, v) in [(256, 16), (512, 16), (512, 24), (384, 24)]:
            cfg = ctypes.pointer(C.LaunchCfg(t, v, 0, 0))
            ws = torch.empty(lib.kf_sort_workspace_bytes(C.U32, 0, n, cfg), dtype=torch.uint8, device="cuda")

            def f():
                rc = lib.kf_sort_keys(C.U32, keys.data_ptr(), dst.data_ptr(), n, ws.data_ptr(), ws.numel(), cfg, st)
                assert rc == 0, rc
            ms = timeit(f, iters=5, warm=2)
            print("| sort u32 keys | %dx%d | %.3f | %.0f |" % (t, v, ms, 36 * n / ms / 1e6), flush=True)
            assert lib.kf_check(ws.data_ptr(), st) == 0
            del ws
    if "mapreduce" in what:
        ws = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
        d1 = torch.empty(1, dtype=torch.float32, device="cuda")
        for (t, v) in [(256, 4), (512, 4), (256, 8)]:
            for per_sm in (2, 4, 8, 16):
                cfg = ctypes.pointer(C.LaunchCfg(t, v, lib.kf_num_sms() * per_sm, 0))

                def f():
                    rc = lib.kf_mapreduce(0, 0, 0, C.F32, xf.data_ptr(), n, d1.data_ptr(), ws.data_ptr(), ws.numel(), cfg, st)
                    assert rc == 0, rc
                ms = timeit(f, iters=20)
                print("| mapreduce f32 + | %dx%d, %d CTAs/SM | %.4f | %.0f |" % (t, v, per_sm, ms, 4 * n / ms / 1e6), flush=True)
        small = xf[: 1 << 20]

        def f():
            rc = lib.kf_mapreduce(1, 0, 0, C.F32, small.data_ptr(), 1 << 20, d1.data_ptr(), ws.data_ptr(), ws.numel(), None, st)
            assert rc == 0, rc
        ms = timeit(f, iters=500, warm=20)
        print("| mapreduce abs2 n=2^20 (C ABI call, memset + kernel) | table | %.4f | %.0f |" % (ms, 4 * (1 << 20) / ms / 1e6))


if __name__ == "__main__":
    main()
