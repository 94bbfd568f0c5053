"""CPU tests of bench.py's host-side pieces: the JSON contract keys both arms share, and the CSV rows in
the reference's benchmark schema. Nothing here needs a GPU or launches a kernel."""
import csv
import importlib.util
import io
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("kf_bench", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_both_arms_share_metric_and_config():
    b = _bench()
    assert isinstance(b.METRIC, str) and "2^28" in b.METRIC
    for world in (1, 2, 8):
        cfg = b.workload_config(world)
        assert cfg["n_per_gpu"] == 1 << 28 and cfg["algorithmic_bytes_per_step"] == world * 2 * 8 * (1 << 28)
        assert b.workload_config(world) == cfg  # the two arms call the same function


def test_primitives_csv_rows_follow_the_reference_schema():
    """Columns of perfs/julia/bench_utils.jl:7-22 of KernelForge.jl first, the added ones after them."""
    b = _bench()
    assert b.CSV_COLUMNS[:7] == ["n", "type", "method", "mean_kernel_us", "std_kernel_us", "mean_total_us", "std_total_us"]
    prim = {"sort_u32_keys_2p28": {"ms": 4.2, "GB/s": 2300.0, "algorithmic_bytes": 36 << 28},
            "scan_affine_f32x2_2p26": {"ms": 0.2, "GB/s": 5400.0, "algorithmic_bytes": 16 << 26},
            "sharded_mapreduce_f32_sum_2p28_per_gpu": {"ms": 0.18, "GB/s": 48000.0}}
    rows = b.primitives_csv_rows(prim, 8, 6540.8)
    assert [r["n"] for r in rows] == [1 << 28, 1 << 26, 1 << 28]
    assert [r["type"] for r in rows] == ["u32", "f32x2", "f32"]
    assert rows[0]["mean_total_us"] == 4200.0 and rows[0]["gpus"] == 8
    assert abs(rows[2]["pct_roofline"] - 100.0 * 48000.0 / (6540.8 * 8)) < 0.01
    out = io.StringIO()
    w = csv.DictWriter(out, fieldnames=b.CSV_COLUMNS)
    w.writeheader()
    w.writerows(rows)
    assert out.getvalue().splitlines()[0] == ",".join(b.CSV_COLUMNS)
