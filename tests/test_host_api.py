"""CPU tests of the host layer that mirrors the Julia API: closure -> enum mapping, argument
checks and error behaviour. Nothing here computes: tensors on the CPU are rejected (there is no CPU
path), exactly like a non-device array would be in the reference."""
import math
import operator

import numpy as np
import pytest
import torch


def test_closure_mapping(kf):
    from kernelforge_jl_b200 import _cabi as C, ops
    assert ops.map_code(kf.identity) == C.MAP_IDENTITY and ops.map_code(kf.abs2) == C.MAP_ABS2
    assert ops.map_code(abs) == C.MAP_ABS and ops.map_code("abs2") == C.MAP_ABS2
    assert ops.op_code(operator.add) == C.OP_ADD and ops.op_code("+") == C.OP_ADD
    assert ops.op_code(min) == C.OP_MIN and ops.op_code(max) == C.OP_MAX and ops.op_code(operator.mul) == C.OP_MUL
    assert ops.op_code(operator.and_) == C.OP_AND and ops.op_code(operator.or_) == C.OP_OR
    assert ops.op_code(operator.xor) == C.OP_XOR and ops.op_code("⊻") == C.OP_XOR
    assert ops.op_code(kf.AffineCompose()) == C.OP_AFFINE and kf.AffineCompose() is kf.AffineCompose()
    assert ops.post_code(math.sqrt) == C.POST_SQRT and ops.post_code(kf.identity) == C.POST_IDENTITY
    for bad in (lambda x: x + 1, print, 3):
        with pytest.raises(kf.ArgumentError):
            ops.map_code(bad)
        with pytest.raises(kf.ArgumentError):
            ops.op_code(bad)
    # the operator itself, on the host: (a1,b1) o (a2,b2) = (a1*a2, a2*b1 + b2)
    assert kf.AffineCompose()((2.0, 1.0), (0.5, -1.0)) == (1.0, -0.5)


def test_no_cpu_path(kf):
    x = torch.ones(16)
    for call in (lambda: kf.mapreduce(kf.identity, "+", x), lambda: kf.scan("+", x), lambda: kf.sort(x),
                 lambda: kf.get_allocation(kf.Scan1D, kf.identity, "+", x)):
        with pytest.raises(kf.ArgumentError):
            call()


def test_argument_checks_that_need_no_device(kf):
    x = torch.ones(16)
    with pytest.raises(kf.ArgumentError):
        kf.mapreduce(kf.identity, "+", x, dims=1)
    with pytest.raises(kf.ArgumentError):
        kf.mapreduce(kf.identity, "+", (x, x))
    with pytest.raises(kf.ArgumentError):
        kf.sort(x, rev=True)
    with pytest.raises(kf.ArgumentError):
        kf.sort(x, by=lambda v: -v)
    with pytest.raises(kf.ArgumentError):
        kf.scan("+", x, g=math.sqrt)
    with pytest.raises(TypeError):
        kf.scan_("+", x)
    with pytest.raises(kf.KernelForgeError):
        kf.get_allocation(object, x)


def test_names_follow_the_reference(kf):
    for name in ("mapreduce", "mapreduce_", "mapreduce1d", "mapreduce1d_", "scan", "scan_", "sort", "sort_",
                 "sortperm", "get_allocation", "KernelBuffer", "MapReduce1D", "Scan1D", "Sort1D", "AffineCompose"):
        assert hasattr(kf, name)


def _load_autotune():
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("kf_autotune", os.path.join(root, "kernelforge.jl_b200", "tuning", "autotune.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_launch_table_chooser_rules():
    """The rules the reference's autotuners use (data/tuning/sort/autotune.jl:143-147,236-253 and
    data/tuning/mapreduce1d/autotune.jl:162-214): the current entry is a candidate, it is replaced only
    by a win of more than 6 %, and regime boundaries lie at geometric midpoints of measured sizes."""
    at = _load_autotune()
    table = [{"primitive": "sort_keys", "elem_bytes": 0, "max_bytes": None, "threads": 512, "items": 16, "blocks_per_sm": 0}]

    def rec(log2n, variant, t, v, ms):
        return {"primitive": "sort_keys", "elem_bytes": 4, "log2n": log2n, "variant": variant, "threads": t, "items": v,
                "blocks_per_sm": 0, "ms": ms}
    meas = [rec(16, "512x16", 512, 16, 1.00), rec(16, "256x16", 256, 16, 0.80),   # 25 % faster: replaces the entry
            rec(18, "512x16", 512, 16, 1.00), rec(18, "256x16", 256, 16, 0.96),   # 4 % faster: the entry stays
            rec(20, "512x16", 512, 16, 1.00), rec(20, "512x24", 512, 24, 0.70)]
    rows, report = at.choose_rows(meas, table)
    assert [(r["threads"], r["items"]) for r in rows] == [(256, 16), (512, 16), (512, 24)]
    assert rows[0]["max_bytes"] == int((2 ** 16 * 2 ** 18) ** 0.5) * 4   # geometric midpoint of 2^16 and 2^18 elements
    assert rows[1]["max_bytes"] == int((2 ** 18 * 2 ** 20) ** 0.5) * 4 and rows[2]["max_bytes"] is None
    assert all("log2 n" in r["from"] for r in rows)
    assert [round(100 * r[7]) for r in report] == [25, 4, 43]


def test_committed_launch_table_matches_the_header_and_the_sweep():
    """launch_table.json and the generated header agree, and every measured row cites sweep cells that
    exist in the committed measurements."""
    import json
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    tdir = os.path.join(root, "kernelforge.jl_b200", "tuning")
    table = json.load(open(os.path.join(tdir, "launch_table.json")))
    header = open(os.path.join(root, "kernelforge.jl_b200", "csrc", "launch_table.h")).read()
    assert "kNumLaunchRows = %d" % len(table["rows"]) in header
    cells = set()
    for line in open(os.path.join(tdir, "sweep_b200.jsonl")):
        r = json.loads(line)
        cells.add((r["primitive"], r["elem_bytes"], r["log2n"]))
    cited = 0
    for row in table["rows"]:
        m = re.match(r"sweep cells (\w+) w=(\d+), log2 n = ([\d,]+)", row.get("from", ""))
        if not m:
            assert row["elem_bytes"] == 0  # only the catch-all rows are not measured
            continue
        for l in m.group(3).split(","):
            assert (m.group(1), int(m.group(2)), int(l)) in cells
            cited += 1
    assert cited >= 100


def test_packed_byte_prefix_arithmetic_of_the_scan_kernel():
    """The one-byte `+` scan keeps four elements per register. This restates `byte_prefix16` of
    csrc/scan_impl.cuh with Python integers (PRMT selectors included) and checks it against a plain
    wrap-around cumulative sum: even and odd bytes travel as two 16-bit lanes per word, so no carry crosses
    a lane, for every carried-in byte and for saturated inputs."""
    mask = 0xFFFFFFFF

    def byte_perm(a, b, sel):  # PRMT: result byte i = byte (sel nibble i) of the 8 bytes {a, b}
        src = [(a >> (8 * i)) & 255 for i in range(4)] + [(b >> (8 * i)) & 255 for i in range(4)]
        return sum(src[(sel >> (4 * i)) & 7] << (8 * i) for i in range(4))

    def byte_prefix16(words, carry_in):
        carry = carry_in | (carry_in << 16)
        out = []
        for w in words:
            lo, hi = byte_perm(w, 0, 0x4240), byte_perm(w, 0, 0x4341)
            s_lo = (lo * 0x00010001 + carry) & mask
            even, odd = ((hi << 16) + s_lo) & mask, (hi * 0x00010001 + s_lo) & mask
            out.append(byte_perm(even, odd, 0x6240))
            carry = byte_perm(odd, 0, 0x4242)
        return out

    rng = np.random.default_rng(5)
    cases = [np.full(16, 255, np.uint8), np.zeros(16, np.uint8), np.arange(16, dtype=np.uint8) * 17]
    cases += [rng.integers(0, 256, 16).astype(np.uint8) for _ in range(500)]
    for x in cases:
        for b in (0, 1, 128, 255, int(rng.integers(0, 256))):
            got = np.array(byte_prefix16([int(v) for v in x.view(np.uint32)], b), dtype=np.uint32).view(np.uint8)
            want = (np.cumsum(x.astype(np.int64)) + b).astype(np.uint8)
            assert (got == want).all()


def test_quaternion_operator_on_the_host(kf):
    """`QuaternionMul()` is a singleton whose host-side call is the Hamilton product (i*j = k, j*i = -k);
    like every operator of this layer it has no CPU execution path for arrays, and it is a scan operator
    only."""
    q = kf.QuaternionMul()
    assert q is kf.QuaternionMul() and repr(q) == "QuaternionMul()"
    one, i, j, k = (1, 0, 0, 0), (0, 1, 0, 0), (0, 0, 1, 0), (0, 0, 0, 1)
    neg = lambda t: tuple(-v for v in t)
    assert q(i, j) == k and q(j, i) == neg(k) and q(j, k) == i and q(k, i) == j
    assert q(i, i) == neg(one) and q(q(i, j), k) == neg(one) and q(one, k) == k
    assert q((1, 2, 3, 4), (5, 6, 7, 8)) == (-60, 12, 30, 24)
    with pytest.raises(kf.ArgumentError):
        kf.scan(q, torch.zeros(8, 4))  # a CPU tensor: there is no CPU path
    with pytest.raises(kf.ArgumentError):
        kf.mapreduce(kf.identity, q, torch.zeros(8, 4))
