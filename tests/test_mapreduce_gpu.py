"""GPU parity tests of `mapreduce` against the CPU oracle, through the C ABI.

Mirrors test/tests/mapreduce/mapreduce1d_test.jl:7-56,218-224 and the dims=nothing cases of
test/tests/mapreduce/mapreduce_test.jl of KernelForge.jl. Tolerances: integers bit-exact; floats
rtol 1e-4 / atol 1e-5 on the reference's sum(1:n) cases, and 1e-5*log2(n) relative against the
Float64 oracle elsewhere.
"""
import math
import operator
import zlib

import numpy as np
import pytest
import torch

from util import pow2_factors, scan_tol, to_dev, to_host

pytestmark = pytest.mark.gpu

NP_OPS = {"+": 0, "*": 1, "min": 2, "max": 3, "&": 4, "|": 5, "xor": 6}


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.int32])
@pytest.mark.parametrize("n", [100_000, 10_001, 100, 33])
def test_sum_1_to_n(kf, dtype, n):
    """sum(1:n), allocating and in-place forms, fresh and reused tmp (flag reset between calls)."""
    src_h = np.arange(1, n + 1).astype(dtype)
    src = to_dev(src_h)
    ref = n * (n + 1) // 2
    if dtype == np.int32:
        ref = int(np.array([ref]).astype(np.int64).astype(np.int32)[0])  # Int32 `+` wraps
    tmp = kf.get_allocation(kf.MapReduce1D, kf.identity, operator.add, src)
    for trial in range(3):
        dst = torch.zeros(1, dtype=src.dtype, device="cuda")
        kf.mapreduce1d_(kf.identity, operator.add, dst, src, tmp=tmp)
        got_inplace = dst.cpu()[0].item()
        got = kf.mapreduce1d(kf.identity, operator.add, src, to_cpu=True)
        got_tmp = kf.mapreduce(kf.identity, operator.add, src, tmp=tmp)
        for g in (got_inplace, got, got_tmp):
            if dtype == np.int32:
                assert g == ref
            else:
                assert math.isclose(g, ref, rel_tol=1e-4, abs_tol=1e-5)


def test_config_abs2_sum_2p20(kf, oracle):
    """mapreduce(abs2, +, x), Float32 n=2^20, x ~ U[0,1) seed 0; 1e-5*log2(n) relative vs Float64."""
    n = 1 << 20
    x = np.random.default_rng(0).random(n, dtype=np.float32)
    ref = oracle.c_mapreduce(oracle.MAP_ABS2, oracle.OP_ADD, x)
    got = kf.mapreduce(kf.abs2, operator.add, to_dev(x))
    assert abs(got - ref) <= scan_tol(n) * abs(ref)


@pytest.mark.parametrize("dtype", [np.uint8, np.int8, np.int16, np.int32, np.uint32, np.int64, np.uint64])
@pytest.mark.parametrize("op", ["+", "*", "min", "max", "&", "|", "xor"])
def test_integer_ops_exact(kf, oracle, dtype, op):
    rng = np.random.default_rng(zlib.crc32((np.dtype(dtype).name + op).encode()))
    info = np.iinfo(dtype)
    for n in (1, 31, 1000, 100_003):
        x = rng.integers(info.min, info.max, size=n, dtype=dtype, endpoint=True)
        if op == "*":
            x = (x | 1).astype(dtype)  # odd factors keep the wrapped product away from 0
        ref = oracle.c_mapreduce(oracle.MAP_IDENTITY, NP_OPS[op], x)
        got = kf.mapreduce(kf.identity, op, to_dev(x))
        assert int(got) == int(ref), (n, got, ref)


@pytest.mark.parametrize("dtype", [np.uint8, np.int8])
def test_one_byte_sum_packed_path(kf, oracle, dtype):
    """One-byte `+` without a map sums whole strips with packed arithmetic (four bytes per dp4a, 32-bit
    running sums taken modulo 256 at the end): sizes around a strip, large inputs, saturated inputs,
    misaligned views, every launch variant; with a map the per-element code runs."""
    rng = np.random.default_rng(41)
    info = np.iinfo(dtype)
    for n in (1, 15, 16, 16_383, 16_384, 16_385, 1_000_003, 50_000_001):
        for x in (rng.integers(info.min, info.max, n, dtype=dtype, endpoint=True), np.full(n, info.max, dtype=dtype),
                  np.full(n, info.min, dtype=dtype)):
            want = int(oracle.c_mapreduce(oracle.MAP_IDENTITY, NP_OPS["+"], x))
            assert int(kf.mapreduce(kf.identity, "+", to_dev(x))) == want, n
    x = rng.integers(info.min, info.max, 3_000_017, dtype=dtype, endpoint=True)
    for off in (1, 7, 15):
        want = int(oracle.c_mapreduce(oracle.MAP_IDENTITY, NP_OPS["+"], x[off:]))
        assert int(kf.mapreduce(kf.identity, "+", to_dev(x)[off:])) == want
    for workgroup, nitem in ((256, 4), (512, 4), (256, 8)):
        for blocks in (1, 148, 1184):
            got = kf.mapreduce(kf.identity, "+", to_dev(x), workgroup=workgroup, Nitem=nitem, blocks=blocks)
            assert int(got) == int(oracle.c_mapreduce(oracle.MAP_IDENTITY, NP_OPS["+"], x))
    if dtype == np.int8:
        got = kf.mapreduce(kf.abs2, "+", to_dev(x))
        assert int(got) == int(oracle.c_mapreduce(oracle.MAP_ABS2, NP_OPS["+"], x))


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("f,op", [("identity", "+"), ("abs2", "+"), ("abs", "max"), ("identity", "min"),
                                  ("identity", "max"), ("identity", "*")])
def test_float_ops(kf, oracle, dtype, f, op):
    rng = np.random.default_rng(7)
    fcode = {"identity": 0, "abs2": 1, "abs": 2}[f]
    for n in (1, 5, 1000, 300_001):
        x = rng.standard_normal(n).astype(dtype)
        if op == "*":
            x = pow2_factors(n, rng, dtype)  # exact products: Float32 drifts by 1e-3 on near-1 factors
        ref = oracle.c_mapreduce(fcode, NP_OPS[op], x)
        got = kf.mapreduce(f, op, to_dev(x))
        if op in ("min", "max", "*"):
            assert got == ref
        else:
            scale = float(np.abs(x.astype(np.float64)).sum()) if op == "+" and f == "identity" else abs(ref)
            assert abs(got - ref) <= scan_tol(n) * max(scale, 1e-30)


def test_post_map_sqrt(kf, oracle):
    x = np.random.default_rng(3).random(12345, dtype=np.float32)
    ref = math.sqrt(oracle.c_mapreduce(oracle.MAP_ABS2, oracle.OP_ADD, x))
    got = kf.mapreduce(kf.abs2, operator.add, to_dev(x), g=math.sqrt)
    assert abs(got - ref) <= 1e-5 * 14 * ref


@pytest.mark.parametrize("workgroup,nitem", [(256, 4), (512, 4), (256, 8)])
@pytest.mark.parametrize("blocks", [None, 1, 7, 148, 1184])
def test_launch_overrides(kf, workgroup, nitem, blocks):
    n = 1_000_003
    x = np.random.default_rng(1).integers(0, 1 << 32, size=n, dtype=np.uint32)
    ref = int(x.sum(dtype=np.uint64) & 0xFFFFFFFF)
    got = kf.mapreduce(kf.identity, "+", to_dev(x), workgroup=workgroup, Nitem=nitem, blocks=blocks)
    assert int(got) == ref
    with pytest.raises(kf.ArgumentError):
        kf.mapreduce(kf.identity, "+", to_dev(x), workgroup=96, Nitem=3)


@pytest.mark.parametrize("dtype", [np.float64, np.uint8, np.int32])
@pytest.mark.parametrize("offset", [1, 2, 3, 5])
def test_views_unaligned(kf, oracle, dtype, offset):
    """view(x, 2:n)-style base pointers (test/tests/views/views_test.jl:14-23)."""
    n = 70_001
    x = (np.random.default_rng(offset).integers(0, 100, size=n)).astype(dtype)
    ref = oracle.c_mapreduce(0, 0, x)
    got = kf.mapreduce(kf.identity, "+", to_dev(x, offset=offset))
    assert got == ref


def test_errors(kf):
    x = torch.ones(100, dtype=torch.float32, device="cuda")
    small = kf.KernelBuffer(kf.MapReduce1D, torch.empty(16, dtype=torch.uint8, device="cuda"))
    with pytest.raises(kf.KernelForgeError):  # wrong-size tmp must throw
        kf.mapreduce(kf.identity, "+", x, tmp=small)
    with pytest.raises(kf.ArgumentError):  # empty reduction
        kf.mapreduce(kf.identity, "+", x[:0])
    with pytest.raises(kf.ArgumentError):  # unsupported closure: no fallback
        kf.mapreduce(lambda v: v + 1, "+", x)
    with pytest.raises(kf.ArgumentError):
        kf.mapreduce(kf.identity, lambda a, b: a - b, x)
    with pytest.raises(kf.ArgumentError):
        kf.mapreduce(kf.identity, "+", x, dims=1)
    with pytest.raises(kf.ArgumentError):
        kf.mapreduce(kf.identity, "+", x.cpu())
    assert kf.mapreduce(kf.identity, "+", x) == 100.0  # the context survives the rejected calls


def test_tuple_inputs_dot_family(kf, oracle):
    """The tuple form (test/tests/mapreduce/mapreduce1d_test.jl:106-194): dot product, weighted sum of
    squares, squared distance with g=sqrt, three arrays, a reused workspace; Float64 as there, plus
    Float32 and integers (bit-exact, wrapping)."""
    rng = np.random.default_rng(5)
    for dtype in (np.float64, np.float32):
        tol = 1e-12 if dtype == np.float64 else 2e-5
        for n in (1, 10_001, 50_000, 1_000_003):
            x, y, z = (rng.random(n).astype(dtype) for _ in range(3))
            dx, dy, dz = to_dev(x), to_dev(y), to_dev(z)
            cases = [(kf.prod, (dx, dy), oracle.np_mapreduce_multi(oracle.MAPN_PROD, 0, (x, y)), kf.identity),
                     (kf.wsq, (dx, dy), oracle.np_mapreduce_multi(oracle.MAPN_WSQ, 0, (x, y)), kf.identity),
                     (operator.mul, (dx, dy), oracle.np_mapreduce_multi(oracle.MAPN_PROD, 0, (x, y), True), kf.sqrt),
                     (kf.sqdiff, (dx, dy), oracle.np_mapreduce_multi(oracle.MAPN_SQDIFF, 0, (x, y), True), math.sqrt),
                     (kf.prod, (dx, dy, dz), oracle.np_mapreduce_multi(oracle.MAPN_PROD, 0, (x, y, z)), kf.identity)]
            for f, srcs, ref, g in cases:
                got = kf.mapreduce1d(f, "+", srcs, g=g)
                assert abs(got - ref) <= tol * max(1.0, math.log2(n + 1)) * abs(ref), (dtype, n, got, ref)
            assert kf.mapreduce(kf.prod, "max", (dx, dy)) == pytest.approx(float((x.astype(np.float64) * y).max()), rel=1e-6)
    # integers wrap in the element type
    for dtype in (np.int32, np.uint8, np.int64):
        info = np.iinfo(dtype)
        a = rng.integers(info.min, info.max, 300_007, dtype=dtype, endpoint=True)
        b = rng.integers(info.min, info.max, 300_007, dtype=dtype, endpoint=True)
        got = kf.mapreduce(kf.prod, "+", (to_dev(a), to_dev(b)), to_cpu=False)
        assert to_host(got)[0] == oracle.np_mapreduce_multi(oracle.MAPN_PROD, 0, (a, b))
    # views that do not share their 16-byte misalignment take the element-wise path
    x, y = rng.random(70_001), rng.random(70_003)
    got = kf.mapreduce(kf.prod, "+", (to_dev(x)[1:], to_dev(y)[3:]))
    assert got == pytest.approx(float((x[1:] * y[3:]).sum()), rel=1e-12)
    got = kf.mapreduce(kf.prod, "+", (to_dev(x)[1:], to_dev(y)[1:70_001]))  # same misalignment: vector path with a head
    assert got == pytest.approx(float((x[1:] * y[1:70_001]).sum()), rel=1e-12)
    # in place with a pre-allocated tmp, reused across trials (:160-178)
    n = 50_000
    dst = torch.zeros(1, dtype=torch.float64, device="cuda")
    dx, dy = to_dev(rng.random(n)), to_dev(rng.random(n))
    tmp = kf.get_allocation(kf.MapReduce1D, kf.prod, "+", (dx, dy))
    for trial in range(5):
        x, y = rng.random(n), rng.random(n)
        dx.copy_(to_dev(x)); dy.copy_(to_dev(y))
        kf.mapreduce1d_(kf.prod, "+", dst, (dx, dy), tmp=tmp)
        assert to_host(dst)[0] == pytest.approx(float((x * y).sum()), rel=1e-12)
    with pytest.raises(kf.ArgumentError):
        kf.mapreduce(lambda a, b: a + b, "+", (dx, dy))
    with pytest.raises(kf.ArgumentError):
        kf.mapreduce(kf.prod, "+", (dx, dy[:10]))
    with pytest.raises(kf.ArgumentError):
        kf.mapreduce(kf.sqdiff, "+", (dx, dy, dx))


def test_full_size_2p28(kf):
    """n = 2^28: UInt32 wrapping sum bit-exact and Float32 sum within tolerance, checked against
    torch reductions in wider types on the same device data."""
    n = 1 << 28
    g = torch.Generator(device="cuda").manual_seed(0)
    xi = torch.randint(0, 256, (n,), dtype=torch.int32, device="cuda", generator=g)
    ref = int(xi.sum(dtype=torch.int64).item()) & 0xFFFFFFFF
    got = kf.mapreduce(kf.identity, "+", xi.view(torch.uint32))
    assert int(got) == ref
    xf = torch.rand(n, dtype=torch.float32, device="cuda", generator=g)
    reff = xf.sum(dtype=torch.float64).item()
    gotf = kf.mapreduce(kf.identity, "+", xf)
    assert abs(gotf - reff) <= scan_tol(n) * reff
    # determinism: same input, same launch -> same bits
    assert kf.mapreduce(kf.identity, "+", xf) == gotf
