"""GPU parity tests of `scan` / `scan!` against the CPU oracle, through the C ABI.

Mirrors test/tests/scan/scan_test.jl of KernelForge.jl (sizes and types :35-65, UInt8 wrap :67-86,
n=1..10 :88-102, reused tmp :107-125, non-commutative operator :22-33) and the unaligned views of
test/tests/views/views_test.jl. Tolerances: integers bit-exact; floats 1e-5*log2(n) relative to
the Float64 left fold (for `+`, relative to the running sum of |x|, which equals the fold for
non-negative data).
"""
import numpy as np
import pytest
import torch

from util import assert_close_rel, pow2_factors, scan_tol, to_dev, to_host

pytestmark = pytest.mark.gpu

OPC = {"+": 0, "*": 1, "min": 2, "max": 3, "&": 4, "|": 5, "xor": 6}


def _check_scan(kf, oracle, x, op, **kw):
    ref = oracle.c_scan(0, OPC[op], x)
    dst = kf.scan(op, to_dev(x), **kw)
    got = to_host(dst)
    if x.dtype.kind == "f":
        if op == "+":
            floor = np.cumsum(np.abs(x.astype(np.float64)))
            err = np.abs(got.astype(np.float64) - ref)
            assert (err <= scan_tol(x.size) * np.maximum(floor, 1e-300)).all(), float((err / floor).max())
        elif op in ("min", "max", "*"):  # `*` is tested on exact power-of-two factors
            assert (got.astype(np.float64) == ref).all()
        else:
            assert_close_rel(got, ref, x.size)
    else:
        assert (got == ref).all()


@pytest.mark.parametrize("dtype", [np.float64, np.int32])
@pytest.mark.parametrize("op", ["+", "min"])
@pytest.mark.parametrize("n", [1, 5, 10, 100, 1000, 1_000_000])
def test_sizes_types_ops(kf, oracle, dtype, op, n):
    rng = np.random.default_rng(n)
    x = rng.random(n).astype(dtype) if dtype == np.float64 else rng.integers(-1000, 1000, n).astype(dtype)
    _check_scan(kf, oracle, x, op)


@pytest.mark.parametrize("n", list(range(1, 11)))
def test_edge_sizes_f64(kf, oracle, n):
    _check_scan(kf, oracle, np.random.default_rng(n).random(n), "+")


@pytest.mark.parametrize("op", ["+", "max", "min"])
def test_uint8_wrapping(kf, oracle, op):
    for trial in range(5):
        x = np.random.default_rng(trial).integers(0, 256, 10_001).astype(np.uint8)
        _check_scan(kf, oracle, x, op)


@pytest.mark.parametrize("dtype", [np.uint8, np.int8, np.int16, np.uint32, np.int64, np.uint64, np.float32])
@pytest.mark.parametrize("op", ["+", "*", "max", "&", "|", "xor"])
def test_dtype_op_matrix(kf, oracle, dtype, op):
    if np.dtype(dtype).kind == "f" and op in ("&", "|", "xor"):
        with pytest.raises(kf.ArgumentError):
            kf.scan(op, torch.ones(8, dtype=torch.float32, device="cuda"))
        return
    rng = np.random.default_rng(11)
    n = 70_003
    if np.dtype(dtype).kind == "f":
        x = pow2_factors(n, rng, dtype) if op == "*" else rng.random(n).astype(dtype)
    else:
        info = np.iinfo(dtype)
        x = rng.integers(info.min, info.max, size=n, dtype=dtype, endpoint=True)
    _check_scan(kf, oracle, x, op)


def test_float32_mul_long(kf, oracle):
    n = 1_000_000
    x = pow2_factors(n, np.random.default_rng(5), np.float32)
    _check_scan(kf, oracle, x, "*")
    x = np.random.default_rng(6).random(100_000).astype(np.float32) + 0.5  # generic factors: tolerance
    got = to_host(kf.scan("*", to_dev(x[:500])))
    ref = oracle.c_scan(0, 1, x[:500])
    assert (np.abs(got - ref) <= 1e-4 * np.abs(ref)).all()


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32, np.float64])
@pytest.mark.parametrize("n", [1000, 100_000, 1_000_000])
def test_reused_tmp(kf, oracle, dtype, n):
    """Same tmp, different data each call: a stale descriptor would leak into the next call."""
    src = torch.zeros(n, dtype=getattr(torch, np.dtype(dtype).name), device="cuda")
    dst = torch.zeros_like(src)
    tmp = kf.get_allocation(kf.Scan1D, kf.identity, "+", src)
    for call in range(6):
        h = np.random.default_rng(call).integers(-4, 5, n).astype(dtype)
        src.copy_(torch.from_numpy(h))
        kf.scan_("+", dst, src, tmp=tmp)
        assert (to_host(dst) == np.cumsum(h, dtype=dtype)).all()  # small integers: exact in every type


@pytest.mark.parametrize("workgroup,nitem", [(256, 4), (512, 4), (256, 8), (128, 8), (768, 4), (384, 8), (512, 8)])
def test_launch_variants(kf, oracle, workgroup, nitem):
    """Every compiled variant: the direct kernels and the persistent kernels (768x4, 384x8, 512x8)."""
    x = np.random.default_rng(2).integers(0, 256, 3_000_017).astype(np.uint32)
    _check_scan(kf, oracle, x, "+", workgroup=workgroup, Nitem=nitem)
    for dt in (np.uint8, np.float64):
        y = np.random.default_rng(3).integers(0, 100, 1_500_011).astype(dt)
        _check_scan(kf, oracle, y, "max" if dt == np.uint8 else "+", workgroup=workgroup, Nitem=nitem)
    a, b = _affine_inputs(700_001, 5)
    ra, rb = oracle.c_scan_affine(a, b)
    da, db = kf.scan(kf.AffineCompose(), (to_dev(a), to_dev(b)), workgroup=workgroup, Nitem=nitem)
    _check_affine(a.size, to_host(da), to_host(db), ra, rb)
    ab = np.stack([a, b], axis=1).copy()
    out = to_host(kf.scan(kf.AffineCompose(), to_dev(ab.reshape(-1)).view(a.size, 2), workgroup=workgroup, Nitem=nitem))
    _check_affine(a.size, out[:, 0], out[:, 1], ra, rb)
    with pytest.raises(kf.ArgumentError):
        kf.scan("+", to_dev(x), workgroup=96, Nitem=3)


@pytest.mark.parametrize("dtype", [np.float64, np.uint8, np.uint32])
@pytest.mark.parametrize("off_src,off_dst", [(1, 1), (3, 3), (1, 2), (0, 3), (5, 0)])
def test_views_unaligned(kf, oracle, dtype, off_src, off_dst):
    n = 40_003
    x = np.random.default_rng(off_src * 7 + off_dst).integers(0, 200, n).astype(dtype)
    src = to_dev(x, offset=off_src)
    dst = to_dev(np.zeros(n, dtype=dtype), offset=off_dst)
    kf.scan_("+", dst, src)
    ref = oracle.c_scan(0, 0, x)
    assert (to_host(dst).astype(np.float64) == ref.astype(np.float64)).all()


def test_in_place_and_init(kf, oracle):
    n = 500_001
    x = np.random.default_rng(9).integers(0, 1 << 32, n, dtype=np.uint32)
    t = to_dev(x)
    kf.scan_("+", t, t)
    assert (to_host(t) == np.cumsum(x, dtype=np.uint32)).all()
    init = to_dev(np.array([12345], dtype=np.uint32))
    got = to_host(kf.scan("+", to_dev(x), init=init))
    assert (got == (np.cumsum(x, dtype=np.uint32) + np.uint32(12345))).all()
    assert kf.scan("+", to_dev(x)[:0]).numel() == 0  # n == 0 is a no-op


def test_map_before_scan(kf, oracle):
    x = np.random.default_rng(4).integers(-50, 50, 30_001).astype(np.int32)
    got = to_host(kf.scan(kf.abs2, "+", to_dev(x)))
    assert (got == oracle.c_scan(oracle.MAP_ABS2, 0, x)).all()
    got = to_host(kf.scan(abs, "max", to_dev(x)))
    assert (got == oracle.c_scan(oracle.MAP_ABS, 3, x)).all()


def _affine_inputs(n, seed):
    rng = np.random.default_rng(seed)
    a = (0.5 + 0.5 * rng.random(n)).astype(np.float32)
    b = (2.0 * rng.random(n) - 1.0).astype(np.float32)
    return a, b


def _check_affine(n, ga, gb, ra, rb):
    """|got - ref| <= tol * max(|ref|, s): s = 1 for the offsets b (a stationary process that
    crosses zero), s = 4*FLT_MIN for the gains a (which decay through the subnormals to 0)."""
    assert_close_rel(gb, rb, n, floor=1.0)
    assert_close_rel(ga, ra, n, floor=4 * float(np.finfo(np.float32).tiny))


@pytest.mark.parametrize("n", [1, 2, 5, 1000, 100_003, 2_000_000])
def test_affine_soa_and_aos(kf, oracle, n):
    """Non-commutative operator: composition of affine maps, both layouts, vs the Float64 left fold."""
    a, b = _affine_inputs(n, n)
    ra, rb = oracle.c_scan_affine(a, b)
    op = kf.AffineCompose()
    da, db = kf.scan(op, (to_dev(a), to_dev(b)))
    _check_affine(n, to_host(da), to_host(db), ra, rb)
    ab = np.stack([a, b], axis=1).copy()
    out = to_host(kf.scan(op, to_dev(ab.reshape(-1)).view(n, 2)))
    _check_affine(n, out[:, 0], out[:, 1], ra, rb)


def test_affine_order_matters(kf, oracle):
    """Exact small-integer maps: any swap of operands would change the result."""
    n = 4099
    rng = np.random.default_rng(1)
    a = rng.integers(1, 3, n).astype(np.float32)
    a[10:] = 1.0  # gains <= 2^10 and offsets below 2^24: every intermediate is an exact Float32 integer
    b = rng.integers(-3, 4, n).astype(np.float32)
    ra, rb = oracle.c_scan_affine(a, b)
    da, db = kf.scan(kf.AffineCompose(), (to_dev(a), to_dev(b)))
    assert (to_host(da).astype(np.float64) == ra).all()
    assert (to_host(db).astype(np.float64) == rb).all()


def test_affine_init_and_views(kf, oracle):
    n = 50_001
    a, b = _affine_inputs(n, 3)
    init = np.array([0.75, -0.5], dtype=np.float32)
    ra, rb = oracle.c_scan_affine(a, b, init=init.astype(np.float64))
    da, db = kf.scan(kf.AffineCompose(), (to_dev(a, offset=1), to_dev(b, offset=1)), init=to_dev(init))
    _check_affine(n, to_host(da), to_host(db), ra, rb)
    # different misalignment of the four arrays -> element-wise path
    oa = to_dev(np.zeros(n, np.float32), offset=2)
    ob = to_dev(np.zeros(n, np.float32), offset=3)
    kf.scan_(kf.AffineCompose(), (oa, ob), (to_dev(a), to_dev(b, offset=1)))
    ra, rb = oracle.c_scan_affine(a, b)
    _check_affine(n, to_host(oa), to_host(ob), ra, rb)


@pytest.mark.parametrize("workgroup,nitem", [(768, 4), (384, 8), (512, 8)])
@pytest.mark.parametrize("dtype", [np.uint8, np.int8])
def test_one_byte_add_packed_path(kf, oracle, dtype, workgroup, nitem):
    """One-byte `+` with no maps runs a packed instantiation of the persistent kernel (four elements per
    register): sizes around its tile (threads x vectors x 16 bytes), a ragged last tile, a misaligned
    view (short head tile), in place, a left seed, saturated inputs (every carry between the packed
    lanes), and the mapped form, which keeps the per-element code."""
    tile = workgroup * nitem * 16
    rng = np.random.default_rng(tile)
    info = np.iinfo(dtype)
    for n in (tile - 1, tile, tile + 1, 2 * tile + 17, 40 * tile + 12_345):
        for x in (rng.integers(info.min, info.max, n, dtype=dtype, endpoint=True), np.full(n, info.max, dtype=dtype),
                  np.full(n, info.min, dtype=dtype)):
            _check_scan(kf, oracle, x, "+", workgroup=workgroup, Nitem=nitem)
    n = 9 * tile + 4321
    x = rng.integers(info.min, info.max, n + 16, dtype=dtype, endpoint=True)
    for off in (1, 5, 15):
        src = to_dev(x)[off:off + n]
        dst = torch.zeros(n + 32, dtype=src.dtype, device="cuda")
        kf.scan_("+", dst[off:off + n], src, workgroup=workgroup, Nitem=nitem)
        got = to_host(dst)
        assert (got[off:off + n] == oracle.c_scan(0, OPC["+"], x[off:off + n])).all()
        assert not got[:off].any() and not got[off + n:].any()
    buf = to_dev(x[:n])
    kf.scan_("+", buf, buf, workgroup=workgroup, Nitem=nitem)  # in place
    assert (to_host(buf) == oracle.c_scan(0, OPC["+"], x[:n])).all()
    seed = np.array([info.max, 3], dtype=dtype)
    got = to_host(kf.scan("+", to_dev(x[:n]), init=to_dev(seed), workgroup=workgroup, Nitem=nitem))
    want = (np.cumsum(x[:n].astype(np.int64)) + int(seed.astype(np.int64).sum())).astype(dtype)
    assert (got == want).all()
    if dtype == np.int8:
        got = to_host(kf.scan(kf.abs2, "+", to_dev(x[:n]), workgroup=workgroup, Nitem=nitem))
        assert (got == oracle.c_scan(oracle.MAP_ABS2, OPC["+"], x[:n])).all()


def _unit_quaternions(n, seed, dtype):
    x = np.random.default_rng(seed).standard_normal((n, 4))
    return (x / np.linalg.norm(x, axis=1, keepdims=True)).astype(dtype)


@pytest.mark.parametrize("dtype,tol", [(np.float64, 1e-10), (np.float32, 2e-3)])
@pytest.mark.parametrize("n", [1, 5, 100, 1023, 1024, 1025, 100_003, 1_000_000])
def test_quaternion_product_scan(kf, oracle, dtype, tol, n):
    """The reference's non-commutative scan case (test/tests/scan/scan_test.jl:22-33: `*` over random
    unit QuaternionF64, n = 10^6, against accumulate(*, src) on the host), for both component widths
    and around the 1024-quaternion tile. Unit quaternions keep every prefix on the unit sphere, so an
    absolute tolerance is meaningful; the Float32 bound is sqrt(n) roundings with room to spare."""
    q = _unit_quaternions(n, n, dtype)
    want = oracle.c_scan_quat(q)
    got = to_host(kf.scan(kf.QuaternionMul(), to_dev(q.reshape(-1)).view(n, 4)))
    assert got.dtype == dtype and got.shape == (n, 4)
    assert np.abs(got.astype(np.float64) - want).max() <= tol
    assert abs(np.linalg.norm(got[-1].astype(np.float64)) - 1.0) <= tol


def test_quaternion_order_matters_and_is_exact_on_the_unit_group(kf, oracle):
    """Products of +-1, +-i, +-j, +-k are exact in any precision and any association, so the scan must
    equal the left fold bit for bit, and any swapped pair of operands would show (i*j = k, j*i = -k)."""
    n = 300_007
    rng = np.random.default_rng(12)
    units = np.concatenate([np.eye(4), -np.eye(4)])
    for dtype in (np.float32, np.float64):
        q = units[rng.integers(0, 8, n)].astype(dtype)
        got = to_host(kf.scan(kf.QuaternionMul(), to_dev(q.reshape(-1)).view(n, 4)))
        assert (got.astype(np.float64) == oracle.c_scan_quat(q)).all()
        # swapping the operands of one product flips the sign of every later prefix whenever the two
        # factors anticommute, which half of all pairs of this group do
        swapped = oracle.c_scan_quat(np.concatenate([q[1:2], q[0:1], q[2:]]))
        pair = oracle.c_scan_quat(q[:2])[1], swapped[1]
        assert (pair[0] == pair[1]).all() or (got[-1].astype(np.float64) == -swapped[-1]).all()


def test_quaternion_init_views_and_reused_tmp(kf, oracle):
    n = 70_001
    q = _unit_quaternions(n, 4, np.float64)
    init = _unit_quaternions(1, 5, np.float64)
    want = oracle.c_scan_quat(q, init=init[0])
    src = to_dev(q.reshape(-1)).view(n, 4)
    dst = torch.empty_like(src)
    tmp = kf.get_allocation(kf.Scan1D, kf.identity, kf.QuaternionMul(), src)
    for _ in range(3):  # a stale descriptor of the call before would leak into the next one
        kf.scan_(kf.QuaternionMul(), dst, src, init=to_dev(init.reshape(-1)), tmp=tmp)
        assert np.abs(to_host(dst) - want).max() <= 1e-10
    kf.scan_(kf.QuaternionMul(), src, src, tmp=tmp)  # in place
    assert np.abs(to_host(src) - oracle.c_scan_quat(q)).max() <= 1e-10
    # a view that starts 8 bytes into the buffer: not 16-byte aligned -> component-wise accesses
    flat = to_dev(np.concatenate([[0.0], q.reshape(-1)]))
    out = torch.zeros(4 * n + 1, dtype=torch.float64, device="cuda")
    kf.scan_(kf.QuaternionMul(), out[1:].view(n, 4), flat[1:].view(n, 4))
    assert np.abs(to_host(out)[1:].reshape(n, 4) - oracle.c_scan_quat(q)).max() <= 1e-10
    assert to_host(out)[0] == 0.0
    with pytest.raises(kf.ArgumentError):
        kf.scan(kf.QuaternionMul(), torch.ones(12, dtype=torch.float32, device="cuda").view(4, 3))
    with pytest.raises(kf.ArgumentError):
        kf.scan(kf.abs2, kf.QuaternionMul(), src)
    with pytest.raises(kf.ArgumentError):
        kf.mapreduce(kf.identity, kf.QuaternionMul(), src)  # not commutative: scan only


def test_quaternion_bounded_wait_runs_out(kf, oracle):
    """Eight self-validating descriptor words per tile: a silent tile still ends in KF_ERR_TIMEOUT, and
    the workspace serves the next call."""
    from kernelforge_jl_b200 import _cabi as C
    n = 30 * 1024 + 7
    q = _unit_quaternions(n, 6, np.float64)
    src = to_dev(q.reshape(-1)).view(n, 4)
    dst = torch.empty_like(src)
    tmp = kf.get_allocation(kf.Scan1D, kf.identity, kf.QuaternionMul(), src)
    kf.scan_(kf.QuaternionMul(), dst, src, tmp=tmp, _test_hook=((1 + 3) << 16) | 400)
    assert kf.lib.kf_check(tmp.ptr(), None) == C.ERR_TIMEOUT
    kf.scan_(kf.QuaternionMul(), dst, src, tmp=tmp)
    assert kf.lib.kf_check(tmp.ptr(), None) == C.OK
    assert np.abs(to_host(dst) - oracle.c_scan_quat(q)).max() <= 1e-10


def test_errors(kf):
    x = torch.ones(100, dtype=torch.float32, device="cuda")
    with pytest.raises(kf.ArgumentError):
        kf.scan(lambda a, b: a - b, x)
    with pytest.raises(kf.ArgumentError):
        kf.scan("+", x, g=lambda v: v * 2)
    with pytest.raises(kf.ArgumentError):
        kf.scan_("+", torch.empty(99, dtype=torch.float32, device="cuda"), x)
    small = kf.KernelBuffer(kf.Scan1D, torch.empty(64, dtype=torch.uint8, device="cuda"))
    with pytest.raises(kf.KernelForgeError):
        kf.scan("+", x, tmp=small)
    tmp = kf.get_allocation(kf.Scan1D, kf.identity, "+", x)
    kf.scan("+", x, tmp=tmp)
    assert kf.lib.kf_check(tmp.ptr(), None) == 0  # (a workspace no call has used yet holds no status)


def test_full_size_2p28_uint32(kf):
    """n = 2^28, UInt32 ~ U{0..255}, wrapping add, bit-exact: verified by the size-independent
    property dst[0] == x[0], dst[i] - dst[i-1] == x[i] (wrapping) on the device, plus the total."""
    n = 1 << 28
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randint(0, 256, (n,), dtype=torch.int32, device="cuda", generator=g)
    dst = torch.empty_like(x)
    tmp = kf.get_allocation(kf.Scan1D, kf.identity, "+", x.view(torch.uint32))
    kf.scan_("+", dst.view(torch.uint32), x.view(torch.uint32), tmp=tmp)
    assert kf.lib.kf_check(tmp.ptr(), None) == 0
    assert bool((dst[0] == x[0]).item())
    assert bool(((dst[1:] - dst[:-1]) == x[1:]).all().item())  # int32 subtraction wraps like uint32
    total = int(x.sum(dtype=torch.int64).item()) & 0xFFFFFFFF
    assert (int(dst[-1].item()) & 0xFFFFFFFF) == total
    assert total != int(x.sum(dtype=torch.int64).item())  # the running sum really wrapped


def test_full_size_2p28_float32(kf):
    """n = 2^28, Float32 ~ U[0,1): element-wise within 1e-5*log2(n) = 2.8e-4 relative of a Float64
    cumulative sum of the same device data."""
    n = 1 << 28
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.rand(n, dtype=torch.float32, device="cuda", generator=g)
    dst = kf.scan("+", x)
    ref = torch.cumsum(x.double(), 0)
    rel = ((dst.double() - ref).abs() / ref.clamp_min(1e-30)).max().item()
    assert rel <= scan_tol(n), rel


def test_full_size_2p26_affine(kf):
    """n = 2^26 affine maps, two Float32 arrays: compared on the device with a Float64 blocked
    evaluation of the same left fold (exact composition per block of 2^16, then a sequential carry
    over the 1024 block summaries)."""
    n = 1 << 26
    g = torch.Generator(device="cuda").manual_seed(2)
    a = 0.5 + 0.5 * torch.rand(n, dtype=torch.float32, device="cuda", generator=g)
    b = 2.0 * torch.rand(n, dtype=torch.float32, device="cuda", generator=g) - 1.0
    da, db = kf.scan(kf.AffineCompose(), (a, b))
    # B_i = a_i*B_{i-1} + b_i forgets its past geometrically (a <= 1, E[log2 a] ~ -0.44): a window of
    # 4096 predecessors reproduces it far below the tolerance. Check random windows in Float64.
    idx = torch.randint(4096, n, (64,), generator=torch.Generator().manual_seed(3)).tolist() + [n - 1, 4096]
    tol = scan_tol(n)
    for i in idx:
        aw = a[i - 4095:i + 1].double().cpu().numpy()
        bw = b[i - 4095:i + 1].double().cpu().numpy()
        B = 0.0
        for k in range(4096):
            B = aw[k] * B + bw[k]
        assert abs(db[i].item() - B) <= tol * max(abs(B), 1.0)
    assert bool((da[2000:] == 0).all().item())  # the running gain has underflowed to exactly 0
    a_h = a[:2000].double().cpu().numpy()
    refA = np.cumprod(a_h)
    got = da[:2000].double().cpu().numpy()
    assert (np.abs(got - refA) <= tol * np.maximum(refA, 4 * float(np.finfo(np.float32).tiny))).all()


def test_host_pipeline_chunk_ring(kf, oracle):
    """Pinned host arrays through the chunked H2D / seeded scan / D2H ring: several arrays in one
    call, ragged chunk counts, more chunks than staging slots, the carry restarting at each array."""
    from kernelforge_jl_b200 import distributed as kfd

    n1, n2 = 1_000_003, 300_001
    rng = np.random.default_rng(7)
    a = rng.integers(0, 256, n1).astype(np.uint32)
    b = rng.integers(-1000, 1000, n2).astype(np.int64)
    ha = torch.from_numpy(a.view(np.int32)).pin_memory().view(torch.uint32)
    hb = torch.from_numpy(b).pin_memory()
    oa = torch.empty(n1, dtype=torch.int32).pin_memory().view(torch.uint32)
    ob = torch.empty(n2, dtype=torch.int64).pin_memory()
    pipe = kfd.HostScanPipeline(kf, max(n1, n2), chunk_bytes=1 << 18, slots=3)  # 16 and 10 chunks
    for _ in range(2):  # a second call reuses slots whose events are still recorded
        pipe.scan_host_many([("+", oa, ha), ("+", ob, hb)])
        torch.cuda.synchronize()
        assert (oa.view(torch.int32).numpy().view(np.uint32) == oracle.c_scan(0, 0, a)).all()
        assert (ob.numpy() == oracle.c_scan(0, 0, b)).all()
    c = rng.random(70_000).astype(np.float32)
    hc = torch.from_numpy(c).pin_memory()
    oc = torch.empty_like(hc).pin_memory()
    pipe.scan_host("max", oc, hc)
    torch.cuda.synchronize()
    assert (oc.numpy().astype(np.float64) == oracle.c_scan(0, 3, c)).all()


@pytest.mark.parametrize("workgroup,nitem", [(768, 4), (384, 8), (512, 8)])
def test_persistent_kernel_edges(kf, oracle, workgroup, nitem):
    """The persistent kernel forced onto sizes around its tile, ring and look-ahead boundaries: fewer
    tiles than ring steps, exactly one tile, one element over, fewer tiles than CTAs, a few more; a
    head tile (views off a 16-byte boundary by the same amount), in place, with a left seed."""
    tile = workgroup * nitem * 4  # elements of 4 bytes per tile
    rng = np.random.default_rng(workgroup)
    for n in (1, 3, tile - 1, tile, tile + 1, 2 * tile, 3 * tile + 5, 4 * tile, 7 * tile - 3, 149 * tile + 7, 400 * tile + 1):
        x = rng.integers(0, 1 << 32, n, dtype=np.uint32)
        got = to_host(kf.scan("+", to_dev(x), workgroup=workgroup, Nitem=nitem))
        assert (got == np.cumsum(x, dtype=np.uint32)).all(), n
    for n in (tile // 2 + 1, 5 * tile // 2 + 3):  # 8-byte elements: half as many per tile
        y = rng.integers(-1000, 1000, n).astype(np.int64)
        assert (to_host(kf.scan("min", to_dev(y), workgroup=workgroup, Nitem=nitem)) == np.minimum.accumulate(y)).all()
    n = 6 * tile + 11
    x = rng.integers(0, 1 << 32, n, dtype=np.uint32)
    for off in (1, 3):
        src = to_dev(x, offset=off)
        dst = to_dev(np.zeros(n, dtype=np.uint32), offset=off)
        kf.scan_("+", dst, src, workgroup=workgroup, Nitem=nitem)
        assert (to_host(dst) == np.cumsum(x, dtype=np.uint32)).all()
    t = to_dev(x)
    seed = to_dev(np.array([12345], dtype=np.uint32))
    kf.scan_("+", t, t, init=seed, workgroup=workgroup, Nitem=nitem)  # in place, seeded
    assert (to_host(t) == (np.cumsum(x, dtype=np.uint32) + np.uint32(12345))).all()
    f = rng.random(5 * tile + 9).astype(np.float32)
    _check_scan(kf, oracle, f, "+", workgroup=workgroup, Nitem=nitem)
    tmp = kf.get_allocation(kf.Scan1D, kf.identity, "+", to_dev(x), workgroup=workgroup, Nitem=nitem)
    for trial in range(4):  # a reused workspace: descriptors of the last call must not leak into the next
        z = rng.integers(0, 1 << 32, n, dtype=np.uint32)
        assert (to_host(kf.scan("+", to_dev(z), tmp=tmp, workgroup=workgroup, Nitem=nitem)) == np.cumsum(z, dtype=np.uint32)).all()


def test_random_sizes_offsets_variants(kf, oracle):
    """Many calls in a row with random lengths, view offsets, element widths and kernel variants,
    in the spirit of the reference's repeated-trial loops (test/tests/scan/scan_test.jl:107-125)."""
    import random

    rnd = random.Random(11)
    rng = np.random.default_rng(11)
    pool = rng.integers(0, 1 << 31, (1 << 22) + 64, dtype=np.int64).astype(np.int32)
    dev32 = to_dev(pool)
    for it in range(60):
        n = int(2 ** rnd.uniform(8, 22)) + rnd.randint(0, 5)
        off = rnd.choice([0, 0, 1, 2, 3, 4])
        var = rnd.choice([None, (768, 4), (384, 8), (512, 8), (256, 8)])
        kw = {} if var is None else dict(workgroup=var[0], Nitem=var[1])
        if rnd.random() < 0.5:
            got = to_host(kf.scan("+", dev32[off:off + n], **kw))
            assert (got == oracle.c_scan(0, 0, pool[off:off + n])).all(), (it, n, off, var)
        else:
            o2 = 2 * (off // 2)
            h = pool[o2:o2 + 2 * (n // 2 + 1)].view(np.int64)
            got = to_host(kf.scan("max", dev32[o2:o2 + 2 * (n // 2 + 1)].view(torch.int64), **kw))
            assert (got == oracle.c_scan(0, 3, h)).all(), (it, n, off, var)


@pytest.mark.parametrize("n", [7, 1000, 3_000_001])
def test_post_map_g_on_every_output(kf, oracle, n):
    """scan!(f, op, dst, src; g): g is applied to every output element, never to the carried prefix
    (src/scan/scan_kernel.jl:463,470,474 of the reference): sqrt of the running sum of squares."""
    x = np.random.default_rng(n).random(n).astype(np.float32)
    got = to_host(kf.scan(kf.abs2, "+", to_dev(x), g=kf.sqrt))
    ref = np.sqrt(oracle.c_scan(oracle.MAP_ABS2, oracle.OP_ADD, x))
    assert_close_rel(got, ref, n)
    xd = x.astype(np.float64)
    gotd = to_host(kf.scan("+", to_dev(xd), g="sqrt", workgroup=256, Nitem=4))  # the direct kernel as well
    assert_close_rel(gotd, np.sqrt(np.cumsum(xd)), n)
    with pytest.raises(kf.ArgumentError):
        kf.scan("+", to_dev(np.arange(10, dtype=np.int32)), g=kf.sqrt)  # sqrt of integers is not in the enum set


@pytest.mark.parametrize("workgroup,nitem", [(256, 8), (384, 8)])
def test_init_of_several_elements_is_folded_left_to_right(kf, oracle, workgroup, nitem):
    """`init` with k elements seeds the scan with init[0] op ... op init[k-1] (what a shard of a sharded
    scan passes: the totals of the shards before it)."""
    rng = np.random.default_rng(5)
    n = 2_000_003
    x = rng.integers(0, 1 << 32, n, dtype=np.uint64).astype(np.uint32)
    seeds = rng.integers(0, 1 << 32, 7, dtype=np.uint64).astype(np.uint32)
    got = to_host(kf.scan("+", to_dev(x), init=to_dev(seeds), workgroup=workgroup, Nitem=nitem))
    ref = oracle.c_scan(0, oracle.OP_ADD, np.concatenate([seeds, x]))[7:]
    assert (got == ref).all()
    # non-commutative: affine pairs, three seed pairs
    a = (0.5 + 0.5 * rng.random(n)).astype(np.float32)
    b = (2 * rng.random(n) - 1).astype(np.float32)
    sa = (0.5 + 0.5 * rng.random(3)).astype(np.float32)
    sb = (2 * rng.random(3) - 1).astype(np.float32)
    init = to_dev(np.stack([sa, sb], axis=1).reshape(-1).copy())
    da, db = kf.scan(kf.AffineCompose(), (to_dev(a), to_dev(b)), init=init, workgroup=workgroup, Nitem=nitem)
    ra, rb = oracle.c_scan_affine(np.concatenate([sa, a]), np.concatenate([sb, b]))
    tol = scan_tol(n)
    assert (np.abs(to_host(db) - rb[3:]) <= tol * np.maximum(np.abs(rb[3:]), 1.0)).all()
    assert (np.abs(to_host(da) - ra[3:]) <= tol * np.maximum(ra[3:], 4 * np.finfo(np.float32).tiny)).all()


@pytest.mark.parametrize("workgroup,nitem,what", [(256, 8, "direct"), (384, 8, "persistent")])
def test_bounded_wait_runs_out_and_the_workspace_recovers(kf, oracle, workgroup, nitem, what):
    """A look-back whose predecessor never publishes gives up after its poll limit: the call returns,
    kf_check reports KF_ERR_TIMEOUT with the tile that gave up, later tiles see the poison and return,
    and the next call on the same workspace is correct. Nothing faults or hangs: the silent tile and
    the short limit come through kf_launch_cfg.reserved (bits 16..31 = 1 + tile, bits 0..15 = polls)."""
    from kernelforge_jl_b200 import _cabi as C
    n = 40 * 384 * 8 * 4 + 17  # about 40 tiles of the persistent kernel, more of the direct one
    x = np.random.default_rng(9).integers(0, 256, n).astype(np.uint32)
    src = to_dev(x)
    dst = torch.empty_like(src)
    tmp = kf.get_allocation(kf.Scan1D, kf.identity, "+", src, workgroup=workgroup, Nitem=nitem)
    hook = ((1 + 3) << 16) | 400  # tile 3 stays silent; 400 polls (well under a millisecond each)
    kf.scan_("+", dst, src, tmp=tmp, workgroup=workgroup, Nitem=nitem, _test_hook=hook)
    assert kf.lib.kf_check(tmp.ptr(), None) == C.ERR_TIMEOUT
    header = tmp.workspace[:8].view(torch.int32).cpu().numpy()
    assert header[0] == C.ERR_TIMEOUT and header[1] >= 3  # word 1: the tile whose wait ran out
    kf.scan_("+", dst, src, tmp=tmp, workgroup=workgroup, Nitem=nitem)  # same workspace, no hook
    assert kf.lib.kf_check(tmp.ptr(), None) == C.OK
    assert (to_host(dst) == oracle.c_scan(0, oracle.OP_ADD, x)).all()
