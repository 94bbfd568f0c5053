"""GPU parity tests of `sort` / `sort!` (keys-only and key-value) against the CPU oracle, bit-exact,
through the C ABI.

Mirrors test/tests/sort/sort_test.jl (types and sizes :15-38, reused tmp :71-87, n=1..16 :94-104,
repeated trials :111-124, adversarial arrays :131-153, float boundary values :161-176, views
:231-267, launch sweep / stability / look-back :277-364) and test/tests/sort/sort_keyval_test.jl
(:15-38, :112-116, :161-185, :212-230) of KernelForge.jl.
"""
import numpy as np
import pytest
import torch

from util import bits, to_dev, to_host

pytestmark = pytest.mark.gpu

KEY_DTYPES = [np.uint8, np.int8, np.uint16, np.int16, np.uint32, np.int32, np.float32, np.uint64, np.int64, np.float64]


def rand_keys(dtype, n, rng):
    dt = np.dtype(dtype)
    if dt.kind == "f":
        return rng.standard_normal(n).astype(dtype)
    info = np.iinfo(dtype)
    return rng.integers(info.min, info.max, size=n, dtype=dtype, endpoint=True)


def assert_same_bits(got, ref):
    assert got.dtype == ref.dtype and got.shape == ref.shape
    assert (bits(got) == bits(ref)).all()


@pytest.mark.parametrize("dtype", KEY_DTYPES)
@pytest.mark.parametrize("n", [1, 33, 100, 10_001, 1_000_000])
def test_keys_types_sizes(kf, oracle, dtype, n):
    x = rand_keys(dtype, n, np.random.default_rng(n))
    src = to_dev(x)
    y = kf.sort(src)
    assert_same_bits(to_host(y), oracle.c_sort(x))
    assert_same_bits(to_host(src), x)  # out-of-place leaves src untouched
    kf.sort_(src)  # in place
    assert_same_bits(to_host(src), oracle.c_sort(x))


@pytest.mark.parametrize("dtype", [np.uint8, np.int8])
def test_one_byte_keys_runs_path(kf, oracle, dtype):
    """One-byte keys without payload are written out as the 256 runs of their histogram: every size
    around the 16-byte vector width, every alignment of dst and src, sparse and one-valued inputs,
    in place, and the single-pass onesweep kernel (taken with a payload) as a second opinion."""
    rng = np.random.default_rng(77)
    info = np.iinfo(dtype)
    for n in (1, 2, 15, 16, 17, 31, 32, 33, 255, 256, 1000, 4097, 65_537, 1_000_003, 9_000_001):
        cases = [rng.integers(info.min, info.max, n, dtype=dtype, endpoint=True),
                 np.full(n, info.min, dtype=dtype), np.full(n, info.max, dtype=dtype),
                 rng.choice(np.array([info.min, -1 if info.min < 0 else 127, 0, 5, info.max], dtype=dtype), n),
                 (np.arange(n) % 256).astype(np.uint8).view(dtype)]
        for x in cases:
            assert_same_bits(to_host(kf.sort(to_dev(x))), oracle.c_sort(x))
    x = rng.integers(info.min, info.max, 100_000, dtype=dtype, endpoint=True)
    for off_src in (0, 1, 7):
        for off_dst in (0, 1, 3, 8, 15):
            for n in (5, 40, 99_000):
                big_src = to_dev(x)
                big_dst = torch.zeros(100_000 + 64, dtype=big_src.dtype, device="cuda")
                kf.sort_(big_dst[off_dst:off_dst + n], big_src[off_src:off_src + n])
                got = to_host(big_dst)
                assert_same_bits(got[off_dst:off_dst + n], oracle.c_sort(x[off_src:off_src + n]))
                assert not got[:off_dst].any() and not got[off_dst + n:].any()  # nothing outside dst
    src = to_dev(x)
    kf.sort_(src[3:90_003])  # in place on a misaligned view
    got = to_host(src)
    assert_same_bits(got[3:90_003], oracle.c_sort(x[3:90_003]))
    assert_same_bits(got[:3], x[:3])
    assert_same_bits(got[90_003:], x[90_003:])
    vals = torch.arange(100_000, dtype=torch.int32, device="cuda")
    _, keys_sorted = kf.sort(vals, keys=to_dev(x))
    assert_same_bits(to_host(keys_sorted), to_host(kf.sort(to_dev(x))))


@pytest.mark.parametrize("n", [1, 33, 10_001, 1_000_000])
def test_bool_input(kf, n):
    """Bool arrays sort as bytes (test/tests/sort/sort_test.jl:183-193 of KernelForge.jl: `rand(Bool, n)`
    against Base.sort): all false before all true, and the same count of each."""
    x = np.random.default_rng(n).integers(0, 2, n).astype(np.bool_)
    y = kf.sort(torch.from_numpy(x).cuda())
    assert y.dtype == torch.bool
    assert (y.cpu().numpy() == np.sort(x)).all()


@pytest.mark.parametrize("dtype", [np.uint16, np.int16])
def test_two_byte_keys_runs_path(kf, oracle, dtype):
    """Two-byte keys without payload, from 2^22 keys on, are written out as the 65 536 runs of their
    histogram: dense and sparse value sets (long stretches of empty bins), one value, every value
    once among long runs, misaligned and in-place arrays; the size just below takes the onesweep."""
    rng = np.random.default_rng(78)
    info = np.iinfo(dtype)
    every = np.arange(65536, dtype=np.uint16).view(dtype)
    for n in ((1 << 22) - 1, 1 << 22, (1 << 22) + 13, 6_000_001):
        cases = [rng.integers(info.min, info.max, n, dtype=dtype, endpoint=True),
                 np.full(n, info.min, dtype=dtype),
                 rng.choice(np.array([info.min, info.min + 1, 0, 77, 30_000, info.max], dtype=dtype), n),
                 rng.integers(0, 1000, n).astype(dtype),
                 np.concatenate([every, np.full(n - 65536, 12_345, dtype=dtype)])[rng.permutation(n)]]
        for x in cases:
            assert_same_bits(to_host(kf.sort(to_dev(x))), oracle.c_sort(x))
    n = (1 << 22) + 40
    x = rng.integers(info.min, info.max, n + 16, dtype=dtype, endpoint=True)
    for off_src, off_dst in ((0, 1), (1, 0), (3, 7), (5, 5)):
        big_dst = torch.zeros(n + 32, dtype=to_dev(x[:1]).dtype, device="cuda")
        kf.sort_(big_dst[off_dst:off_dst + n], to_dev(x)[off_src:off_src + n])
        got = to_host(big_dst)
        assert_same_bits(got[off_dst:off_dst + n], oracle.c_sort(x[off_src:off_src + n]))
        assert not got[:off_dst].any() and not got[off_dst + n:].any()  # nothing outside dst
    src = to_dev(x)
    kf.sort_(src[3:3 + n])  # in place on a misaligned view
    got = to_host(src)
    assert_same_bits(got[3:3 + n], oracle.c_sort(x[3:3 + n]))
    assert_same_bits(got[:3], x[:3])
    assert_same_bits(got[3 + n:], x[3 + n:])


@pytest.mark.parametrize("n", list(range(1, 17)))
def test_tiny_sizes(kf, oracle, n):
    for dtype in (np.uint32, np.float32):
        x = rand_keys(dtype, n, np.random.default_rng(100 + n))
        assert_same_bits(to_host(kf.sort(to_dev(x))), oracle.c_sort(x))


def test_repeated_trials(kf, oracle):
    for trial in range(10):
        x = rand_keys(np.uint32, 300_007, np.random.default_rng(trial))
        assert_same_bits(to_host(kf.sort(to_dev(x))), oracle.c_sort(x))


@pytest.mark.parametrize("dtype", [np.uint32, np.int32, np.float32])
def test_adversarial(kf, oracle, dtype):
    n = 10_001
    rng = np.random.default_rng(5)
    T = np.dtype(dtype).type
    lo = T(-np.inf) if np.dtype(dtype).kind == "f" else np.iinfo(dtype).min
    hi = T(np.inf) if np.dtype(dtype).kind == "f" else np.iinfo(dtype).max
    outlier = np.full(n, 3, dtype=dtype)
    outlier[n // 2] = 99
    cases = {
        "all-equal": np.full(n, 7, dtype=dtype),
        "sorted": np.sort(rand_keys(dtype, n, rng)),
        "reverse": np.sort(rand_keys(dtype, n, rng))[::-1].copy(),
        "two-value": (np.arange(1, n + 1) % 2).astype(dtype),
        "typemin/max": np.where(np.arange(1, n + 1) % 2 == 0, lo, hi).astype(dtype),
        "single-outlier": outlier,
    }
    for name, x in cases.items():
        assert_same_bits(to_host(kf.sort(to_dev(x))), oracle.c_sort(x))


def test_float_boundary_values(kf, oracle):
    """+-Inf, -0.0 before +0.0, subnormals; compared bit for bit (`isequal` in the reference)."""
    n = 10_001
    rng = np.random.default_rng(6)
    i = np.arange(1, n + 1)
    sub = (rng.integers(1, 1 << 23, n).astype(np.uint32) | (rng.integers(0, 2, n).astype(np.uint32) << 31)).view(np.float32)
    mixed = np.concatenate([rng.standard_normal(n - 4).astype(np.float32),
                            np.array([np.inf, -np.inf, 0.0, -0.0], dtype=np.float32)])
    cases = [
        np.where(i % 2 == 1, np.float32(np.inf), np.float32(-np.inf)).astype(np.float32),
        np.where(i % 2 == 0, np.float32(-0.0), np.float32(0.0)).astype(np.float32),
        mixed, sub, np.concatenate([mixed, sub]),
    ]
    for x in cases:
        got = to_host(kf.sort(to_dev(x)))
        assert_same_bits(got, oracle.c_sort(x))
    z = to_host(kf.sort(to_dev(cases[1])))
    assert np.signbit(z[: n // 2]).all() and not np.signbit(z[n // 2:]).any()
    x64 = np.concatenate([mixed, sub]).astype(np.float64)
    x64[::5] = -0.0
    assert_same_bits(to_host(kf.sort(to_dev(x64))), oracle.c_sort(x64))


@pytest.mark.parametrize("key_dtype", [np.uint8, np.int16, np.uint32, np.int32, np.float32, np.uint64, np.int64, np.float64])
@pytest.mark.parametrize("val_dtype", [np.int32, np.int64, np.float32, np.float64])
def test_key_value(kf, oracle, key_dtype, val_dtype):
    """`keys` drives the order, `vals` follows: vals_out == vals[sortperm(keys)] (stable)."""
    for n in (1, 100, 10_001, 400_003):
        rng = np.random.default_rng(n)
        keys = rand_keys(key_dtype, n, rng)
        if n > 100:
            keys[::3] = keys[0]  # duplicates make stability observable
        vals = rng.standard_normal(n).astype(val_dtype) if np.dtype(val_dtype).kind == "f" else \
            rng.integers(-1000, 1000, n).astype(val_dtype)
        rk, rv = oracle.c_sort_pairs(keys, vals)
        k_dev, v_dev = to_dev(keys), to_dev(vals)
        v_out, k_out = kf.sort(v_dev, keys=k_dev)
        assert_same_bits(to_host(k_out), rk)
        assert_same_bits(to_host(v_out), rv)
        assert_same_bits(to_host(k_dev), keys)  # sources untouched
        assert_same_bits(to_host(v_dev), vals)
        v2, k2 = kf.sort_(v_dev, keys=k_dev)  # in place sorts both
        assert v2 is v_dev and k2 is k_dev
        assert_same_bits(to_host(k_dev), rk)
        assert_same_bits(to_host(v_dev), rv)


def test_key_value_index_payload_and_sortperm(kf, oracle):
    """UInt32 keys with payload = original index (0-based): the payload is the stable sortperm."""
    n = 1_000_003
    keys = np.random.default_rng(0).integers(0, 5000, n).astype(np.uint32)  # ~200 duplicates per key
    idx = np.arange(n, dtype=np.uint32)
    v_out, k_out = kf.sort(to_dev(idx), keys=to_dev(keys))
    perm = oracle.c_sortperm(keys)
    assert (to_host(v_out).astype(np.uint64) == perm).all()
    assert (to_host(kf.sortperm(to_dev(keys))).astype(np.uint64) == perm).all()


def test_key_value_errors(kf):
    v = torch.zeros(10, dtype=torch.int32, device="cuda")
    with pytest.raises(kf.KernelForgeError):
        kf.sort(v, keys=torch.zeros(9, dtype=torch.int32, device="cuda"))
    with pytest.raises(kf.ArgumentError):
        kf.sort(v.to(torch.int16), keys=v)
    for bad in (dict(by=lambda t: -t), dict(rev=True), dict(lt=lambda a, b: a > b), dict(uint_map=lambda t: t),
                dict(algorithm="sample")):
        with pytest.raises(kf.ArgumentError):
            kf.sort(v, **bad)
    with pytest.raises(kf.ArgumentError):
        kf.sort(v.to(torch.float16))  # no radix mapping for this element type here
    assert kf.sort(v.to(torch.int16)).dtype == torch.int16  # every integer width is a key type


@pytest.mark.parametrize("workgroup,nitem", [(256, 16), (512, 16), (512, 24), (384, 24)])
def test_launch_variants_and_stability(kf, oracle, workgroup, nitem):
    """Every compiled tile shape: same bits as the oracle, stable at every shape, and a tile shape
    outside the compiled set raises while the context stays usable."""
    n = 2_000_003
    rng = np.random.default_rng(workgroup + nitem)
    x = rand_keys(np.uint32, n, rng)
    assert_same_bits(to_host(kf.sort(to_dev(x), workgroup=workgroup, Nitem=nitem)), oracle.c_sort(x))
    keys = rng.integers(0, 1000, n).astype(np.int32)  # ~2000 duplicates per key
    idx = np.arange(n, dtype=np.int32)
    v_out, k_out = kf.sort(to_dev(idx), keys=to_dev(keys), workgroup=workgroup, Nitem=nitem)
    assert (to_host(v_out).astype(np.uint64) == oracle.c_sortperm(keys)).all()
    with pytest.raises(kf.ArgumentError):
        kf.sort(to_dev(x), workgroup=4096, Nitem=64)
    assert_same_bits(to_host(kf.sort(to_dev(x[:1000]))), oracle.c_sort(x[:1000]))


def test_reused_tmp(kf, oracle):
    n = 250_000
    src = torch.zeros(n, dtype=torch.float32, device="cuda")
    tmp = kf.get_allocation(kf.Sort1D, src)
    for call in range(5):
        x = rand_keys(np.float32, n, np.random.default_rng(call))
        src.copy_(torch.from_numpy(x))
        dst = torch.empty_like(src)
        kf.sort_(dst, src, tmp=tmp)
        assert_same_bits(to_host(dst), oracle.c_sort(x))
    keys = torch.zeros(n, dtype=torch.int32, device="cuda")
    tmp2 = kf.get_allocation(kf.Sort1D, src, keys=keys)
    for call in range(3):
        k = rand_keys(np.int32, n, np.random.default_rng(10 + call))
        x = rand_keys(np.float32, n, np.random.default_rng(20 + call))
        v_out, k_out = kf.sort(to_dev(x), keys=to_dev(k), tmp=tmp2)
        rk, rv = oracle.c_sort_pairs(k, x)
        assert_same_bits(to_host(k_out), rk)
        assert_same_bits(to_host(v_out), rv)
    small = kf.KernelBuffer(kf.Sort1D, torch.empty(1024, dtype=torch.uint8, device="cuda"))
    with pytest.raises(kf.KernelForgeError):
        kf.sort(src, tmp=small)


@pytest.mark.parametrize("offset", [1, 2, 3])
def test_views_unaligned(kf, oracle, offset):
    n = 100_001
    x = rand_keys(np.float32, n, np.random.default_rng(offset))
    src = to_dev(x, offset=offset)
    dst = to_dev(np.zeros(n, np.float32), offset=(offset + 1) % 4)
    kf.sort_(dst, src)
    assert_same_bits(to_host(dst), oracle.c_sort(x))
    kf.sort_(src)
    assert_same_bits(to_host(src), oracle.c_sort(x))


def test_lookback_many_tiles(kf, oracle):
    """n = 4e6 (hundreds of tiles): the digit offsets really come from the look-back chain."""
    n = 4_000_000
    x = rand_keys(np.uint32, n, np.random.default_rng(42))
    src = to_dev(x)
    tmp = kf.get_allocation(kf.Sort1D, src)
    y = kf.sort(src, tmp=tmp)
    assert kf.lib.kf_check(tmp.ptr(), None) == 0
    assert_same_bits(to_host(y), oracle.c_sort(x))
    skew = (x & np.uint32(0x000000FF)) | np.uint32(0xABCD0000)  # three of four digits constant
    assert_same_bits(to_host(kf.sort(to_dev(skew))), oracle.c_sort(skew))


def _mapped_i64(t):
    """Order-preserving int64 image of uint32 / float32 keys held in a device tensor."""
    u = t.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    if t.dtype == torch.float32:
        neg = (u >> 31) == 1
        u = torch.where(neg, (~u) & 0xFFFFFFFF, u | 0x80000000)
    return u


def _checksums(t):
    u = t.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    return int(u.sum().item()), int((u * u + 7 * u).sum().item())  # int64 wrap-around sums


@pytest.mark.parametrize("kind", ["uint32", "float32"])
def test_full_size_2p28_keys(kf, kind):
    """n = 2^28 keys: sorted under the key map, and the same multiset (two wrap-around checksums)."""
    n = 1 << 28
    g = torch.Generator(device="cuda").manual_seed(0)
    if kind == "uint32":
        x = torch.randint(-2**31, 2**31, (n,), dtype=torch.int32, device="cuda", generator=g).view(torch.uint32)
    else:
        x = torch.randn(n, dtype=torch.float32, device="cuda", generator=g)
        pos = torch.randint(0, n, (n // 1000,), device="cuda", generator=g)
        special = torch.randint(0, 1 << 23, (n // 1000,), dtype=torch.int32, device="cuda", generator=g)
        special = torch.where(special % 4 == 0, torch.zeros_like(special), special)  # zeros and subnormals
        sign = torch.randint(0, 2, (n // 1000,), dtype=torch.int32, device="cuda", generator=g) << 31
        x.view(torch.int32)[pos] = special | sign
    before = _checksums(x)
    tmp = kf.get_allocation(kf.Sort1D, x)
    kf.sort_(x, tmp=tmp)
    assert kf.lib.kf_check(tmp.ptr(), None) == 0
    assert _checksums(x) == before
    m = _mapped_i64(x)
    assert bool((m[1:] >= m[:-1]).all().item())


def test_full_size_2p28_pairs(kf):
    """n = 2^28 UInt32 keys + UInt32 payload = original index: keys sorted, payload a permutation that
    maps back to the keys (keys_src[payload] == keys_dst), ascending within equal keys (stable)."""
    n = 1 << 28
    g = torch.Generator(device="cuda").manual_seed(1)
    keys = torch.randint(-2**31, 2**31, (n,), dtype=torch.int32, device="cuda", generator=g).view(torch.uint32)
    keys.view(torch.int32)[: n // 2] &= 0x000FFFFF  # half the keys collide heavily
    idx = torch.arange(n, dtype=torch.int32, device="cuda").view(torch.uint32)
    v_out, k_out = kf.sort(idx, keys=keys)
    gathered = keys.view(torch.int32)[v_out.view(torch.int32).to(torch.int64)]
    assert bool((gathered == k_out.view(torch.int32)).all().item())
    del gathered
    m = _mapped_i64(k_out)
    assert bool((m[1:] >= m[:-1]).all().item())
    same = m[1:] == m[:-1]
    del m
    v = v_out.view(torch.int32)
    assert bool((v[1:][same] > v[:-1][same]).all().item())


def test_bounded_wait_runs_out_in_a_sort_pass(kf, oracle):
    """One tile of every pass publishes nothing: the look-back of the next tile gives up after its poll
    limit, records KF_ERR_TIMEOUT and poisons its descriptors, later tiles return, the call returns.
    The next sort on the same workspace is correct."""
    from kernelforge_jl_b200 import _cabi as C
    n = 30 * 512 * 24 + 5
    x = rand_keys(np.uint32, n, np.random.default_rng(3))
    src = to_dev(x)
    dst = torch.empty_like(src)
    tmp = kf.get_allocation(kf.Sort1D, src)
    kf.sort_(dst, src, tmp=tmp, _test_hook=((1 + 2) << 16) | 300)
    assert kf.lib.kf_check(tmp.ptr(), None) == C.ERR_TIMEOUT
    header = tmp.workspace[:8].view(torch.int32).cpu().numpy()
    assert header[0] == C.ERR_TIMEOUT and header[1] >= 2
    kf.sort_(dst, src, tmp=tmp)
    assert kf.lib.kf_check(tmp.ptr(), None) == C.OK
    assert_same_bits(to_host(dst), oracle.c_sort(x))


@pytest.mark.parametrize("seed", [3, 4])
def test_random_stress_stability_every_variant(kf, oracle, seed):
    """Seeded random cases (sizes 2^4..2^24, six key kinds including heavy duplicates, every compiled
    launch variant): key-value sort with the original index as payload against the oracle's stable
    permutation, and the keys-only sort, bit for bit. Restates the stability tests of the reference
    (test/tests/sort/sort_test.jl:316-334) as a randomised sweep."""
    import random
    rnd = random.Random(seed)
    rng = np.random.default_rng(seed)
    for it in range(60):
        n = int(2 ** rnd.uniform(4, 24)) + rnd.randint(0, 7)
        kind = rnd.choice(["i32", "i64", "f32", "i16", "u8", "few", "few64"])
        if kind == "i32":
            k = rng.integers(-2**31, 2**31, n).astype(np.int32)
        elif kind == "i64":
            k = rng.integers(-2**62, 2**62, n).astype(np.int64)
        elif kind == "f32":
            k = rng.standard_normal(n).astype(np.float32)
            k[::97] = -0.0
        elif kind == "i16":
            k = rng.integers(-2**15, 2**15, n).astype(np.int16)
        elif kind == "u8":
            k = rng.integers(0, 256, n).astype(np.uint8)
        elif kind == "few":
            k = rng.integers(0, 5, n).astype(np.int32)  # long groups of equal digits inside every half-warp
        else:
            k = (rng.integers(0, 3, n) * (1 << 40)).astype(np.int64)
        var = rnd.choice([None, (512, 24), (512, 16), (384, 24), (256, 16)])
        kw = {} if var is None else dict(workgroup=var[0], Nitem=var[1])
        dk = to_dev(k)
        idx = torch.arange(n, dtype=torch.int32, device="cuda")
        vals, keys = kf.sort(idx, keys=dk, **kw)
        perm = oracle.c_sortperm(k)
        assert (to_host(vals).astype(np.uint64) == perm).all(), (it, n, kind, var)
        assert_same_bits(to_host(keys), k[perm.astype(np.int64)])
        assert_same_bits(to_host(kf.sort(dk, **kw)), k[perm.astype(np.int64)])


@pytest.mark.parametrize("n,kind", [(30_000_001, "uint32"), (20_000_003, "float32"), (12_500_000, "int64")])
def test_tens_of_millions_against_the_oracle(kf, oracle, n, kind):
    """Thousands of tiles compared bit for bit with the oracle (the full-size tests check properties)."""
    rng = np.random.default_rng(n)
    x = rand_keys(np.dtype(kind).type, n, rng)
    assert_same_bits(to_host(kf.sort(to_dev(x))), oracle.c_sort(x))


@pytest.mark.parametrize("dtype", [np.uint8, np.int16, np.uint32, np.int32, np.float32, np.uint64, np.float64])
@pytest.mark.parametrize("n,offset", [(1, 0), (15, 0), (16, 0), (1000, 0), (100_003, 0), (100_003, 3), (1 << 20, 0)])
def test_bucket_ids_and_upper_bounds(kf, oracle, dtype, n, offset):
    """The two helpers of the sharded sample sort against numpy on the mapped keys: destination ids of an
    unsorted shard (vector path, scalar tail, misaligned view) and the cut points of a sorted one."""
    import ctypes
    from kernelforge_jl_b200 import _cabi as C, ops
    rng = np.random.default_rng(n + offset)
    x = rand_keys(dtype, n, rng)
    nsplit = 7
    spl = np.sort(oracle.np_uint_map(rand_keys(dtype, nsplit, rng)))
    # splitters are keys: map the sorted unsigned images back through the sort order of real keys
    cand = rand_keys(dtype, 4096, rng)
    cand = cand[np.argsort(oracle.np_uint_map(cand), kind="stable")]
    splitters = cand[np.linspace(100, 4000, nsplit).astype(int)]
    ms = oracle.np_uint_map(splitters)
    dx, ds = to_dev(x, offset=offset), to_dev(splitters)
    out = torch.empty(n, dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    rc = kf.lib.kf_bucket_ids(ops.dtype_code(dx), dx.data_ptr(), n, ds.data_ptr(), nsplit, out.data_ptr(), st)
    assert rc == C.OK
    want = np.searchsorted(ms, oracle.np_uint_map(x), side="left").astype(np.uint8)
    assert (out.cpu().numpy() == want).all()
    srt = oracle.c_sort(x)
    dsrt = to_dev(srt)
    cuts = torch.empty(nsplit, dtype=torch.int64, device="cuda")
    assert kf.lib.kf_upper_bounds(ops.dtype_code(dsrt), dsrt.data_ptr(), n, ds.data_ptr(), nsplit, cuts.data_ptr(), st) == C.OK
    assert (cuts.cpu().numpy() == np.searchsorted(oracle.np_uint_map(srt), ms, side="right")).all()
