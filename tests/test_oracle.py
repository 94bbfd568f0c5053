"""CPU tests of the oracle (oracle/kf_oracle.c via oracle/oracle.py).

The oracle is pinned three ways:
  1. against the closed-form cases of the reference's own tests (sum(1:n) of
     test/tests/mapreduce/mapreduce1d_test.jl:14-29; the adversarial and boundary arrays of
     test/tests/sort/sort_test.jl:131-176, whose sorted form is known without sorting);
  2. against an independent numpy restatement of the same Base semantics;
  3. the committed fixtures of tests/golden/ (written by make_golden.py FROM THE ORACLE ITSELF) are a
     regression freeze of the oracle, not a pin: they only show that it has not changed since.
The reference stores no golden vectors for this path and cannot run here (it is Julia), so parity
against it stays "partial": what is restated below are the cases of its tests whose expected
values follow from their construction (n = 1..16 sorts, the stability pairs with about 2000
duplicates per key, UInt8 wrap-around with +/max/min, n = 1..10 scans).
"""
import os

import numpy as np
import pytest

from util import bits

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("n", [33, 100, 10_001, 100_000])
def test_sum_1_to_n_closed_form(oracle, n):
    exact = n * (n + 1) // 2
    assert oracle.c_mapreduce(0, 0, np.arange(1, n + 1, dtype=np.float64)) == float(exact)
    assert oracle.c_mapreduce(0, 0, np.arange(1, n + 1, dtype=np.float32)) == float(exact)  # Float64 fold of exact ints
    wrapped = np.array([exact], dtype=np.int64).astype(np.int32)[0]
    assert oracle.c_mapreduce(0, 0, np.arange(1, n + 1, dtype=np.int32)) == wrapped
    scan = oracle.c_scan(0, 0, np.arange(1, n + 1, dtype=np.int64))
    k = np.arange(1, n + 1, dtype=np.int64)
    assert (scan == k * (k + 1) // 2).all()


@pytest.mark.parametrize("dtype", [np.uint32, np.int32, np.float32, np.uint64, np.int64, np.float64])
def test_sort_adversarial_closed_form(oracle, dtype):
    n = 10_001
    T = np.dtype(dtype).type
    assert (oracle.c_sort(np.full(n, 7, dtype=dtype)) == 7).all()
    two = (np.arange(1, n + 1) % 2).astype(dtype)  # iseven(i) ? 0 : 1
    s = oracle.c_sort(two)
    assert (s[: n // 2] == 0).all() and (s[n // 2:] == 1).all()
    if np.dtype(dtype).kind == "f":
        lo, hi = T(-np.inf), T(np.inf)
    else:
        lo, hi = np.iinfo(dtype).min, np.iinfo(dtype).max
    mm = np.where(np.arange(1, n + 1) % 2 == 0, lo, hi).astype(dtype)
    s = oracle.c_sort(mm)
    assert (s[: n // 2] == lo).all() and (s[n // 2:] == hi).all()
    out = np.full(n, 3, dtype=dtype)
    out[n // 2] = 99
    s = oracle.c_sort(out)
    assert (s[:-1] == 3).all() and s[-1] == 99
    rev = np.arange(n, 0, -1).astype(dtype)
    assert (oracle.c_sort(rev) == np.arange(1, n + 1).astype(dtype)).all()


def test_sort_float_zero_and_inf_order(oracle):
    n = 10_001
    i = np.arange(1, n + 1)
    z = np.where(i % 2 == 0, np.float32(-0.0), np.float32(0.0)).astype(np.float32)
    s = oracle.c_sort(z)
    assert np.signbit(s[: n // 2]).all() and not np.signbit(s[n // 2:]).any()  # -0.0 sorts before +0.0
    x = np.array([np.inf, -np.inf, 0.0, -0.0, 1e-45, -1e-45, 1.0, -1.0], dtype=np.float32)
    expect = np.array([-np.inf, -1.0, -1e-45, -0.0, 0.0, 1e-45, 1.0, np.inf], dtype=np.float32)
    assert (bits(oracle.c_sort(x)) == bits(expect)).all()
    # stability: equal keys keep their input order
    keys = np.array([2, 1, 2, 1, 2], dtype=np.int32)
    assert list(oracle.c_sortperm(keys)) == [1, 3, 0, 2, 4]


@pytest.mark.parametrize("dtype", [np.uint8, np.int8, np.uint16, np.int16, np.uint32, np.int32, np.uint64, np.int64])
@pytest.mark.parametrize("op", range(7))
def test_integer_ops_match_numpy(oracle, dtype, op):
    rng = np.random.default_rng(op)
    info = np.iinfo(dtype)
    x = rng.integers(info.min, info.max, size=5003, dtype=dtype, endpoint=True)
    assert (oracle.c_scan(0, op, x) == oracle.np_scan(0, op, x)).all()
    assert oracle.c_mapreduce(0, op, x) == oracle.np_mapreduce(0, op, x)
    for f in (1, 2):
        if f == 2 and np.dtype(dtype).kind == "u":
            continue
        assert (oracle.c_scan(f, 0, x) == oracle.np_scan(f, 0, x)).all()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_float_scan_matches_numpy_float64(oracle, dtype):
    x = np.random.default_rng(1).random(100_003).astype(dtype)
    for op in (0, 2, 3):
        a, b = oracle.c_scan(0, op, x), oracle.np_scan(0, op, x)
        assert np.allclose(a, b, rtol=1e-13, atol=0)
    assert abs(oracle.c_mapreduce(1, 0, x) - float(np.sum(x.astype(np.float64) ** 2))) <= 1e-9 * x.size
    assert oracle.c_scan(0, 0, x, init=2.5)[0] == 2.5 + float(x[0])


@pytest.mark.parametrize("dtype", [np.uint32, np.int32, np.float32, np.uint64, np.int64, np.float64, np.uint8, np.int16])
def test_sort_matches_numpy_stable_argsort(oracle, dtype):
    rng = np.random.default_rng(2)
    n = 50_001
    if np.dtype(dtype).kind == "f":
        x = rng.standard_normal(n).astype(dtype)
        x[::7] = -0.0
        x[::11] = 0.0
        x[5] = np.inf
        x[6] = -np.inf
    else:
        info = np.iinfo(dtype)
        x = rng.integers(info.min, info.max, size=n, dtype=dtype, endpoint=True)
        x[::3] = x[0]
    assert (oracle.c_sortperm(x).astype(np.int64) == oracle.np_sortperm(x)).all()
    if np.dtype(dtype).kind != "f":
        assert (oracle.c_sort(x) == np.sort(x, kind="stable")).all()


def test_affine_fold_small_by_hand(oracle):
    a = np.array([2.0, 0.5, 3.0], dtype=np.float32)
    b = np.array([1.0, -1.0, 0.25], dtype=np.float32)
    # x -> 2x+1, then 0.5x-1, then 3x+0.25:  (2,1); (1,-0.5); (3,-1.25)
    oa, ob = oracle.c_scan_affine(a, b)
    assert list(oa) == [2.0, 1.0, 3.0] and list(ob) == [1.0, -0.5, -1.25]
    oa, ob = oracle.c_scan_affine(a, b, init=(1.0, 4.0))  # seed x -> x + 4
    assert list(oa) == [2.0, 1.0, 3.0] and list(ob) == [9.0, 3.5, 10.75]


def test_quaternion_fold_known_products(oracle):
    """The Hamilton product's defining identities (i*j = k, j*i = -k, i*i = j*j = k*k = i*j*k = -1),
    which fix every sign of the product that Quaternions.jl's `*` uses, and the left-to-right order of
    the fold (the reference's non-commutative scan test, test/tests/scan/scan_test.jl:22-33)."""
    one, i, j, k = np.eye(4)
    for dt in (np.float32, np.float64):
        q = lambda *rows: np.array(rows, dtype=dt)
        assert (oracle.c_scan_quat(q(i, j)) == [i, k]).all()
        assert (oracle.c_scan_quat(q(j, i)) == [j, -k]).all()
        assert (oracle.c_scan_quat(q(j, k)) == [j, i]).all()
        assert (oracle.c_scan_quat(q(k, i)) == [k, j]).all()
        assert (oracle.c_scan_quat(q(i, i)) == [i, -one]).all()
        assert (oracle.c_scan_quat(q(i, j, k)) == [i, k, -one]).all()
        assert (oracle.c_scan_quat(q(j, k), init=i) == [k, -one]).all()  # seed from the left: i*j, i*j*k
        # (1 + 2i + 3j + 4k)(5 + 6i + 7j + 8k) = -60 + 12i + 30j + 24k
        assert (oracle.c_scan_quat(q([1, 2, 3, 4], [5, 6, 7, 8]))[1] == [-60, 12, 30, 24]).all()
    rng = np.random.default_rng(8)
    x = rng.standard_normal((200, 4))
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    out = oracle.c_scan_quat(x)
    assert np.allclose(np.linalg.norm(out, axis=1), 1.0, atol=1e-12)  # unit quaternions stay on the sphere
    assert not np.allclose(out[-1], oracle.c_scan_quat(x[::-1].copy())[-1])  # order matters


def test_base_like_baseline_agrees_with_oracle(oracle):
    rng = np.random.default_rng(3)
    x = rng.random(1 << 18, dtype=np.float32)
    for threads in (1, 4):
        assert abs(oracle.base_mapreduce_add_f32(1, x, threads) - oracle.c_mapreduce(1, 0, x)) <= 1e-4 * x.size / 3
        out = oracle.base_accumulate(x, np.empty_like(x), threads)
        assert np.allclose(out, oracle.c_scan(0, 0, x), rtol=1e-3)
        u = rng.integers(0, 256, 1 << 18).astype(np.uint32)
        assert (oracle.base_accumulate(u, np.empty_like(u), threads) == np.cumsum(u, dtype=np.uint32)).all()
        for dt in (np.uint32, np.int32, np.float32):
            k = rng.standard_normal(70_001).astype(dt) if dt == np.float32 else \
                rng.integers(np.iinfo(dt).min, np.iinfo(dt).max, 70_001, dtype=dt)
            kk, v = k.copy(), np.arange(k.size, dtype=np.uint32)
            oracle.base_sort_k32(kk, v, np.empty_like(kk), np.empty_like(v), threads)
            assert (bits(kk) == bits(oracle.c_sort(k))).all()
            assert (v == oracle.c_sortperm(k)).all()


@pytest.mark.parametrize("n", range(1, 17))
def test_sort_edge_sizes_1_to_16(oracle, n):
    """test/tests/sort/sort_test.jl:94-104: every n in 1..16, UInt32 and Float32. The expected value is
    built without sorting: a known permutation of a strictly increasing sequence."""
    base_u = (np.arange(n, dtype=np.uint64) * 0x01000193 + 7).astype(np.uint32)  # strictly increasing, all bytes busy
    base_f = (np.arange(n, dtype=np.float32) - n / 2) * np.float32(1.5)          # negative, zero, positive
    perm = (np.arange(n) * 7 + 3) % n if n % 7 else np.arange(n)[::-1]
    assert sorted(perm) == list(range(n))
    assert (oracle.c_sort(base_u[perm]) == base_u).all()
    assert (bits(oracle.c_sort(base_f[perm])) == bits(base_f)).all()


def test_stability_pairs_with_about_2000_duplicates_per_key(oracle):
    """test/tests/sort/sort_test.jl:316-334: n = 200 003 keys in 0..99 (about 2000 duplicates per key),
    payload = source index. The stable order is known by construction: key k's payloads are exactly
    the positions of k, ascending."""
    n = 200_003
    keys = ((np.arange(n, dtype=np.uint64) * 2654435761) % 100).astype(np.uint32)  # a fixed, well-mixed pattern
    perm = oracle.c_sortperm(keys).astype(np.int64)
    expect = np.concatenate([np.flatnonzero(keys == k) for k in range(100)])
    assert (perm == expect).all()
    assert (np.bincount(keys, minlength=100) > 1900).all()
    sk, sv = oracle.c_sort_pairs(keys, np.arange(n, dtype=np.uint32))
    assert (sk == keys[expect]).all() and (sv == expect).all()


@pytest.mark.parametrize("op,name", [(0, "+"), (3, "max"), (2, "min")])
def test_uint8_wraparound_scan(oracle, op, name):
    """test/tests/scan/scan_test.jl:67-86: n = 10 001 UInt8 under +, max and min. For + the closed form
    is the wrapped triangular number of a ramp; max and min of a sawtooth are known by construction."""
    n = 10_001
    ramp = (np.arange(1, n + 1) % 256).astype(np.uint8)
    got = oracle.c_scan(0, op, ramp)
    if name == "+":
        exact = np.cumsum(np.arange(1, n + 1) % 256)  # int64, no wrap
        assert (got == (exact % 256).astype(np.uint8)).all()
    elif name == "max":
        assert (got[:255] == ramp[:255]).all() and (got[254:] == 255).all()
    else:
        assert (got[:255] == 1).all() and (got[255:] == 0).all()


@pytest.mark.parametrize("n", range(1, 11))
def test_scan_edge_sizes_1_to_10(oracle, n):
    """test/tests/scan/scan_test.jl:88-102: Float64 + for n = 1..10; powers of two add exactly."""
    x = np.ldexp(1.0, -np.arange(n))  # 1, 1/2, 1/4, ...
    assert (oracle.c_scan(0, 0, x) == 2.0 - np.ldexp(1.0, -np.arange(n))).all()


def test_golden_fixtures(oracle):
    """Regression freeze: the committed vectors (inputs and the oracle's own outputs at the time they were
    written) still reproduce. This checks the oracle against its past self, not against the reference."""
    path = os.path.join(GOLDEN, "golden_small.npz")
    g = np.load(path)
    assert oracle.c_mapreduce(1, 0, g["mr_x"]) == float(g["mr_abs2_sum"])
    assert (oracle.c_scan(0, 0, g["scan_u32_x"]) == g["scan_u32_out"]).all()
    assert (oracle.c_scan(0, 0, g["scan_u8_x"]) == g["scan_u8_out"]).all()
    assert np.array_equal(oracle.c_scan(0, 0, g["scan_f32_x"]), g["scan_f32_out"])
    oa, ob = oracle.c_scan_affine(g["aff_a"], g["aff_b"])
    assert np.array_equal(oa, g["aff_oa"]) and np.array_equal(ob, g["aff_ob"])
    assert (bits(oracle.c_sort(g["sort_f32_x"])) == bits(g["sort_f32_out"])).all()
    assert (oracle.c_sort(g["sort_u32_x"]) == g["sort_u32_out"]).all()
    assert (oracle.c_sortperm(g["pairs_keys"]) == g["pairs_perm"]).all()
