"""GPU tests of argmax / argmin, findfirst / findlast, vcopy! and setvalue! through the C ABI.

Mirror test/tests/search/argmax_test.jl (basic, argmin, first-index tie-breaking, large arrays),
test/tests/search/findfirst_test.jl (first / last position, no match, empty, single element, NaN,
sizes around a workgroup, many blocks) and test/tests/copy/copy_test.jl of KernelForge.jl. The
checker is numpy (`np.argmax` / `np.argmin` return the first extremal index, as the reference does).
Indices are 0-based here.
"""
import numpy as np
import pytest
import torch

from util import to_dev, to_host

pytestmark = pytest.mark.gpu


def test_argmax_basic_and_ties(kf):
    cases = [([5.0, 1, 2, 3], 0, 1), ([1.0, 5, 2, 3], 1, 0), ([3.0, 1, 4, 1, 5], 4, 1), ([2.0, 2, 2], 0, 0),
             ([1.0, 3, 3, 2], 1, 0), ([4.0, 1, 1, 4], 0, 1)]
    for data, imax, imin in cases:
        x = to_dev(np.array(data, dtype=np.float32))
        assert kf.argmax(">", x) == imax and kf.argmax(x) == imax
        assert kf.argmax("<", x) == imin and kf.argmin(x) == imin
    assert kf.argmax(to_dev(np.array([7], dtype=np.int32))) == 0
    with pytest.raises(kf.ArgumentError):
        kf.argmax(to_dev(np.array([], dtype=np.float32)))
    with pytest.raises(kf.ArgumentError):
        kf.argmax(lambda a, b: a != b, to_dev(np.array([1.0])))


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.int32, np.uint8, np.int64, np.int16])
@pytest.mark.parametrize("n", [33, 1000, 10_001, 1_000_003])
def test_argmax_types_sizes(kf, dtype, n):
    rng = np.random.default_rng(n)
    if np.dtype(dtype).kind == "f":
        x = rng.standard_normal(n).astype(dtype)
    else:
        info = np.iinfo(dtype)
        x = rng.integers(max(info.min, -1000), min(info.max, 1000), n).astype(dtype)  # many ties
    d = to_dev(x)
    assert kf.argmax(d) == int(np.argmax(x))
    assert kf.argmin(d) == int(np.argmin(x))
    v, i = kf.argmax1d(kf.identity, ">", d, with_value=True)
    assert i == int(np.argmax(x)) and v == x.max()
    if np.dtype(dtype).kind == "f" or np.dtype(dtype).kind == "i":
        ax = np.abs(x.astype(np.float64)) if np.dtype(dtype).kind == "f" else np.abs(x.astype(np.int64))
        if np.dtype(dtype).kind == "f" or ax.max() <= np.iinfo(dtype).max:
            assert kf.argmax1d("abs", "<", d) == int(np.argmin(ax))
    off = to_dev(np.concatenate([np.zeros(3, dtype), x]))[3:]  # a view that starts off a 16-byte boundary
    assert kf.argmax(off) == int(np.argmax(x))


def test_argmax_ties_and_nans_at_scale(kf):
    """Ties across vectors, threads and CTAs go to the smallest index (the kernel keeps a value and the
    vector that held it per thread and resolves the element afterwards); a NaN never wins against a
    number, wherever it sits, and an all-NaN array answers its first index."""
    n = 5_000_017
    rng = np.random.default_rng(21)
    for dtype in (np.float32, np.int8, np.uint16, np.float64):
        x = rng.integers(0, 50, n).astype(dtype)  # thousands of ties for the maximum and the minimum
        for off in (0, 1, 3):
            assert kf.argmax(to_dev(x)[off:]) == int(np.argmax(x[off:]))
            assert kf.argmin(to_dev(x)[off:]) == int(np.argmin(x[off:]))
        if dtype != np.int8:  # (squares of Int8 values wrap around in the element type)
            assert kf.argmax1d(kf.abs2, ">", to_dev(x)) == int(np.argmax(x.astype(np.float64) ** 2))
    y = rng.random(n).astype(np.float32)
    y[::97] = np.nan
    y[0] = np.nan
    want_max = int(np.nanargmax(y))
    want_min = int(np.nanargmin(y))
    assert kf.argmax(to_dev(y)) == want_max and kf.argmin(to_dev(y)) == want_min
    y[want_max + 1:want_max + 5] = y[want_max]  # later ties, with NaNs in between
    assert kf.argmax(to_dev(y)) == want_max
    assert kf.argmax(to_dev(np.full(100_000, np.nan, dtype=np.float32))) == 0


def test_argmax_extreme_positions(kf):
    n = 3_000_001
    x = np.zeros(n, dtype=np.float32)
    for pos in (0, 9, n // 2, n - 1):
        y = x.copy()
        y[pos] = 1.0
        assert kf.argmax(to_dev(y)) == pos
        assert kf.argmin(to_dev(-y)) == pos
    assert kf.argmax(to_dev(np.full(1000, -np.inf, dtype=np.float32))) == 0


def test_findfirst_and_findlast(kf):
    x = to_dev(np.array([5, 1, 2, 3], dtype=np.int32))
    assert kf.findfirst(kf.eq(5), x) == 0 and kf.findfirst(kf.eq(3), x) == 3
    assert kf.findfirst(kf.gt(10), x) is None and kf.findlast(kf.gt(10), x) is None
    assert kf.findfirst(kf.gt(0), x) == 0 and kf.findlast(kf.gt(0), x) == 3
    assert kf.findfirst(kf.eq(1), to_dev(np.array([], dtype=np.int32))) is None
    assert kf.findfirst(kf.eq(1), to_dev(np.array([1], dtype=np.int32))) == 0
    assert kf.findfirst(kf.eq(2), to_dev(np.array([1], dtype=np.int32))) is None
    f = to_dev(np.array([np.nan, 1.0, np.nan], dtype=np.float32))
    assert kf.findfirst(kf.eq(1.0), f) == 1 and kf.findfirst(kf.eq(float("nan")), f) is None  # NaN != NaN
    assert kf.findfirst(kf.lt(-0.5), to_dev(np.array([0.0, -0.25, -0.75, -1.0], dtype=np.float32))) == 2
    for n, pos in ((255, 254), (256, 15), (257, 32), (100_000, 699), (5_000_000, 4_999_999), (5_000_000, 0)):
        y = np.zeros(n, dtype=np.int32)
        y[pos] = 9
        assert kf.findfirst(kf.eq(9), to_dev(y)) == pos and kf.findlast(kf.ne(0), to_dev(y)) == pos
    rng = np.random.default_rng(3)
    z = rng.random(4_000_003).astype(np.float32)
    hits = np.nonzero(z > 0.9999)[0]
    assert kf.findfirst(kf.gt(0.9999), to_dev(z)) == int(hits[0])
    assert kf.findlast(kf.gt(0.9999), to_dev(z)) == int(hits[-1])
    assert kf.findfirst(kf.ge(2.0), to_dev(z)) is None
    with pytest.raises(kf.ArgumentError):
        kf.findfirst(lambda v: v > 1, to_dev(z))


@pytest.mark.parametrize("dtype,n", [(np.float32, 1024), (np.uint8, 1000), (np.float64, 12_345), (np.int16, 1_000_001),
                                     (np.uint8, 7), (np.int64, 1)])
def test_vcopy_and_setvalue(kf, dtype, n):
    rng = np.random.default_rng(n)
    x = (rng.random(n) * 200).astype(dtype)
    src = to_dev(x)
    dst = torch.zeros_like(src)
    kf.vcopy_(dst, src)
    assert (to_host(dst) == x).all()
    if n > 8:  # views: same misalignment (vector path with head and tail) and different (element-wise path)
        big = torch.zeros(n + 8, dtype=src.dtype, device="cuda")
        kf.vcopy_(big[3:n - 1], src[:n - 4])
        assert (to_host(big[3:n - 1]) == x[: n - 4]).all() and to_host(big[:3]).sum() == 0 and to_host(big[n - 1:]).sum() == 0
        big.zero_()
        kf.vcopy_(big[1:n - 3], src[1:n - 3])
        assert (to_host(big[1:n - 3]) == x[1:n - 3]).all() and to_host(big[0:1]).sum() == 0 and to_host(big[n - 3:]).sum() == 0
    val = np.array([37]).astype(dtype)[0]
    kf.setvalue_(dst, val)
    assert (to_host(dst) == val).all()
    if n > 8:
        big = torch.zeros(n + 8, dtype=src.dtype, device="cuda")
        kf.setvalue_(big[3:n + 1], val)
        h = to_host(big)
        assert (h[3:n + 1] == val).all() and h[:3].sum() == 0 and h[n + 1:].sum() == 0
    with pytest.raises(kf.ArgumentError):
        kf.vcopy_(dst[:-1] if n > 1 else torch.zeros(2, dtype=src.dtype, device="cuda"), src)


def test_vcopy_is_the_copy_yardstick(kf):
    """n = 2^28 Float32: the copy must reproduce the input exactly (checked by checksums)."""
    n = 1 << 28
    src = torch.rand(n, dtype=torch.float32, device="cuda")
    dst = torch.empty_like(src)
    kf.vcopy_(dst, src)
    assert torch.equal(dst, src)
