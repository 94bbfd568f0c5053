"""Helpers shared by the GPU parity tests."""
import math

import numpy as np
import torch

NP2TORCH = {
    np.dtype("uint8"): torch.uint8, np.dtype("int8"): torch.int8, np.dtype("int16"): torch.int16,
    np.dtype("int32"): torch.int32, np.dtype("int64"): torch.int64, np.dtype("float32"): torch.float32,
    np.dtype("float64"): torch.float64, np.dtype("uint16"): torch.uint16, np.dtype("uint32"): torch.uint32,
    np.dtype("uint64"): torch.uint64,
}


def to_dev(a: np.ndarray, offset: int = 0) -> torch.Tensor:
    """Host array -> device tensor of the same dtype. `offset` > 0 returns a view that starts
    `offset` elements into a larger buffer (an unaligned base pointer, like view(x, 2:n))."""
    a = np.ascontiguousarray(a)
    tdt = NP2TORCH[a.dtype]
    signed = {torch.uint16: np.int16, torch.uint32: np.int32, torch.uint64: np.int64}
    if tdt in signed:  # torch cannot always copy unsigned numpy arrays directly: go through the bits
        t = torch.from_numpy(a.view(signed[tdt])).cuda().view(tdt)
    else:
        t = torch.from_numpy(a).cuda()
    if offset:
        big = torch.empty(a.size + offset, dtype=tdt, device="cuda")
        v = big[offset:]
        v.copy_(t)
        return v
    return t


def to_host(t: torch.Tensor) -> np.ndarray:
    back = {torch.uint16: (torch.int16, np.uint16), torch.uint32: (torch.int32, np.uint32),
            torch.uint64: (torch.int64, np.uint64)}
    if t.dtype in back:
        s, u = back[t.dtype]
        return t.view(s).cpu().numpy().view(u)
    return t.cpu().numpy()


def scan_tol(n: int) -> float:
    """Relative tolerance of Float32 reductions and scans against the Float64 oracle: 1e-5*log2(n)."""
    return 1e-5 * max(1.0, math.log2(max(n, 2)))


def assert_close_rel(got: np.ndarray, ref: np.ndarray, n: int, floor: float = 0.0):
    """|got - ref| <= tol * max(|ref|, floor), element-wise, tol = 1e-5*log2(n)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    tol = scan_tol(n)
    bound = tol * np.maximum(np.abs(ref), floor)
    err = np.abs(got - ref)
    bad = err > bound
    assert not bad.any(), "max rel err %.3e at %d (tol %.3e)" % (
        float((err / np.maximum(np.abs(ref), max(floor, 1e-300))).max()), int(np.argmax(err - bound)), tol)


def bits(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a).view("uint%d" % (a.dtype.itemsize * 8))


def pow2_factors(n: int, rng, dtype) -> np.ndarray:
    """Mostly 1.0 with up to 60 factors of 2.0 or 0.5: every product of any subset, in any
    association order, is an exact power of two within 2^+-60, so `*` can be checked bit for bit."""
    x = np.ones(n, dtype=dtype)
    k = min(60, n)
    pos = rng.choice(n, size=k, replace=False)
    x[pos] = np.where(rng.integers(0, 2, k) == 0, 2.0, 0.5).astype(dtype)
    return x
