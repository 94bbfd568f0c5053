"""numpy-facing wrapper of the CPU oracle (libkf_oracle.so) plus an independent numpy restatement.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by bench.py's CPU-baseline leg;
never by the product package. Build the library with `make -C oracle`.

Two implementations of every oracle function live here so that each pins the other:
  * `c_*`  — calls into kf_oracle.c (fast enough for millions of elements);
  * `np_*` — the same semantics written with numpy primitives (float64 cumsum / reduce,
             stable argsort of the mapped unsigned keys).
The semantics restated are those of Julia `Base` as used by the reference's tests (see the header
of kf_oracle.c for the citations).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_double, c_float, c_int, c_int64, c_size_t, c_uint64, c_void_p

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libkf_oracle.so")

U8, I8, U16, I16, U32, I32, U64, I64, F32, F64 = range(10)
MAP_IDENTITY, MAP_ABS2, MAP_ABS = range(3)
OP_ADD, OP_MUL, OP_MIN, OP_MAX, OP_AND, OP_OR, OP_XOR = range(7)

DTYPE_CODE = {np.dtype(k): v for k, v in {
    "uint8": U8, "int8": I8, "uint16": U16, "int16": I16, "uint32": U32, "int32": I32,
    "uint64": U64, "int64": I64, "float32": F32, "float64": F64}.items()}

_lib = None


def build() -> str:
    """Compiles libkf_oracle.so with the committed Makefile."""
    subprocess.run(["make", "-C", HERE], check=True, capture_output=True)
    return LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        src = os.path.join(HERE, "kf_oracle.c")
        if not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
            build()
        L = ctypes.CDLL(LIB_PATH)
        L.kfo_max_threads.restype = c_int
        L.kfo_mapreduce_f32.restype = c_double
        L.kfo_mapreduce_f32.argtypes = [c_int, c_int, c_void_p, c_size_t]
        L.kfo_mapreduce_f64.restype = c_double
        L.kfo_mapreduce_f64.argtypes = [c_int, c_int, c_void_p, c_size_t]
        L.kfo_scan_f32.argtypes = [c_int, c_int, c_void_p, c_size_t, POINTER(c_double), c_void_p]
        L.kfo_scan_f64.argtypes = [c_int, c_int, c_void_p, c_size_t, POINTER(c_double), c_void_p]
        L.kfo_scan_affine.argtypes = [c_void_p, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p]
        L.kfo_scan_quat.argtypes = [c_void_p, c_int, c_size_t, c_void_p, c_void_p]
        L.kfo_mapreduce_int.restype = c_int64
        L.kfo_mapreduce_int.argtypes = [c_int, c_int, c_int, c_void_p, c_size_t]
        L.kfo_scan_int.argtypes = [c_int, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p]
        L.kfo_uint_map.restype = c_uint64
        L.kfo_uint_map.argtypes = [c_int, c_uint64]
        L.kfo_sort_perm.restype = c_int
        L.kfo_sort_perm.argtypes = [c_int, c_void_p, c_size_t, c_void_p]
        L.kfo_gather.argtypes = [c_void_p, c_void_p, c_size_t, c_int, c_void_p]
        L.kfb_mapreduce_add_f32.restype = c_float
        L.kfb_mapreduce_add_f32.argtypes = [c_int, c_void_p, c_size_t, c_int]
        L.kfb_accumulate_f32.argtypes = [c_void_p, c_size_t, c_void_p, c_int]
        L.kfb_accumulate_u32.argtypes = [c_void_p, c_size_t, c_void_p, c_int]
        L.kfb_accumulate_affine_f32.argtypes = [c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]
        L.kfb_sort_k32.argtypes = [c_int, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p, c_int]
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(c_void_p)


def _c(a) -> np.ndarray:
    return np.ascontiguousarray(a)


# ---- C oracle -----------------------------------------------------------------------------------
def c_mapreduce(f: int, op: int, x: np.ndarray):
    """Float inputs: Float64 left fold (python float). Integer inputs: wrapped in the element type."""
    x = _c(x)
    if x.size == 0:
        raise ValueError("reducing over an empty collection is not allowed")
    if x.dtype == np.float32:
        return lib().kfo_mapreduce_f32(f, op, _p(x), x.size)
    if x.dtype == np.float64:
        return lib().kfo_mapreduce_f64(f, op, _p(x), x.size)
    code = DTYPE_CODE[x.dtype]
    v = lib().kfo_mapreduce_int(f, op, code, _p(x), x.size)
    return np.array([v], dtype=np.int64).astype(x.dtype)[0] if x.dtype != np.uint64 else np.uint64(v & (2**64 - 1))


def c_scan(f: int, op: int, x: np.ndarray, init=None) -> np.ndarray:
    """Inclusive scan. Float inputs return float64 (the Float64 left fold); integers wrap in dtype."""
    x = _c(x)
    if x.dtype in (np.float32, np.float64):
        out = np.empty(x.size, dtype=np.float64)
        ini = ctypes.byref(c_double(float(init))) if init is not None else None
        (lib().kfo_scan_f32 if x.dtype == np.float32 else lib().kfo_scan_f64)(f, op, _p(x), x.size, ini, _p(out))
        return out
    out = np.empty_like(x)
    ini = _p(np.array([init], dtype=x.dtype)) if init is not None else None
    lib().kfo_scan_int(f, op, DTYPE_CODE[x.dtype], _p(x), x.size, ini, _p(out))
    return out


def c_scan_affine(a: np.ndarray, b: np.ndarray, init=None):
    a, b = _c(a.astype(np.float32, copy=False)), _c(b.astype(np.float32, copy=False))
    oa, ob = np.empty(a.size, np.float64), np.empty(a.size, np.float64)
    ini = _p(np.array(init, dtype=np.float64)) if init is not None else None
    lib().kfo_scan_affine(_p(a), _p(b), a.size, ini, _p(oa), _p(ob))
    return oa, ob


def c_scan_quat(q: np.ndarray, init=None) -> np.ndarray:
    """accumulate(*, q) for an [n, 4] Float32/Float64 array of (w, x, y, z); Float64 result."""
    q = _c(q)
    assert q.ndim == 2 and q.shape[1] == 4 and q.dtype in (np.float32, np.float64)
    out = np.empty(q.shape, np.float64)
    ini = np.array(init, dtype=np.float64) if init is not None else None
    lib().kfo_scan_quat(_p(q), 1 if q.dtype == np.float64 else 0, q.shape[0], _p(ini) if ini is not None else None, _p(out))
    return out


def c_sortperm(keys: np.ndarray) -> np.ndarray:
    """Stable permutation (0-based) that sorts `keys` by the reference's uint_map order."""
    keys = _c(keys)
    perm = np.empty(keys.size, dtype=np.uint64)
    if lib().kfo_sort_perm(DTYPE_CODE[keys.dtype], _p(keys), keys.size, _p(perm)) != 0:
        raise MemoryError("oracle sort ran out of memory")
    return perm


def c_sort(keys: np.ndarray) -> np.ndarray:
    return _c(keys)[c_sortperm(keys).astype(np.int64)]


def c_sort_pairs(keys: np.ndarray, vals: np.ndarray):
    p = c_sortperm(keys).astype(np.int64)
    return _c(keys)[p], _c(vals)[p]


# ---- independent numpy restatement ---------------------------------------------------------------
def np_uint_map(keys: np.ndarray) -> np.ndarray:
    """Order-preserving unsigned image of the keys (uint_map.jl:11-35)."""
    k = _c(keys)
    bits = k.dtype.itemsize * 8
    u = k.view("uint%d" % bits)
    sign = np.array(1 << (bits - 1), dtype=u.dtype)
    if k.dtype.kind == "u":
        return u.copy()
    if k.dtype.kind == "i":
        return u ^ sign
    neg = (u & sign) != 0
    return np.where(neg, ~u, u | sign)


def np_sortperm(keys: np.ndarray) -> np.ndarray:
    return np.argsort(np_uint_map(keys), kind="stable")


def np_sort(keys: np.ndarray) -> np.ndarray:
    return _c(keys)[np_sortperm(keys)]


_NP_OPS = {OP_ADD: np.add, OP_MUL: np.multiply, OP_MIN: np.minimum, OP_MAX: np.maximum,
           OP_AND: np.bitwise_and, OP_OR: np.bitwise_or, OP_XOR: np.bitwise_xor}


def np_map(f: int, x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        if f == MAP_ABS2:
            return x * x
        if f == MAP_ABS:
            return np.abs(x)
    return x


def np_scan(f: int, op: int, x: np.ndarray) -> np.ndarray:
    x = _c(x)
    y = np_map(f, x.astype(np.float64) if x.dtype.kind == "f" else x)
    with np.errstate(over="ignore"):
        return _NP_OPS[op].accumulate(y, dtype=y.dtype)  # keep the element type: integers wrap


def np_mapreduce(f: int, op: int, x: np.ndarray):
    return np_scan(f, op, x)[-1]


MAPN_PROD, MAPN_SQDIFF, MAPN_WSQ = range(3)


def np_mapreduce_multi(fn: int, op: int, arrays, post_sqrt: bool = False):
    """Tuple form mapreduce(f, op, (x1, ..., xk)) as the reference's tests state it
    (test/tests/mapreduce/mapreduce1d_test.jl:106-194): floats are mapped and folded in Float64,
    integers in the element type (wrapping)."""
    xs = [_c(a) for a in arrays]
    if xs[0].dtype.kind == "f":
        xs = [a.astype(np.float64) for a in xs]
    with np.errstate(over="ignore"):
        if fn == MAPN_SQDIFF:
            m = (xs[0] - xs[1]) * (xs[0] - xs[1])
        elif fn == MAPN_WSQ:
            m = xs[0] * xs[1] * xs[1]
        else:
            m = xs[0].copy()
            for a in xs[1:]:
                m = m * a
        r = _NP_OPS[op].reduce(m, dtype=m.dtype)
    return np.sqrt(r) if post_sqrt else r


# ---- timed CPU baseline (Base-like) ----------------------------------------------------------------
def max_threads() -> int:
    return int(lib().kfo_max_threads())


def base_mapreduce_add_f32(f: int, x: np.ndarray, threads: int = 1) -> float:
    return float(lib().kfb_mapreduce_add_f32(f, _p(x), x.size, threads))


def base_accumulate(x: np.ndarray, out: np.ndarray, threads: int = 1) -> np.ndarray:
    fn = lib().kfb_accumulate_f32 if x.dtype == np.float32 else lib().kfb_accumulate_u32
    fn(_p(x), x.size, _p(out), threads)
    return out


def base_accumulate_affine(a, b, oa, ob):
    lib().kfb_accumulate_affine_f32(_p(a), _p(b), a.size, _p(oa), _p(ob))
    return oa, ob


def base_sort_k32(keys: np.ndarray, vals, tmp_k: np.ndarray, tmp_v, threads: int = 1) -> None:
    """In-place LSD radix sort of 4-byte keys (uint32 / int32 / float32), optional 4-byte payload."""
    lib().kfb_sort_k32(DTYPE_CODE[keys.dtype], _p(keys), _p(vals) if vals is not None else None, keys.size,
                       _p(tmp_k), _p(tmp_v) if tmp_v is not None else None, threads)
