"""Closure -> enum mapping and dtype tables.

The reference compiles arbitrary Julia closures into its kernels. This library has a fixed
operator set; the host layer recognises the supported functions by identity and raises
`ArgumentError` for anything else (no fallback). Julia names map as follows:

    identity -> identity     abs2 -> abs2     abs -> abs / builtins.abs
    +  -> operator.add       *  -> operator.mul      min / max -> builtins.min / max
    &  -> operator.and_      |  -> operator.or_      xor (⊻) -> operator.xor
    sqrt (as g) -> math.sqrt / sqrt
    (a, b, ...) -> a*b*...  -> prod / operator.mul     (a, b) -> (a-b)^2 -> sqdiff     (w, x) -> w*x*x -> wsq
    AffineCompose() -> the non-commutative composition of affine maps (new in this library)
    QuaternionMul() -> the Hamilton product on [n, 4] arrays (`*` on a Quaternion array in the reference)

Strings ("+", "min", "abs2", ...) are accepted as well.
"""
from __future__ import annotations

import builtins
import contextlib
import math
import operator

import torch

from . import _cabi as C


def identity(x):
    """Julia's `identity`."""
    return x


def abs2(x):
    """Julia's `abs2` for real numbers: x*x."""
    return x * x


def sqrt(x):
    """Julia's `sqrt` (usable as the post-map `g` of mapreduce)."""
    return math.sqrt(x)


def prod(*xs):
    """Map over a tuple of arrays: x1*x2*...*xk (`(a, b) -> a * b` is the dot product)."""
    r = xs[0]
    for x in xs[1:]:
        r = r * x
    return r


def sqdiff(a, b):
    """Map over two arrays: (a - b)^2."""
    return (a - b) * (a - b)


def wsq(w, x):
    """Map over two arrays: w * x * x (weighted sum of squares)."""
    return w * x * x


class AffineCompose:
    """Operator singleton: (a1,b1) ∘ (a2,b2) = (a1*a2, a2*b1 + b2) on Float32 pairs.

    Composition of the affine maps x -> a*x + b, left map applied first. Associative, not
    commutative. Usable with `scan` / `scan_` only.
    """

    _inst = None

    def __new__(cls):
        if cls._inst is None:
            cls._inst = super().__new__(cls)
        return cls._inst

    def __call__(self, l, r):
        return (l[0] * r[0], r[0] * l[1] + r[1])

    def __repr__(self):
        return "AffineCompose()"


class QuaternionMul:
    """Operator singleton: the Hamilton product of quaternions stored as [n, 4] Float32 or Float64
    arrays of (w, x, y, z). Associative, not commutative: the operator of the reference's
    non-commutative scan test (test/tests/scan/scan_test.jl:22-33 of KernelForge.jl, where it is `*`
    on a QuaternionF64 array). Usable with `scan` / `scan_` only.
    """

    _inst = None

    def __new__(cls):
        if cls._inst is None:
            cls._inst = super().__new__(cls)
        return cls._inst

    def __call__(self, l, r):
        lw, lx, ly, lz = l
        rw, rx, ry, rz = r
        return (lw * rw - lx * rx - ly * ry - lz * rz, lw * rx + lx * rw + ly * rz - lz * ry,
                lw * ry - lx * rz + ly * rw + lz * rx, lw * rz + lx * ry - ly * rx + lz * rw)

    def __repr__(self):
        return "QuaternionMul()"


_MAPS = {identity: C.MAP_IDENTITY, abs2: C.MAP_ABS2, builtins.abs: C.MAP_ABS, operator.abs: C.MAP_ABS,
         torch.abs: C.MAP_ABS, "identity": C.MAP_IDENTITY, "abs2": C.MAP_ABS2, "abs": C.MAP_ABS, None: C.MAP_IDENTITY}
_OPS = {operator.add: C.OP_ADD, operator.mul: C.OP_MUL, builtins.min: C.OP_MIN, builtins.max: C.OP_MAX,
        operator.and_: C.OP_AND, operator.or_: C.OP_OR, operator.xor: C.OP_XOR,
        torch.add: C.OP_ADD, torch.mul: C.OP_MUL, torch.minimum: C.OP_MIN, torch.maximum: C.OP_MAX,
        "+": C.OP_ADD, "*": C.OP_MUL, "min": C.OP_MIN, "max": C.OP_MAX, "&": C.OP_AND, "|": C.OP_OR,
        "xor": C.OP_XOR, "⊻": C.OP_XOR}
_POSTS = {identity: C.POST_IDENTITY, math.sqrt: C.POST_SQRT, sqrt: C.POST_SQRT, torch.sqrt: C.POST_SQRT,
          "identity": C.POST_IDENTITY, "sqrt": C.POST_SQRT, None: C.POST_IDENTITY}


_MAPNS = {prod: C.MAPN_PROD, operator.mul: C.MAPN_PROD, torch.mul: C.MAPN_PROD, "prod": C.MAPN_PROD, "*": C.MAPN_PROD,
          sqdiff: C.MAPN_SQDIFF, "sqdiff": C.MAPN_SQDIFF, wsq: C.MAPN_WSQ, "wsq": C.MAPN_WSQ}


def _lookup(table, fn, what):
    try:
        if fn in table:
            return table[fn]
    except TypeError:
        pass
    raise C.ArgumentError(
        "unsupported %s %r: this library implements a fixed operator set (see kernelforge ops) "
        "and has no fallback for other closures" % (what, fn))


def map_code(f) -> int:
    return _lookup(_MAPS, f, "map function f")


def mapn_code(f) -> int:
    return _lookup(_MAPNS, f, "map function f over a tuple of arrays")


def op_code(op) -> int:
    if isinstance(op, AffineCompose):
        return C.OP_AFFINE
    return _lookup(_OPS, op, "operator op")


def post_code(g) -> int:
    return _lookup(_POSTS, g, "post-map g")


DTYPES = {
    torch.uint8: C.U8, torch.int8: C.I8, torch.int16: C.I16, torch.int32: C.I32, torch.int64: C.I64,
    torch.float32: C.F32, torch.float64: C.F64, torch.bool: C.U8,
}
for _name, _code in (("uint16", C.U16), ("uint32", C.U32), ("uint64", C.U64)):
    if hasattr(torch, _name):
        DTYPES[getattr(torch, _name)] = _code

DTYPE_BYTES = {C.U8: 1, C.I8: 1, C.U16: 2, C.I16: 2, C.U32: 4, C.I32: 4, C.U64: 8, C.I64: 8, C.F32: 4, C.F64: 8}


def dtype_code(t: torch.Tensor) -> int:
    try:
        return DTYPES[t.dtype]
    except KeyError:
        raise C.ArgumentError("unsupported element type %s" % t.dtype) from None


def require_device_vector(t, name: str) -> None:
    """Dense device storage is required, as for the reference's arrays (views with an offset are fine)."""
    if not isinstance(t, torch.Tensor):
        raise C.ArgumentError("%s must be a torch.Tensor on a CUDA device" % name)
    if not t.is_cuda:
        raise C.ArgumentError("%s must live on a CUDA device; there is no CPU path" % name)
    if not t.is_contiguous():
        raise C.ArgumentError("%s must be contiguous (dense views only)" % name)


_NO_SWITCH = contextlib.nullcontext()


def on_device(device):
    """Context in which `device` is the current CUDA device. The common case, where it already is,
    costs one query instead of torch's save / set / restore sequence."""
    if device.index is None or torch.cuda.current_device() == device.index:
        return _NO_SWITCH
    return torch.cuda.device(device)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_handle(t: torch.Tensor) -> int:
    """The cudaStream_t of torch's current stream on the tensor's device."""
    if _raw_stream is not None and t.device.index is not None:
        return _raw_stream(t.device.index)  # one C call; torch.cuda.current_stream builds a Stream object (~7 us)
    return torch.cuda.current_stream(t.device).cuda_stream
