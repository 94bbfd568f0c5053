"""`KernelForge.argmax` / `argmin` / `argmax1d`, `findfirst` / `findlast`, `vcopy!`, `setvalue!`.

Mirrors src/search/highlevel.jl:1-52, src/search/argmax.jl:8-270, src/search/findfirst.jl:3-110 and
src/copy/copy.jl:1-55 of KernelForge.jl. Indices are 0-based here (1-based in Julia), `None` stands
for Julia's `nothing`. The relation of argmax is `">"` / `"<"` (or operator.gt / operator.lt); the
predicate of findfirst is a comparison with a scalar, written `gt(v)`, `lt(v)`, `ge(v)`, `le(v)`,
`eq(v)`, `ne(v)` (Julia: `>(v)`, `<(v)`, ...). Other closures raise ArgumentError: no fallback.
"""
from __future__ import annotations

import ctypes
import operator

import numpy as np
import torch

from . import _cabi as C
from . import ops

_RELS = {">": 1, "<": 0, operator.gt: 1, operator.lt: 0}
_NP = {C.U8: np.uint8, C.I8: np.int8, C.U16: np.uint16, C.I16: np.int16, C.U32: np.uint32, C.I32: np.int32,
       C.U64: np.uint64, C.I64: np.int64, C.F32: np.float32, C.F64: np.float64}


class Pred:
    """A comparison with a scalar: the predicates findfirst / findlast accept."""

    def __init__(self, code, value):
        self.code, self.value = code, value


def gt(v): return Pred(C.PRED_GT, v)
def lt(v): return Pred(C.PRED_LT, v)
def ge(v): return Pred(C.PRED_GE, v)
def le(v): return Pred(C.PRED_LE, v)
def eq(v): return Pred(C.PRED_EQ, v)
def ne(v): return Pred(C.PRED_NE, v)


def _host_scalar(code, value):
    arr = np.array([value]).astype(_NP[code])
    return arr, arr.ctypes.data_as(ctypes.c_void_p)


def argmax1d(f, rel, src, *, to_cpu=True, with_value=False, tmp=None):
    """Index of the first element whose f(src[i]) is extremal under `rel`; ties go to the smallest index."""
    ops.require_device_vector(src, "src")
    try:
        greater = _RELS[rel]
    except (KeyError, TypeError):
        raise C.ArgumentError("unsupported relation %r: argmax takes '>' or '<'" % (rel,)) from None
    n = src.numel()
    if n == 0:
        raise C.ArgumentError("argmax over an empty collection is not allowed")
    code = ops.dtype_code(src)
    lib = C.load()
    need = lib.kf_argmax_workspace_bytes(code, n)
    ws = tmp if tmp is not None else torch.empty(need, dtype=torch.uint8, device=src.device)
    idx = torch.empty(1, dtype=torch.int64, device=src.device)
    val = torch.empty(1, dtype=src.dtype, device=src.device)
    with ops.on_device(src.device):
        rc = lib.kf_argmax(ops.map_code(f), greater, code, src.data_ptr(), n, val.data_ptr(), idx.data_ptr(), ws.data_ptr(),
                           ws.numel(), ops.stream_handle(src))
    C.check(rc, "argmax")
    if not to_cpu:
        return (val, idx) if with_value else idx
    i = int(idx.cpu()[0])
    return (val.cpu()[0].item(), i) if with_value else i


def argmax(*args, **kw):
    """argmax(src) or argmax(rel, src)."""
    if len(args) == 1:
        return argmax1d(ops.identity, ">", args[0], **kw)
    return argmax1d(ops.identity, args[0], args[1], **kw)


def argmin(src, **kw):
    return argmax1d(ops.identity, "<", src, **kw)


def _find(pred, src, last):
    ops.require_device_vector(src, "src")
    if not isinstance(pred, Pred):
        raise C.ArgumentError("unsupported predicate %r: use gt(v), lt(v), ge(v), le(v), eq(v) or ne(v)" % (pred,))
    n = src.numel()
    code = ops.dtype_code(src)
    keep, ptr = _host_scalar(code, pred.value)
    out = torch.empty(1, dtype=torch.int64, device=src.device)
    with ops.on_device(src.device):
        rc = C.load().kf_find(pred.code, 1 if last else 0, code, src.data_ptr(), n, ptr, out.data_ptr(), ops.stream_handle(src))
    C.check(rc, "findfirst")
    r = int(out.cpu()[0])
    if last:
        return None if r == 0 else r - 1
    return None if r < 0 or r >= n else r


def findfirst(pred, src):
    """Index of the first element satisfying the predicate, or None."""
    return _find(pred, src, False)


def findlast(pred, src):
    """Index of the last element satisfying the predicate, or None."""
    return _find(pred, src, True)


def vcopy_(dst, src):
    """`vcopy!(dst, src)`: vectorised device copy."""
    ops.require_device_vector(src, "src")
    ops.require_device_vector(dst, "dst")
    if dst.dtype != src.dtype or dst.numel() != src.numel():
        raise C.ArgumentError("dst and src must have the same element type and length")
    with ops.on_device(src.device):
        rc = C.load().kf_vcopy(dst.data_ptr(), src.data_ptr(), src.numel() * src.element_size(), ops.stream_handle(src))
    C.check(rc, "vcopy!")
    return dst


def setvalue_(dst, value):
    """`setvalue!(dst, val)`: vectorised fill."""
    ops.require_device_vector(dst, "dst")
    code = ops.dtype_code(dst)
    keep, ptr = _host_scalar(code, value)
    with ops.on_device(dst.device):
        rc = C.load().kf_setvalue(code, dst.data_ptr(), dst.numel(), ptr, ops.stream_handle(dst))
    C.check(rc, "setvalue!")
    return dst
