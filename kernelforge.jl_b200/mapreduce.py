"""`KernelForge.mapreduce` / `mapreduce!` for full (dims=nothing) reductions.

Mirrors src/mapreduce/mapreduce.jl:51-62,151-162 and src/mapreduce/1D/mapreduce1d.jl:177-288 of
KernelForge.jl. The reduction runs in one kernel launch of libkf_b200.so; the value comes back
through a one-element device array exactly as in the reference (`Array(dst)[1]`).
"""
from __future__ import annotations

import torch

from . import _cabi as C
from . import ops
from .allocations import MapReduce1D, mapreduce_bytes, resolve_tmp


def _check_common(dims, src):
    if dims is not None and dims != slice(None):
        raise C.ArgumentError("only full reductions (dims=nothing) are implemented by this library")
    if isinstance(src, (tuple, list)):
        if len(src) == 1:
            src = src[0]
        else:
            return _check_tuple(src)
    ops.require_device_vector(src, "src")
    return src


def _check_tuple(srcs):
    """The tuple form mapreduce(f, op, (x, y, ...)) (src/mapreduce/1D/mapreduce1d.jl:177-288)."""
    if not 2 <= len(srcs) <= 4:
        raise C.ArgumentError("the tuple form takes 2 to 4 arrays, got %d" % len(srcs))
    for i, t in enumerate(srcs):
        ops.require_device_vector(t, "src[%d]" % i)
        if t.dtype != srcs[0].dtype or t.numel() != srcs[0].numel() or t.device != srcs[0].device:
            raise C.ArgumentError("the arrays of the tuple form must agree in element type, length and device")
    return tuple(srcs)


def _mapreduce_tuple(f, op, dst, srcs, g, tmp, cfg):
    import ctypes

    first = srcs[0]
    fcode, opcode, gcode = ops.mapn_code(f), ops.op_code(op), ops.post_code(g)
    if opcode not in (C.OP_ADD, C.OP_MUL, C.OP_MIN, C.OP_MAX):
        raise C.ArgumentError("the tuple form supports +, *, min and max")
    n = first.numel()
    if n == 0:
        raise C.ArgumentError("reducing over an empty collection is not allowed")
    buf = resolve_tmp(tmp, MapReduce1D, mapreduce_bytes(first, cfg), first.device)
    ptrs = (ctypes.c_void_p * len(srcs))(*[t.data_ptr() for t in srcs])
    with ops.on_device(first.device):
        rc = C.load().kf_mapreduce_multi(fcode, opcode, gcode, ops.dtype_code(first), ptrs, len(srcs), n, dst.data_ptr(),
                                         buf.ptr(), buf.nbytes, cfg, ops.stream_handle(first))
    C.check(rc, "mapreduce")
    return dst


def mapreduce_(f, op, dst, src, *, dims=None, g=ops.identity, tmp=None, Nitem=None, workgroup=None,
               blocks=None, arch=None):
    """`mapreduce!(f, op, dst, src)`: dst[0] = g(op-reduce of f over src). Returns dst (asynchronous)."""
    src = _check_common(dims, src)
    ops.require_device_vector(dst, "dst")
    if isinstance(src, tuple):
        if dst.dtype != src[0].dtype or dst.numel() < 1:
            raise C.ArgumentError("dst must hold one element of the arrays' element type")
        return _mapreduce_tuple(f, op, dst, src, g, tmp, C.make_cfg(workgroup, Nitem, blocks))
    if dst.dtype != src.dtype:
        raise C.ArgumentError("dst must have the element type of f(src) (%s), got %s" % (src.dtype, dst.dtype))
    if dst.numel() < 1:
        raise C.ArgumentError("dst must hold at least one element")
    fcode, opcode, gcode = ops.map_code(f), ops.op_code(op), ops.post_code(g)
    if opcode == C.OP_AFFINE:
        raise C.ArgumentError("AffineCompose is not commutative: mapreduce combines in strided order; use scan")
    n = src.numel()
    if n == 0:
        raise C.ArgumentError("reducing over an empty collection is not allowed")
    cfg = C.make_cfg(workgroup, Nitem, blocks)
    buf = resolve_tmp(tmp, MapReduce1D, mapreduce_bytes(src, cfg), src.device)
    with ops.on_device(src.device):
        rc = C.load().kf_mapreduce(fcode, opcode, gcode, ops.dtype_code(src), src.data_ptr(), n, dst.data_ptr(),
                                   buf.ptr(), buf.nbytes, cfg, ops.stream_handle(src))
    C.check(rc, "mapreduce")
    return dst


def mapreduce(f, op, src, *, dims=None, g=ops.identity, tmp=None, Nitem=None, workgroup=None, blocks=None,
              arch=None, to_cpu=True):
    """`mapreduce(f, op, src; g)`: the reduced value as a host scalar (or a 1-element device tensor)."""
    s = _check_common(dims, src)
    first = s[0] if isinstance(s, tuple) else s
    dst = torch.empty(1, dtype=first.dtype, device=first.device)
    mapreduce_(f, op, dst, s, g=g, tmp=tmp, Nitem=Nitem, workgroup=workgroup, blocks=blocks, arch=arch)
    return dst.cpu()[0].item() if to_cpu else dst


# The reference's 1-D names (src/mapreduce/1D/mapreduce1d.jl:177-288).
mapreduce1d = mapreduce
mapreduce1d_ = mapreduce_
