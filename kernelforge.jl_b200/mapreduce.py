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
        if len(src) != 1:
            raise C.ArgumentError("multi-array mapreduce is not implemented by this library")
        src = src[0]
    ops.require_device_vector(src, "src")
    return src


def mapreduce_(f, op, dst, src, *, dims=None, g=ops.identity, tmp=None, Nitem=None, workgroup=None,
               blocks=None, arch=None):
    """`mapreduce!(f, op, dst, src)`: dst[0] = g(op-reduce of f over src). Returns dst (asynchronous)."""
    src = _check_common(dims, src)
    ops.require_device_vector(dst, "dst")
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
    with torch.cuda.device(src.device):
        rc = C.load().kf_mapreduce(fcode, opcode, gcode, ops.dtype_code(src), src.data_ptr(), n, dst.data_ptr(),
                                   buf.ptr(), buf.nbytes, cfg, ops.stream_handle(src))
    C.check(rc, "mapreduce")
    return dst


def mapreduce(f, op, src, *, dims=None, g=ops.identity, tmp=None, Nitem=None, workgroup=None, blocks=None,
              arch=None, to_cpu=True):
    """`mapreduce(f, op, src; g)`: the reduced value as a host scalar (or a 1-element device tensor)."""
    s = _check_common(dims, src)
    dst = torch.empty(1, dtype=s.dtype, device=s.device)
    mapreduce_(f, op, dst, s, g=g, tmp=tmp, Nitem=Nitem, workgroup=workgroup, blocks=blocks, arch=arch)
    return dst.cpu()[0].item() if to_cpu else dst


# The reference's 1-D names (src/mapreduce/1D/mapreduce1d.jl:177-288).
mapreduce1d = mapreduce
mapreduce1d_ = mapreduce_
