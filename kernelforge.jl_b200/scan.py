"""`KernelForge.scan` / `scan!`: inclusive prefix scan, non-commutative operators allowed.

Mirrors src/scan/scan.jl:218-284 of KernelForge.jl. Calling forms:

    scan_(op, dst, src)            scan_(f, op, dst, src)
    scan(op, src)                  scan(f, op, src)
    scan_(AffineCompose(), (a_dst, b_dst), (a_src, b_src))      # two Float32 arrays
    scan_(AffineCompose(), dst_ab, src_ab)                      # [n, 2] Float32 (NTuple{2,Float32})
    scan_(QuaternionMul(), dst_q, src_q)                        # [n, 4] Float32 / Float64 (Quaternion{T})

`g=` is applied to every output element (src/scan/scan_kernel.jl:463,470,474): identity or sqrt.
`init=` (a device tensor of one or more elements; [k, 2] (a, b) pairs for the affine form) is folded
left to right and seeds the scan from the left; the sharded scan passes the totals of the shards
before it.
"""
from __future__ import annotations

import torch

from . import _cabi as C
from . import ops
from .allocations import Scan1D, quaternion_scan_bytes, resolve_tmp, scan_bytes


def _split_args(args, n_tail):
    if len(args) == n_tail + 1:
        return (ops.identity,) + tuple(args)
    if len(args) == n_tail + 2:
        return tuple(args)
    raise TypeError("expected ([f,] op, %s)" % ("dst, src" if n_tail == 2 else "src"))


def _scan_affine(dst, src, init, tmp, cfg):
    lib = C.load()
    if isinstance(src, (tuple, list)):
        if not (isinstance(dst, (tuple, list)) and len(src) == 2 and len(dst) == 2):
            raise C.ArgumentError("AffineCompose expects (a_dst, b_dst), (a_src, b_src)")
        for t in (*src, *dst):
            ops.require_device_vector(t, "affine array")
            if t.dtype != torch.float32:
                raise C.ArgumentError("AffineCompose is implemented for Float32 pairs only")
        n = src[0].numel()
        if any(t.numel() != n for t in (*src, *dst)):
            raise C.ArgumentError("affine arrays must have equal lengths")
        if n == 0:
            return dst
        buf = resolve_tmp(tmp, Scan1D, scan_bytes(C.F32, True, n, cfg), src[0].device)
        with ops.on_device(src[0].device):
            rc = lib.kf_scan_affine_soa(src[0].data_ptr(), src[1].data_ptr(), dst[0].data_ptr(), dst[1].data_ptr(),
                                        n, init.data_ptr() if init is not None else None,
                                        init.numel() // 2 if init is not None else 0,
                                        buf.ptr(), buf.nbytes, cfg, ops.stream_handle(src[0]))
        C.check(rc, "scan!")
        return dst
    ops.require_device_vector(src, "src")
    ops.require_device_vector(dst, "dst")
    if src.dtype != torch.float32 or dst.dtype != torch.float32 or src.dim() != 2 or src.shape[1] != 2 \
            or dst.shape != src.shape:
        raise C.ArgumentError("AffineCompose expects [n, 2] Float32 arrays of (a, b) pairs")
    n = src.shape[0]
    if n == 0:
        return dst
    buf = resolve_tmp(tmp, Scan1D, scan_bytes(C.F32, True, n, cfg), src.device)
    with ops.on_device(src.device):
        rc = lib.kf_scan_affine_aos(src.data_ptr(), dst.data_ptr(), n, init.data_ptr() if init is not None else None,
                                    init.numel() // 2 if init is not None else 0,
                                    buf.ptr(), buf.nbytes, cfg, ops.stream_handle(src))
    C.check(rc, "scan!")
    return dst


def _scan_quaternion(dst, src, init, tmp, cfg):
    ops.require_device_vector(src, "src")
    ops.require_device_vector(dst, "dst")
    if src.dtype not in (torch.float32, torch.float64) or dst.dtype != src.dtype or src.dim() != 2 \
            or src.shape[1] != 4 or dst.shape != src.shape:
        raise C.ArgumentError("QuaternionMul expects [n, 4] Float32 or Float64 arrays of (w, x, y, z)")
    if init is not None and (init.dtype != src.dtype or init.numel() == 0 or init.numel() % 4):
        raise C.ArgumentError("init must hold quaternions of the element type")
    n = src.shape[0]
    if n == 0:
        return dst
    code = C.F32 if src.dtype == torch.float32 else C.F64
    buf = resolve_tmp(tmp, Scan1D, quaternion_scan_bytes(code, n), src.device)
    with ops.on_device(src.device):
        rc = C.load().kf_scan_quaternion(code, src.data_ptr(), dst.data_ptr(), n,
                                         init.data_ptr() if init is not None else None,
                                         init.numel() // 4 if init is not None else 0,
                                         buf.ptr(), buf.nbytes, cfg, ops.stream_handle(src))
    C.check(rc, "scan!")
    return dst


def scan_(*args, g=ops.identity, tmp=None, Nitem=None, workgroup=None, family=None, arch=None, init=None,
          _test_hook=0):
    """`scan!([f,] op, dst, src)`: dst[i] = g(f(src[0]) op ... op f(src[i])). Returns dst (asynchronous)."""
    f, op, dst, src = _split_args(args, 2)
    gcode = ops.post_code(g)
    cfg = C.make_cfg(workgroup, Nitem, None, _test_hook)
    if init is not None:
        ops.require_device_vector(init, "init")
        if not init.is_contiguous():
            raise C.ArgumentError("init must be contiguous")
    if isinstance(op, ops.AffineCompose):
        if ops.map_code(f) != C.MAP_IDENTITY or gcode != C.POST_IDENTITY:
            raise C.ArgumentError("AffineCompose supports f=identity and g=identity only")
        if init is not None and (init.dtype != torch.float32 or init.numel() == 0 or init.numel() % 2):
            raise C.ArgumentError("init must hold Float32 (a, b) pairs")
        return _scan_affine(dst, src, init, tmp, cfg)
    if isinstance(op, ops.QuaternionMul):
        if ops.map_code(f) != C.MAP_IDENTITY or gcode != C.POST_IDENTITY:
            raise C.ArgumentError("QuaternionMul supports f=identity and g=identity only")
        return _scan_quaternion(dst, src, init, tmp, cfg)
    fcode, opcode = ops.map_code(f), ops.op_code(op)
    ops.require_device_vector(src, "src")
    ops.require_device_vector(dst, "dst")
    if dst.dtype != src.dtype:
        raise C.ArgumentError("dst must have the element type of f(src) (%s), got %s" % (src.dtype, dst.dtype))
    n = src.numel()
    if dst.numel() != n:
        raise C.ArgumentError("dst and src must have equal lengths")
    if init is not None and (init.dtype != src.dtype or init.numel() < 1):
        raise C.ArgumentError("init must hold one or more elements of the element type")
    if n == 0:
        return dst
    code = ops.dtype_code(src)
    buf = resolve_tmp(tmp, Scan1D, scan_bytes(code, False, n, cfg), src.device)
    with ops.on_device(src.device):
        rc = C.load().kf_scan(fcode, opcode, gcode, code, src.data_ptr(), dst.data_ptr(), n,
                              init.data_ptr() if init is not None else None, init.numel() if init is not None else 0,
                              buf.ptr(), buf.nbytes, cfg, ops.stream_handle(src))
    C.check(rc, "scan!")
    return dst


def scan(*args, **kwargs):
    """`scan([f,] op, src)`: allocating form, returns the scanned array."""
    f, op, src = _split_args(args, 1)
    if isinstance(src, (tuple, list)):
        dst = tuple(torch.empty_like(t) for t in src)
    else:
        dst = torch.empty_like(src)
    return scan_(f, op, dst, src, **kwargs)
