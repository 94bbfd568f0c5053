"""Workspaces: `KernelBuffer`, algorithm tags and `get_allocation`.

Mirrors src/allocations.jl:16-49 and the per-algorithm `get_allocation` methods of KernelForge.jl
(src/mapreduce/1D/mapreduce1d.jl:140-170, src/scan/scan.jl:156-211, src/sort/sort1d.jl:237-300).
The reference's buffers are NamedTuples of typed arrays; here a workspace is one byte buffer whose
layout is private to the C library and whose size comes from the `kf_*_workspace_bytes` queries.
A buffer can be reused across calls; passing one that is too small raises, as in the reference
(test/tests/mapreduce/mapreduce1d_test.jl:218-224).
"""
from __future__ import annotations

import torch

from . import _cabi as C
from . import ops


class MapReduce1D:
    """Algorithm tag (src/algorithms.jl:9-50)."""


class Scan1D:
    """Algorithm tag (src/algorithms.jl:9-50)."""


class Sort1D:
    """Algorithm tag (src/algorithms.jl:9-50)."""


class KernelBuffer:
    """Pre-allocated workspace for one primitive (src/allocations.jl:16-18).

    `arrays` is a dict of named device tensors like the reference's NamedTuple; the single entry
    `workspace` is the byte buffer handed to the C library.
    """

    def __init__(self, tag, workspace: torch.Tensor):
        self.tag = tag
        self.arrays = {"workspace": workspace}

    @property
    def workspace(self) -> torch.Tensor:
        return self.arrays["workspace"]

    @property
    def nbytes(self) -> int:
        return self.workspace.numel()

    def ptr(self) -> int:
        return self.workspace.data_ptr()


def _alloc(tag, nbytes: int, device) -> KernelBuffer:
    if nbytes <= 0:
        raise C.ArgumentError("no workspace layout for these arguments (unsupported type or launch override)")
    return KernelBuffer(tag, torch.empty(nbytes, dtype=torch.uint8, device=device))


def mapreduce_bytes(src, cfg) -> int:
    return C.load().kf_mapreduce_workspace_bytes(ops.dtype_code(src), src.numel(), cfg)


def scan_bytes(dtype_code: int, pair: bool, n: int, cfg) -> int:
    return C.load().kf_scan_workspace_bytes(dtype_code, 1 if pair else 0, n, cfg)


def quaternion_scan_bytes(dtype_code: int, n: int) -> int:
    return C.load().kf_scan_quaternion_workspace_bytes(dtype_code, n)


def sort_bytes(key_code: int, val_bytes: int, n: int, cfg) -> int:
    return C.load().kf_sort_workspace_bytes(key_code, val_bytes, n, cfg)


def get_allocation(tag, *args, **kwargs) -> KernelBuffer:
    """`KernelForge.get_allocation(Tag, ...)` / `@allocate`.

    get_allocation(MapReduce1D, f, op, src, workgroup=None, blocks=None, arch=None)
    get_allocation(Scan1D, f, op, src, workgroup=None, blocks=None, arch=None)
    get_allocation(Sort1D, src, Nitem=None, Nchunks=None, workgroup=None, arch=None, keys=None)
    """
    if tag is MapReduce1D:
        f, op, src = args[:3]
        workgroup = args[3] if len(args) > 3 else kwargs.get("workgroup")
        blocks = args[4] if len(args) > 4 else kwargs.get("blocks")
        if isinstance(src, (tuple, list)):
            src = src[0]
        ops.require_device_vector(src, "src")
        cfg = C.make_cfg(workgroup, kwargs.get("Nitem"), blocks)
        return _alloc(tag, mapreduce_bytes(src, cfg), src.device)
    if tag is Scan1D:
        f, op, src = args[:3]
        workgroup = args[3] if len(args) > 3 else kwargs.get("workgroup")
        cfg = C.make_cfg(workgroup, kwargs.get("Nitem"), None)
        if isinstance(op, ops.AffineCompose):
            a = src[0] if isinstance(src, (tuple, list)) else src
            n = a.shape[0]
            return _alloc(tag, scan_bytes(C.F32, True, n, cfg), a.device)
        ops.require_device_vector(src, "src")
        if isinstance(op, ops.QuaternionMul):
            return _alloc(tag, quaternion_scan_bytes(ops.dtype_code(src), src.shape[0]), src.device)
        return _alloc(tag, scan_bytes(ops.dtype_code(src), False, src.numel(), cfg), src.device)
    if tag is Sort1D:
        src = args[0]
        ops.require_device_vector(src, "src")
        keys = kwargs.get("keys")
        cfg = C.make_cfg(kwargs.get("workgroup"), kwargs.get("Nitem"), None)
        if keys is None:
            nbytes = sort_bytes(ops.dtype_code(src), 0, src.numel(), cfg)
        else:
            ops.require_device_vector(keys, "keys")
            nbytes = sort_bytes(ops.dtype_code(keys), src.element_size(), src.numel(), cfg)
        return _alloc(tag, nbytes, src.device)
    raise C.KernelForgeError("Unknown ForgeAlgorithm: %r" % (tag,))


def resolve_tmp(tmp, tag, need_bytes: int, device) -> KernelBuffer:
    """Returns `tmp` if it fits, allocates when it is None, raises when it is too small."""
    if need_bytes <= 0:
        raise C.ArgumentError("unsupported element type or launch override for this primitive")
    if tmp is None:
        return _alloc(tag, need_bytes, device)
    if not isinstance(tmp, KernelBuffer):
        raise C.ArgumentError("tmp must be a KernelBuffer from get_allocation")
    if tmp.nbytes < need_bytes:
        raise C.KernelForgeError(
            "tmp holds %d bytes but this call needs %d: allocate it with get_allocation for the same "
            "arguments" % (tmp.nbytes, need_bytes))
    if tmp.workspace.device != device:
        raise C.ArgumentError("tmp lives on another device than the data")
    return tmp
