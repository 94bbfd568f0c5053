"""`KernelForge.sort` / `sort!`: stable ascending radix (onesweep) sort, keys-only and key-value.

Mirrors src/sort/sort1d.jl:307-502 of KernelForge.jl:

    sort_(src)                         in place
    sort_(dst, src)                    out of place (src is left untouched)
    sort(src)                          allocating
    sort_(vals, keys=k) / sort_(dst, vals, keys=k) / sort(vals, keys=k)
        `keys` drives the order, `vals` is the payload that follows; returns (dst, keys_dst)
        (src/sort/sort1d.jl:427-465, test/tests/sort/sort_keyval_test.jl:29-36). In the in-place
        form `keys` is sorted in place as well.

Only the radix path exists: `lt`, `by`, `rev`, a custom `uint_map` or another `algorithm` raise
`ArgumentError` (the reference would route those to its comparison sorts; there is no fallback here).
"""
from __future__ import annotations

import torch

from . import _cabi as C
from . import ops
from .allocations import Sort1D, resolve_tmp, sort_bytes

_SORT_KEY_CODES = {C.U8, C.I8, C.U16, C.I16, C.U32, C.I32, C.F32, C.U64, C.I64, C.F64}


def _reject(by, uint_map, lt, rev, algorithm):
    if by is not None and by is not ops.identity:
        raise C.ArgumentError("sort: `by` other than identity is not supported (fixed key maps only)")
    if uint_map is not None:
        raise C.ArgumentError("sort: a custom `uint_map` is not supported (fixed key maps only)")
    if lt is not None or rev:
        raise C.ArgumentError("sort: `lt` / `rev` need a comparison sort, which this library does not have")
    if algorithm not in (None, "radix", "onesweep"):
        raise C.ArgumentError("sort: only the radix onesweep algorithm is implemented")


def sort_(*args, keys=None, keys_dst=None, by=None, uint_map=None, lt=None, rev=False, algorithm=None, tmp=None,
          Nitem=None, Nchunks=None, workgroup=None, arch=None, family=None, rr=None, _test_hook=0):
    """`sort!(src)` / `sort!(dst, src)`; with `keys=` the key-value form returning (dst, keys_dst)."""
    _reject(by, uint_map, lt, rev, algorithm)
    if len(args) == 1:
        dst = src = args[0]
    elif len(args) == 2:
        dst, src = args
    else:
        raise TypeError("sort_(src) or sort_(dst, src)")
    ops.require_device_vector(src, "src")
    ops.require_device_vector(dst, "dst")
    if dst.dtype != src.dtype or dst.numel() != src.numel():
        raise C.ArgumentError("dst and src must have the same element type and length")
    n = src.numel()
    cfg = C.make_cfg(workgroup, Nitem, None, _test_hook)
    lib = C.load()
    if keys is None:
        code = ops.dtype_code(src)
        if code not in _SORT_KEY_CODES:
            raise C.ArgumentError("sort: element type %s is not supported by the radix path of this library" % src.dtype)
        if n == 0:
            return dst
        buf = resolve_tmp(tmp, Sort1D, sort_bytes(code, 0, n, cfg), src.device)
        with ops.on_device(src.device):
            rc = lib.kf_sort_keys(code, src.data_ptr(), dst.data_ptr(), n, buf.ptr(), buf.nbytes, cfg,
                                  ops.stream_handle(src))
        C.check(rc, "sort!")
        return dst
    # key-value
    ops.require_device_vector(keys, "keys")
    if keys.numel() != n:
        raise C.KernelForgeError("sort!: `keys` must have the same length as `src` (%d vs %d)" % (keys.numel(), n))
    kcode = ops.dtype_code(keys)
    if kcode not in _SORT_KEY_CODES:
        raise C.ArgumentError("sort: key type %s is not supported by the radix path of this library" % keys.dtype)
    vb = src.element_size()
    if vb not in (4, 8):
        raise C.ArgumentError("sort: payload elements must be 4 or 8 bytes wide, got %d" % vb)
    if keys_dst is None:
        keys_dst = keys if dst is src else torch.empty_like(keys)
    ops.require_device_vector(keys_dst, "keys_dst")
    if keys_dst.dtype != keys.dtype or keys_dst.numel() != n:
        raise C.ArgumentError("keys_dst must match keys in type and length")
    if n == 0:
        return dst, keys_dst
    buf = resolve_tmp(tmp, Sort1D, sort_bytes(kcode, vb, n, cfg), src.device)
    with ops.on_device(src.device):
        rc = lib.kf_sort_pairs(kcode, keys.data_ptr(), keys_dst.data_ptr(), vb, src.data_ptr(), dst.data_ptr(), n,
                               buf.ptr(), buf.nbytes, cfg, ops.stream_handle(src))
    C.check(rc, "sort!")
    return dst, keys_dst


def sort(src, **kwargs):
    """`sort(src)`: allocating form (src is left untouched)."""
    ops.require_device_vector(src, "src")
    dst = torch.empty_like(src)
    return sort_(dst, src, **kwargs)


def sortperm(keys, **kwargs):
    """`sortperm(keys)`: the stable permutation that sorts `keys` (0-based indices, int64 when
    n >= 2^31 else int32). Iota fill + key-value sort, like src/sort/sortperm.jl:162-214."""
    ops.require_device_vector(keys, "keys")
    n = keys.numel()
    wide = n >= 2 ** 31
    idx = torch.empty(n, dtype=torch.int64 if wide else torch.int32, device=keys.device)
    if n:
        with ops.on_device(keys.device):
            rc = C.load().kf_iota(C.I64 if wide else C.I32, idx.data_ptr(), n, 0, ops.stream_handle(keys))
        C.check(rc, "sortperm")
    out, _ = sort_(torch.empty_like(idx), idx, keys=keys, keys_dst=torch.empty_like(keys), **kwargs)
    return out
