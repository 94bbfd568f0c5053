"""ctypes binding of libkf_b200.so: the executable twin of the Julia `ccall` layer.

Every C entry point declared in include/kf_b200.h is bound here with its exact signature. The
library is the only compute path: if it cannot be loaded, importing this module raises; there is
no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_int32, c_size_t, c_uint32, c_uint64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libkf_b200.so")

ABI_VERSION = 2  # KF_B200_ABI_VERSION of include/kf_b200.h

# kf_status
OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE_TOO_SMALL, ERR_LAUNCH_FAILED, ERR_TIMEOUT, ERR_EMPTY, \
    ERR_EXCEEDS_STATIC_SCRATCH = range(8)
# kf_dtype
U8, I8, U16, I16, U32, I32, U64, I64, F32, F64 = range(10)
# kf_map / kf_op / kf_post / kf_primitive
MAP_IDENTITY, MAP_ABS2, MAP_ABS = range(3)
OP_ADD, OP_MUL, OP_MIN, OP_MAX, OP_AND, OP_OR, OP_XOR, OP_AFFINE = range(8)
POST_IDENTITY, POST_SQRT = range(2)
MAPN_PROD, MAPN_SQDIFF, MAPN_WSQ = range(3)
PRED_GT, PRED_LT, PRED_GE, PRED_LE, PRED_EQ, PRED_NE = range(6)
PRIM_MAPREDUCE, PRIM_SCAN, PRIM_SORT_KEYS, PRIM_SORT_PAIRS = range(4)


class LaunchCfg(Structure):
    """Mirror of `kf_launch_cfg`."""

    _fields_ = [("threads", c_int32), ("items", c_int32), ("blocks", c_int32), ("reserved", c_int32)]


class ArgumentError(ValueError):
    """The Python stand-in for Julia's `ArgumentError` (bad or unsupported arguments)."""


class KernelForgeError(RuntimeError):
    """The Python stand-in for Julia's `ErrorException` (`error(...)`) raised by the library."""


# name -> (restype, argtypes); must list every symbol of include/kf_b200.h
PROTOTYPES = {
    "kf_abi_version": (c_int32, []),
    "kf_error_string": (c_char_p, [c_int32]),
    "kf_last_cuda_error": (c_int32, []),
    "kf_check": (c_int32, [c_void_p, c_void_p]),
    "kf_launch_table_lookup": (c_int32, [c_int32, c_int32, c_uint64, POINTER(LaunchCfg)]),
    "kf_launch_count": (c_uint64, []),
    "kf_num_sms": (c_int32, []),
    "kf_mapreduce_workspace_bytes": (c_size_t, [c_int32, c_uint64, POINTER(LaunchCfg)]),
    "kf_mapreduce": (c_int32, [c_int32, c_int32, c_int32, c_int32, c_void_p, c_uint64, c_void_p,
                               c_void_p, c_size_t, POINTER(LaunchCfg), c_void_p]),
    "kf_mapreduce_multi": (c_int32, [c_int32, c_int32, c_int32, c_int32, POINTER(c_void_p), c_int32, c_uint64, c_void_p,
                                     c_void_p, c_size_t, POINTER(LaunchCfg), c_void_p]),
    "kf_scan_workspace_bytes": (c_size_t, [c_int32, c_int32, c_uint64, POINTER(LaunchCfg)]),
    "kf_scan": (c_int32, [c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_uint64, c_void_p, c_uint32,
                          c_void_p, c_size_t, POINTER(LaunchCfg), c_void_p]),
    "kf_scan_static": (c_int32, [c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_uint64, c_void_p, c_uint32,
                                 c_void_p]),
    "kf_scan_static_max_n": (c_uint64, [c_int32]),
    "kf_scan_static_check": (c_int32, [c_void_p]),
    "kf_scan_affine_soa": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_uint64, c_void_p, c_uint32,
                                     c_void_p, c_size_t, POINTER(LaunchCfg), c_void_p]),
    "kf_scan_affine_aos": (c_int32, [c_void_p, c_void_p, c_uint64, c_void_p, c_uint32,
                                     c_void_p, c_size_t, POINTER(LaunchCfg), c_void_p]),
    "kf_scan_quaternion_workspace_bytes": (c_size_t, [c_int32, c_uint64]),
    "kf_scan_quaternion": (c_int32, [c_int32, c_void_p, c_void_p, c_uint64, c_void_p, c_uint32,
                                     c_void_p, c_size_t, POINTER(LaunchCfg), c_void_p]),
    "kf_sort_workspace_bytes": (c_size_t, [c_int32, c_int32, c_uint64, POINTER(LaunchCfg)]),
    "kf_sort_keys": (c_int32, [c_int32, c_void_p, c_void_p, c_uint64,
                               c_void_p, c_size_t, POINTER(LaunchCfg), c_void_p]),
    "kf_sort_pairs": (c_int32, [c_int32, c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_uint64,
                                c_void_p, c_size_t, POINTER(LaunchCfg), c_void_p]),
    "kf_iota": (c_int32, [c_int32, c_void_p, c_uint64, c_uint64, c_void_p]),
    "kf_upper_bounds": (c_int32, [c_int32, c_void_p, c_uint64, c_void_p, c_int32, c_void_p, c_void_p]),
    "kf_argmax_workspace_bytes": (c_size_t, [c_int32, c_uint64]),
    "kf_argmax": (c_int32, [c_int32, c_int32, c_int32, c_void_p, c_uint64, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "kf_find": (c_int32, [c_int32, c_int32, c_int32, c_void_p, c_uint64, c_void_p, c_void_p, c_void_p]),
    "kf_vcopy": (c_int32, [c_void_p, c_void_p, c_uint64, c_void_p]),
    "kf_setvalue": (c_int32, [c_int32, c_void_p, c_uint64, c_void_p, c_void_p]),
    "kf_xbuf_alloc": (c_int32, [c_size_t, POINTER(c_void_p)]),
    "kf_xbuf_free": (c_int32, [c_void_p]),
    "kf_ipc_export": (c_int32, [c_void_p, c_void_p]),
    "kf_ipc_open": (c_int32, [c_void_p, POINTER(c_void_p)]),
    "kf_ipc_close": (c_int32, [c_void_p]),
    "kf_copy_d2d": (c_int32, [c_void_p, c_void_p, c_uint64, c_void_p]),
    "kf_peer_region_bytes": (c_size_t, []),
    "kf_peer_allgather": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_uint32, c_void_p, c_int32, c_void_p, c_void_p,
                                    POINTER(LaunchCfg), c_void_p]),
    "kf_bucket_ids": (c_int32, [c_int32, c_void_p, c_uint64, c_void_p, c_int32, c_void_p, c_void_p]),
}

_lib = None


def load(path: str | None = None) -> ctypes.CDLL:
    """Loads the shared library (once) and attaches the prototypes. Raises if it is missing."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise KernelForgeError(
            "libkf_b200.so is not built (%s). Run `python kernelforge.jl_b200/build.py`; "
            "there is no fallback path." % p)
    lib = ctypes.CDLL(p)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    if lib.kf_abi_version() != ABI_VERSION:
        raise KernelForgeError("libkf_b200.so has ABI version %d, expected %d" % (lib.kf_abi_version(), ABI_VERSION))
    if path is None:
        _lib = lib
    return lib


def error_string(code: int) -> str:
    return load().kf_error_string(code).decode()


def check(code: int, what: str) -> None:
    """Turns a non-zero kf_status into the exception the reference would raise."""
    if code == OK:
        return
    msg = "%s: %s" % (what, error_string(code))
    if code == ERR_LAUNCH_FAILED:
        msg += " [cudaError %d]" % load().kf_last_cuda_error()
    if code in (ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_EMPTY, ERR_EXCEEDS_STATIC_SCRATCH):
        raise ArgumentError(msg)
    raise KernelForgeError(msg)


def make_cfg(threads=None, items=None, blocks=None, reserved=0):
    """A `kf_launch_cfg*` (or None) from the reference's `workgroup` / `Nitem` / `blocks` kwargs.
    `reserved` is the test hook of kf_launch_cfg (spin limit and silent tile); 0 in production."""
    if threads is None and items is None and blocks is None and not reserved:
        return None
    return ctypes.pointer(LaunchCfg(int(threads or 0), int(items or 0), int(blocks or 0), int(reserved)))
