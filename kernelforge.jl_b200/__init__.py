"""kernelforge.jl_b200 — B200-native (sm_100a) mapreduce / scan / radix sort behind KernelForge.jl's call
signatures.

The compute path is libkf_b200.so (hand-written CUDA kernels, C ABI in include/kf_b200.h). This
package is the executable host-side mirror of the Julia layer in `julia/`: same function names
(`mapreduce`, `scan`, `sort`, `get_allocation`; a trailing underscore stands for Julia's `!`),
same argument meaning and error behaviour. PyTorch only provides device memory, streams and
`torch.distributed`. Importing the package loads the library and fails loudly when it is missing.
"""
from . import _cabi
from ._cabi import ArgumentError, KernelForgeError
from .allocations import KernelBuffer, MapReduce1D, Scan1D, Sort1D, get_allocation
from .mapreduce import mapreduce, mapreduce_, mapreduce1d, mapreduce1d_
from .ops import AffineCompose, QuaternionMul, abs2, identity, prod, sqdiff, sqrt, wsq
from .scan import scan, scan_
from .graphs import CapturedStep
from .search import (argmax, argmax1d, argmin, eq, findfirst, findlast, ge, gt, le, lt, ne, setvalue_, vcopy_)
from .sort import sort, sort_, sortperm

lib = _cabi.load()

__all__ = [
    "ArgumentError", "KernelForgeError", "KernelBuffer", "MapReduce1D", "Scan1D", "Sort1D", "get_allocation",
    "mapreduce", "mapreduce_", "mapreduce1d", "mapreduce1d_", "scan", "scan_", "sort", "sort_", "sortperm",
    "AffineCompose", "QuaternionMul", "abs2", "identity", "sqrt", "prod", "sqdiff", "wsq", "lib", "argmax", "argmax1d", "argmin", "findfirst", "findlast", "gt", "lt", "ge", "le",
    "eq", "ne", "vcopy_", "setvalue_", "CapturedStep",
]
