"""CUDA-graph capture of a sequence of library calls.

Every entry point of libkf_b200.so is a fixed sequence of stream operations (the workspace clear and one
or a few kernel launches, no host synchronisation, no allocation when `tmp=` is given), so a step made
of several calls can be recorded once and replayed with a single launch. Replaying removes the gaps
between the memsets and kernels of consecutive calls (about 3 % of a step of two 2^28-element scans).
The reference has no counterpart: CUDA.jl launches every kernel of `scan!` separately
(src/scan/scan.jl:414-479 of KernelForge.jl).
"""
from __future__ import annotations

import torch

from . import _cabi as C


class CapturedStep:
    """`CapturedStep(fn)` runs `fn` twice on a side stream (first calls set kernel attributes), then
    records one more run into a CUDA graph. `fn` must call the library with pre-allocated `tmp=` buffers
    and fixed tensors; `replay()` repeats exactly those operations on the current stream, reading whatever
    the tensors hold then. `launches` is the number of library kernels in one replay."""

    def __init__(self, fn, device=None, warmup: int = 2):
        lib = C.load()
        self.stream = torch.cuda.Stream(device)
        self.graph = torch.cuda.CUDAGraph()
        self.stream.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(self.stream):
            for _ in range(warmup):
                fn()
            self.stream.synchronize()
            before = lib.kf_launch_count()
            with torch.cuda.graph(self.graph, stream=self.stream):
                fn()
            self.launches = int(lib.kf_launch_count() - before)
        torch.cuda.current_stream(device).wait_stream(self.stream)

    def replay(self) -> None:
        self.graph.replay()
