"""`kf_scan_static`: the scan for callers that cannot allocate device memory for a workspace (code
under a framework's memory pool, processes at the device's memory limit, loops that cannot afford
the synchronisation of cudaMalloc). Its tile descriptors live in a fixed 1 MiB device array inside
the library. Collected last on purpose: a failure here cannot hide the other tests from a run that
stops at the first failure.

The GPU test calls the entry point through the C ABI twice in a row on different data and compares
each result with the workspace-taking `kf_scan`: bit for bit for integers, within the scan tolerance
(1e-5*log2 n) for Float32, whose look-back association may differ from run to run.
"""
import ctypes

import numpy as np
import pytest
import torch

from util import scan_tol


def test_size_limit_is_refused_before_touching_the_device(kf):
    """Needs no GPU: the size check comes first and nothing is dereferenced."""
    from kernelforge_jl_b200 import _cabi as C
    lib = kf.lib
    fake = ctypes.c_void_p(0x1000)
    assert lib.kf_scan_static(0, 0, C.U32, fake, fake, 1 << 40, None, None) == C.ERR_EXCEEDS_STATIC_SCRATCH
    assert lib.kf_scan_static(0, 0, C.F64, fake, fake, 1 << 31, None, None) == C.ERR_EXCEEDS_STATIC_SCRATCH
    assert lib.kf_scan_static(0, 0, C.U32, fake, fake, 0, None, None) == C.OK  # n == 0 is a no-op
    assert lib.kf_scan_static(0, 0, 42, fake, fake, 10, None, None) == C.ERR_INVALID_ARG
    assert "kf_scan_static" in lib.kf_error_string(C.ERR_EXCEEDS_STATIC_SCRATCH).decode()


@pytest.mark.gpu
def test_static_scratch_scan_matches_workspace_scan_twice(kf):
    from kernelforge_jl_b200 import _cabi as C
    lib = kf.lib
    stream = torch.cuda.current_stream().cuda_stream
    n = (1 << 24) + 12345  # several thousand tiles, ragged tail, ring kernel
    g = torch.Generator(device="cuda").manual_seed(7)
    for call in range(2):  # two calls in a row: the second one finds the first one's descriptors in the array
        xi = torch.randint(0, 1 << 31, (n,), dtype=torch.int32, device="cuda", generator=g)
        ref = kf.scan("+", xi.view(torch.uint32))
        out = torch.empty_like(xi)
        rc = lib.kf_scan_static(C.MAP_IDENTITY, C.OP_ADD, C.U32, xi.data_ptr(), out.data_ptr(), n, None, stream)
        assert rc == C.OK
        assert torch.equal(out, ref.view(torch.int32))

        xf = torch.rand(n, dtype=torch.float32, device="cuda", generator=g)
        reff = kf.scan("+", xf)
        outf = torch.empty_like(xf)
        assert lib.kf_scan_static(C.MAP_IDENTITY, C.OP_ADD, C.F32, xf.data_ptr(), outf.data_ptr(), n, None, stream) == C.OK
        rel = ((outf.double() - reff.double()).abs() / reff.double().clamp_min(1e-30)).max().item()
        assert rel <= scan_tol(n), rel

    # a small, misaligned, seeded call through the direct kernel, and the same array used in place
    small = torch.arange(1, 1001, dtype=torch.int64, device="cuda")[1:]
    seed = torch.tensor([5], dtype=torch.int64, device="cuda")
    assert lib.kf_scan_static(C.MAP_IDENTITY, C.OP_ADD, C.I64, small.data_ptr(), small.data_ptr(), small.numel(),
                              seed.data_ptr(), stream) == C.OK
    k = torch.arange(2, 1001, dtype=torch.int64, device="cuda")
    assert torch.equal(small, torch.cumsum(k, 0) + 5)
