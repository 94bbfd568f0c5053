"""`kf_scan_static`: the scan for callers that cannot allocate device memory for a workspace (code
under a framework's memory pool, processes at the device's memory limit, loops that cannot afford
the synchronisation of cudaMalloc). Its tile descriptors live in a fixed 1 MiB device array inside
the library. Collected last on purpose: a failure here cannot hide the other tests from a run that
stops at the first failure.

The GPU test calls the entry point through the C ABI twice in a row on different data and compares
each result with the CPU oracle and with the workspace-taking `kf_scan`: bit for bit for integers,
within the scan tolerance (1e-5*log2 n) for Float32, whose look-back association may differ from run
to run. It also checks that the second round of calls leaves the device's free memory unchanged.
"""
import ctypes

import numpy as np
import pytest
import torch

from util import scan_tol, to_host


def test_size_limit_is_refused_before_touching_the_device(kf):
    """Needs no GPU: argument and size checks come first and nothing is dereferenced."""
    from kernelforge_jl_b200 import _cabi as C
    lib = kf.lib
    fake = ctypes.c_void_p(0x1000)
    assert lib.kf_scan_static(0, 0, 0, C.U32, fake, fake, 1 << 40, None, 0, None) == C.ERR_EXCEEDS_STATIC_SCRATCH
    assert lib.kf_scan_static(0, 0, 0, C.F64, fake, fake, 1 << 31, None, 0, None) == C.ERR_EXCEEDS_STATIC_SCRATCH
    # a plan with more than 2^31 tiles has no workspace size at all: still "too large", not "unsupported"
    assert lib.kf_scan_static(0, 0, 0, C.F64, fake, fake, 1 << 50, None, 0, None) == C.ERR_EXCEEDS_STATIC_SCRATCH
    assert lib.kf_scan_static(0, 0, 0, C.U32, fake, fake, 0, None, 0, None) == C.OK  # n == 0 is a no-op
    # the same codes, in the same order, as kf_scan: enums are checked before the n == 0 return
    for n in (0, 10):
        assert lib.kf_scan_static(0, 0, 0, 42, fake, fake, n, None, 0, None) == C.ERR_INVALID_ARG
        assert lib.kf_scan(0, 0, 0, 42, fake, fake, n, None, 0, fake, 1 << 20, None, None) == C.ERR_INVALID_ARG
        assert lib.kf_scan_static(9, 0, 0, C.U32, fake, fake, n, None, 0, None) == C.ERR_UNSUPPORTED
        assert lib.kf_scan_static(0, C.OP_AFFINE, 0, C.F32, fake, fake, n, None, 0, None) == C.ERR_UNSUPPORTED
        assert lib.kf_scan_static(0, 0, C.POST_SQRT, C.I32, fake, fake, n, None, 0, None) == C.ERR_UNSUPPORTED
    assert "kf_scan_static" in lib.kf_error_string(C.ERR_EXCEEDS_STATIC_SCRATCH).decode()


def test_documented_maximum_sizes(kf):
    """The header states the largest n per element width; the query and the refusal agree with it."""
    from kernelforge_jl_b200 import _cabi as C
    lib = kf.lib
    fake = ctypes.c_void_p(0x1000)
    stated = {C.U8: 4293885952, C.I16: 2146942976, C.F32: 1073471488, C.U32: 1073471488, C.F64: 268365824}
    for dtype, nmax in stated.items():
        assert lib.kf_scan_static_max_n(dtype) == nmax
        assert 0 < lib.kf_scan_workspace_bytes(dtype, 0, nmax, None) <= (1 << 20)
        assert lib.kf_scan_static(0, 0, 0, dtype, fake, fake, nmax + 1, None, 0, None) == C.ERR_EXCEEDS_STATIC_SCRATCH
    assert lib.kf_scan_static_max_n(42) == 0


@pytest.mark.gpu
def test_static_scratch_scan_matches_workspace_scan_twice(kf, oracle):
    from kernelforge_jl_b200 import _cabi as C
    lib = kf.lib
    stream = torch.cuda.current_stream().cuda_stream
    n = (1 << 24) + 12345  # several thousand tiles, ragged tail, ring kernel
    g = torch.Generator(device="cuda").manual_seed(7)
    outs = [torch.empty(n, dtype=torch.int32, device="cuda"), torch.empty(n, dtype=torch.float32, device="cuda")]
    free_before = None
    for call in range(2):  # two calls in a row: the second one finds the first one's descriptors in the array
        xi = torch.randint(0, 1 << 31, (n,), dtype=torch.int32, device="cuda", generator=g)
        xf = torch.rand(n, dtype=torch.float32, device="cuda", generator=g)
        ref = kf.scan("+", xi.view(torch.uint32))
        reff = kf.scan("+", xf)
        torch.cuda.synchronize()
        if call == 1:  # every buffer of this round exists: what follows must not allocate device memory
            free_before = torch.cuda.mem_get_info()[0]
        out, outf = outs
        rc = lib.kf_scan_static(C.MAP_IDENTITY, C.OP_ADD, C.POST_IDENTITY, C.U32, xi.data_ptr(), out.data_ptr(), n,
                                None, 0, stream)
        assert rc == C.OK
        assert lib.kf_scan_static(C.MAP_IDENTITY, C.OP_ADD, C.POST_IDENTITY, C.F32, xf.data_ptr(), outf.data_ptr(), n,
                                  None, 0, stream) == C.OK
        assert lib.kf_scan_static_check(stream) == C.OK
        if call == 1:
            assert torch.cuda.mem_get_info()[0] == free_before, "kf_scan_static changed the device's free memory"
        # against the workspace-taking entry point ...
        assert torch.equal(out, ref.view(torch.int32))
        rel = ((outf.double() - reff.double()).abs() / reff.double().clamp_min(1e-30)).max().item()
        assert rel <= scan_tol(n), rel
        # ... and against the CPU oracle (wrapping UInt32 sum; Float64 left fold)
        want = oracle.c_scan(oracle.MAP_IDENTITY, oracle.OP_ADD, to_host(xi.view(torch.uint32)))
        assert np.array_equal(to_host(out.view(torch.uint32)), want)
        wantf = oracle.c_scan(oracle.MAP_IDENTITY, oracle.OP_ADD, to_host(xf))
        relo = np.max(np.abs(to_host(outf).astype(np.float64) - wantf) / np.maximum(wantf, 1e-30))
        assert relo <= scan_tol(n), relo

    # a small, misaligned, seeded call through the direct kernel, and the same array used in place
    small = torch.arange(1, 1001, dtype=torch.int64, device="cuda")[1:]
    seed = torch.tensor([5], dtype=torch.int64, device="cuda")
    assert lib.kf_scan_static(C.MAP_IDENTITY, C.OP_ADD, C.POST_IDENTITY, C.I64, small.data_ptr(), small.data_ptr(),
                              small.numel(), seed.data_ptr(), 1, stream) == C.OK
    k = torch.arange(2, 1001, dtype=torch.int64, device="cuda")
    assert torch.equal(small, torch.cumsum(k, 0) + 5)
    assert lib.kf_scan_static_check(stream) == C.OK
