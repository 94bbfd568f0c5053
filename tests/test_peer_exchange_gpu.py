"""GPU tests of `kf_peer_allgather`, the one-element allgather over peer memory that the sharded
mapreduce and scan use instead of a communication library, on ONE GPU: the "peers" are this rank's own
region, and the other rank's element is either written by the test (the exchange completes) or never
arrives (the bounded wait runs out and the kernel reports KF_ERR_TIMEOUT; nothing hangs or faults). The
two-rank path over NVLink is covered by tests/test_distributed_gpu.py when two GPUs are visible."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _region(kf):
    nbytes = int(kf.lib.kf_peer_region_bytes())
    region = torch.zeros(nbytes // 8, dtype=torch.int64, device="cuda")
    table = torch.tensor([region.data_ptr(), region.data_ptr()], dtype=torch.int64, device="cuda")
    status = torch.zeros(256, dtype=torch.uint8, device="cuda")
    return region, table, status


@pytest.mark.parametrize("dtype,val,other", [(torch.int32, -123456, 77), (torch.float32, 3.5, -0.25), (torch.float64, 1e300, 2.0),
                                             (torch.uint8, 200, 9), (torch.int64, -(1 << 60), 1 << 40)])
def test_exchange_completes_when_the_other_element_is_there(kf, dtype, val, other):
    from kernelforge_jl_b200 import _cabi as C
    region, table, status = _region(kf)
    st = torch.cuda.current_stream().cuda_stream
    for epoch in (1, 2, 5):  # slots rotate with the epoch
        mine = torch.tensor([val], dtype=dtype, device="cuda")
        theirs = torch.tensor([other], dtype=dtype, device="cuda")
        # what rank 1 would store: entry (slot, rank 1) = {epoch | low half}, {epoch | high half}
        bits = int.from_bytes(theirs.cpu().numpy().tobytes().ljust(8, b"\0"), "little")
        slot = epoch % 4
        w = [(epoch << 32) | (bits & 0xFFFFFFFF), (epoch << 32) | (bits >> 32)]
        w = [x - (1 << 64) if x >= (1 << 63) else x for x in w]
        region[(slot * 64 + 1) * 2 + 0] = w[0]
        region[(slot * 64 + 1) * 2 + 1] = w[1]
        out = torch.empty(2, dtype=dtype, device="cuda")
        rc = kf.lib.kf_peer_allgather(table.data_ptr(), region.data_ptr(), 2, 0, epoch, mine.data_ptr(), mine.element_size(),
                                      out.data_ptr(), status.data_ptr(), None, st)
        assert rc == C.OK
        assert kf.lib.kf_check(status.data_ptr(), None) == C.OK
        assert out.cpu().numpy().tobytes() == torch.cat([mine, theirs]).cpu().numpy().tobytes()


def test_a_missing_rank_runs_into_the_limit_and_is_reported(kf):
    from kernelforge_jl_b200 import _cabi as C
    region, table, status = _region(kf)
    st = torch.cuda.current_stream().cuda_stream
    mine = torch.tensor([42], dtype=torch.int32, device="cuda")
    out = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    cfg = ctypes.pointer(C.LaunchCfg(0, 0, 0, 500))  # test hook: give up after 500 polls
    rc = kf.lib.kf_peer_allgather(table.data_ptr(), region.data_ptr(), 2, 0, 1, mine.data_ptr(), 4, out.data_ptr(),
                                  status.data_ptr(), cfg, st)
    assert rc == C.OK  # the launch itself succeeds; the device reports
    assert kf.lib.kf_check(status.data_ptr(), None) == C.ERR_TIMEOUT
    header = status[:8].view(torch.int32).cpu().numpy()
    assert header[0] == C.ERR_TIMEOUT and header[1] == 1  # word 1: the rank whose element never came
    assert out.cpu().tolist() == [42, -1]  # the own element did arrive (through the own region)
    # bad arguments never reach the device
    assert kf.lib.kf_peer_allgather(table.data_ptr(), region.data_ptr(), 2, 0, 0, mine.data_ptr(), 4, out.data_ptr(),
                                    status.data_ptr(), None, st) == C.ERR_INVALID_ARG  # epoch 0 is reserved
    assert kf.lib.kf_peer_allgather(table.data_ptr(), region.data_ptr(), 65, 0, 1, mine.data_ptr(), 4, out.data_ptr(),
                                    status.data_ptr(), None, st) == C.ERR_INVALID_ARG
    assert kf.lib.kf_peer_allgather(table.data_ptr(), region.data_ptr(), 2, 0, 1, mine.data_ptr(), 3, out.data_ptr(),
                                    status.data_ptr(), None, st) == C.ERR_UNSUPPORTED
