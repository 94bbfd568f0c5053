"""A step made of several library calls recorded into a CUDA graph (`CapturedStep`) and replayed: the
replay does what the calls did, on whatever the tensors hold at replay time, with no host code of the
library in between."""
import numpy as np
import pytest
import torch

from util import to_dev, to_host

pytestmark = pytest.mark.gpu


def test_captured_step_replays_scan_mapreduce_and_sort(kf, oracle):
    n = 3_000_017
    rng = np.random.default_rng(31)
    x = to_dev(rng.integers(0, 256, n).astype(np.uint32))
    keys = to_dev(rng.integers(0, 1 << 32, n, dtype=np.uint64).astype(np.uint32))
    scanned, total, sorted_keys = torch.empty_like(x), torch.empty(1, dtype=x.dtype, device="cuda"), torch.empty_like(keys)
    tmp_scan = kf.get_allocation(kf.Scan1D, kf.identity, "+", x)
    tmp_red = kf.get_allocation(kf.MapReduce1D, kf.identity, "+", x)
    tmp_sort = kf.get_allocation(kf.Sort1D, keys)

    def step():
        kf.scan_("+", scanned, x, tmp=tmp_scan)
        kf.mapreduce_(kf.identity, "+", total, x, tmp=tmp_red)
        kf.sort_(sorted_keys, keys, tmp=tmp_sort)

    captured = kf.CapturedStep(step)
    assert captured.launches == 1 + 2 + 6  # scan kernel; header clear + reduction; histogram + bin scan + 4 passes
    before = int(kf.lib.kf_launch_count())
    for trial in range(3):  # new data in the same buffers, then one replay
        hx = rng.integers(0, 256, n).astype(np.uint32)
        hk = rng.integers(0, 1 << 32, n, dtype=np.uint64).astype(np.uint32)
        x.copy_(to_dev(hx))
        keys.copy_(to_dev(hk))
        scanned.zero_()
        sorted_keys.zero_()
        captured.replay()
        assert (to_host(scanned) == np.cumsum(hx, dtype=np.uint32)).all()
        assert int(to_host(total)[0]) == int(hx.sum(dtype=np.uint64) & 0xFFFFFFFF)
        assert (to_host(sorted_keys) == np.sort(hk)).all()
    assert int(kf.lib.kf_launch_count()) == before  # a replay does not pass through the library's host code
    for tmp in (tmp_scan, tmp_sort):
        assert kf.lib.kf_check(tmp.ptr(), None) == 0
