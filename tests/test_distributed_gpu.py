"""GPU tests of the sharded layer on 2 ranks (one process per GPU, NCCL): mapreduce, scan (also the
non-commutative affine operator) and the sample sort against the CPU oracle on the global array.
Skipped when fewer than two GPUs are visible. NVLS is switched off for the test processes."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_per, tmpdir):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    from conftest import load_package
    from oracle import oracle as O
    kf = load_package()
    from kernelforge_jl_b200 import distributed as kfd
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        group = kfd.ShardGroup()
        rng = np.random.default_rng(99)  # same global arrays on every rank
        n = n_per * world
        lo, hi = rank * n_per, (rank + 1) * n_per
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()

        xf = rng.random(n, dtype=np.float32)
        got = kfd.mapreduce(group, kf.identity, "+", dev(xf[lo:hi]))
        ref = float(xf.astype(np.float64).sum())
        assert abs(got - ref) <= 1e-5 * np.log2(n) * ref
        xi = rng.integers(-2**31, 2**31, n).astype(np.int32)
        assert kfd.mapreduce(group, kf.identity, "xor", dev(xi[lo:hi])) == int(np.bitwise_xor.reduce(xi))
        assert kfd.mapreduce(group, kf.identity, "max", dev(xi[lo:hi])) == int(xi.max())

        xu = rng.integers(0, 256, n).astype(np.int32)
        dst = torch.empty(n_per, dtype=torch.int32, device="cuda")
        kfd.scan_(group, "+", dst.view(torch.uint32), dev(xu[lo:hi]).view(torch.uint32))
        assert (dst.cpu().numpy() == np.cumsum(xu, dtype=np.int32)[lo:hi]).all()

        a = (0.5 + 0.5 * rng.random(n)).astype(np.float32)
        b = (2 * rng.random(n) - 1).astype(np.float32)
        ra, rb = O.c_scan_affine(a, b)
        da, db = torch.empty(n_per, device="cuda"), torch.empty(n_per, device="cuda")
        kfd.scan_(group, kf.AffineCompose(), (da, db), (dev(a[lo:hi]), dev(b[lo:hi])))
        tol = 1e-5 * np.log2(n)
        assert (np.abs(db.cpu().numpy() - rb[lo:hi]) <= tol * np.maximum(np.abs(rb[lo:hi]), 1.0)).all()
        assert (np.abs(da.cpu().numpy() - ra[lo:hi]) <= tol * np.maximum(ra[lo:hi], 4 * np.finfo(np.float32).tiny)).all()

        keys = rng.integers(0, 1 << 32, n, dtype=np.uint64).astype(np.uint32)
        keys[::7] = 12345  # a heavy duplicate
        for first in (True, False):  # cut the unsorted shard with one pass / sort it first
            chunk, counts = kfd.sort(group, dev(keys[lo:hi].view(np.int32)).view(torch.uint32), partition_first=first)
            assert sum(counts) == n and counts[rank] == chunk.numel()
            off = sum(counts[:rank])
            assert (chunk.view(torch.int32).cpu().numpy().view(np.uint32) == np.sort(keys)[off:off + counts[rank]]).all()
        fk = rng.standard_normal(n).astype(np.float32)  # float keys: order by the mapped bits
        chunk, counts = kfd.sort(group, dev(fk[lo:hi]))
        off = sum(counts[:rank])
        assert (chunk.cpu().numpy().view(np.uint32) == np.sort(fk)[off:off + counts[rank]].view(np.uint32)).all()
        k16 = rng.integers(-30000, 30000, n).astype(np.int16)  # 2-byte keys take the sort-first route
        chunk, counts = kfd.sort(group, dev(k16[lo:hi]))
        off = sum(counts[:rank])
        assert (chunk.cpu().numpy() == np.sort(k16)[off:off + counts[rank]]).all()
        torch.cuda.synchronize()
        group.close()
        with open(os.path.join(tmpdir, "ok%d" % rank), "w") as fh:
            fh.write("ok")
    finally:
        dist.destroy_process_group()


def test_sharded_primitives_on_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), 3_000_017, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / ("ok%d" % r)).exists()
