"""CPU tests of the sharded layer's exchange logic: world_size-2 and -3 `gloo` process groups, with
the local (per-shard) steps done by the CPU oracle instead of the CUDA kernels. What is tested is
what the layer adds on top of the kernels: partial combination, carry folding in rank order
(also for the non-commutative operator), splitter choice, run cutting, all-to-all sizes."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class HostOps:
    """LocalOps on host tensors through the oracle (test infrastructure only)."""

    def __init__(self, kfd, O):
        self.kfd, self.O = kfd, O
        self.opc = {"+": 0, "*": 1, "min": 2, "max": 3}

    def reduce(self, f, op, x, out=None):
        v = torch.tensor([self.O.c_mapreduce(0, self.opc[op], x.numpy())], dtype=x.dtype)
        if out is None:
            return v
        out.copy_(v)
        return out

    def fold(self, op, partials, g=None):
        return self.reduce(None, op, partials)

    def scan_(self, f, op, dst, src, init=None, tmp=None):
        from kernelforge_jl_b200 import ops
        if isinstance(op, ops.AffineCompose):
            if isinstance(src, (tuple, list)):
                a, b = src[0].numpy(), src[1].numpy()
            else:
                a, b = src[:, 0].contiguous().numpy(), src[:, 1].contiguous().numpy()
            seed = None
            if init is not None:  # (a, b) pairs of the shards before this one, folded left to right
                pa, pb = self.O.c_scan_affine(init[0::2].contiguous().numpy(), init[1::2].contiguous().numpy())
                seed = np.array([pa[-1], pb[-1]])
            oa, ob = self.O.c_scan_affine(a, b, init=seed)
            if isinstance(dst, (tuple, list)):
                dst[0].copy_(torch.from_numpy(oa).float())
                dst[1].copy_(torch.from_numpy(ob).float())
            else:
                dst[:, 0] = torch.from_numpy(oa).float()
                dst[:, 1] = torch.from_numpy(ob).float()
            return dst
        seed = None
        if init is not None:  # totals of the shards before this one, folded left to right
            seed = self.O.c_scan(0, self.opc[op], init.numpy())[-1]
        out = self.O.c_scan(0, self.opc[op], src.numpy(), init=seed)
        dst.copy_(torch.from_numpy(np.asarray(out)).to(dst.dtype))
        return dst

    def sort(self, x):
        return torch.from_numpy(self.O.c_sort(x.numpy()))

    def upper_bounds(self, sorted_keys, splitters):
        return torch.from_numpy(np.searchsorted(sorted_keys.numpy(), splitters.numpy(), side="right").astype(np.int64))

    def bucket_ids(self, x, splitters):
        u = self.O.np_uint_map(x.numpy())
        return torch.from_numpy(np.searchsorted(self.O.np_uint_map(splitters.numpy()), u, side="left").astype(np.uint8))

    def partition(self, ids, x):
        p = np.argsort(ids.numpy(), kind="stable")
        return x[torch.from_numpy(p)], ids[torch.from_numpy(p)]

    def take(self, x, positions):
        return x[positions]


def _worker(rank, world, port, n_per, tmpdir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from conftest import load_package
    from oracle import oracle as O
    load_package()
    from kernelforge_jl_b200 import distributed as kfd, ops
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        group = kfd.ShardGroup()
        host = HostOps(kfd, O)
        rng = np.random.default_rng(1234)  # the same global arrays on every rank; each takes its shard
        n = n_per * world
        lo, hi = rank * n_per, (rank + 1) * n_per

        gi = rng.integers(-1000, 1000, n).astype(np.int64)
        got = kfd.mapreduce(group, ops.identity, "+", torch.from_numpy(gi[lo:hi]), local=host)
        assert got == int(gi.sum())
        got = kfd.mapreduce(group, ops.identity, "max", torch.from_numpy(gi[lo:hi]), local=host)
        assert got == int(gi.max())

        gu = rng.integers(0, 256, n).astype(np.int32)
        dst = torch.empty(n_per, dtype=torch.int32)
        kfd.scan_(group, "+", dst, torch.from_numpy(gu[lo:hi]), local=host)
        assert (dst.numpy() == np.cumsum(gu, dtype=np.int32)[lo:hi]).all()
        # two arrays of one element size with one exchange: wrapping + over Int32 and min over Float32
        gf = rng.random(n).astype(np.float32)
        d1, d2 = torch.empty(n_per, dtype=torch.int32), torch.empty(n_per, dtype=torch.float32)
        kfd.scan_many_(group, [("+", d1, torch.from_numpy(gu[lo:hi])), ("min", d2, torch.from_numpy(gf[lo:hi]))], local=host)
        assert (d1.numpy() == np.cumsum(gu, dtype=np.int32)[lo:hi]).all()
        assert (d2.numpy() == np.minimum.accumulate(gf)[lo:hi]).all()

        a = (0.5 + 0.5 * rng.random(n)).astype(np.float32)
        b = (2 * rng.random(n) - 1).astype(np.float32)
        ra, rb = O.c_scan_affine(a, b)
        da, db = torch.empty(n_per), torch.empty(n_per)
        kfd.scan_(group, ops.AffineCompose(), (da, db), (torch.from_numpy(a[lo:hi]), torch.from_numpy(b[lo:hi])), local=host)
        assert np.abs(db.numpy() - rb[lo:hi]).max() < 1e-4 and np.abs(da.numpy() - ra[lo:hi]).max() < 1e-5

        keys = rng.integers(0, 1 << 31, n).astype(np.int32)
        keys[::5] = 7  # a heavy duplicate straddling the splitters
        for first in (True, False):  # cut the unsorted shard with one pass / sort it first
            chunk, counts = kfd.sort(group, torch.from_numpy(keys[lo:hi]), local=host, samples_per_rank=64, partition_first=first)
            assert sum(counts) == n and counts[rank] == chunk.numel()
            off = sum(counts[:rank])
            assert (chunk.numpy() == np.sort(keys)[off:off + counts[rank]]).all()
            assert max(counts) < 2.0 * n / world  # the heavy duplicate (20 % of the keys) lands in one piece
        k16 = rng.integers(-30000, 30000, n).astype(np.int16)  # 2-byte keys: sort-first route, carried as bytes
        chunk, counts = kfd.sort(group, torch.from_numpy(k16[lo:hi]), local=host, samples_per_rank=64)
        off = sum(counts[:rank])
        assert sum(counts) == n and (chunk.numpy() == np.sort(k16)[off:off + counts[rank]]).all()
        with open(os.path.join(tmpdir, "ok%d" % rank), "w") as fh:
            fh.write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_layer_over_gloo(world, tmp_path, oracle):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, 5003, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / ("ok%d" % r)).exists()


def test_splitter_choice(kf):
    from kernelforge_jl_b200 import distributed as kfd
    s = torch.arange(0, 4 * 8)
    assert kfd.choose_splitters(s, 4).tolist() == [8, 16, 24]
