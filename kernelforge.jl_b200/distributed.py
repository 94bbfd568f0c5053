"""Sharded (multi-GPU) mapreduce, scan and sample sort: one process per GPU over torch.distributed.

The reference has no multi-device layer; this one follows the plan the primitives suggest. Every
rank owns one contiguous shard of a global array (rank order = array order) and each primitive is
"local kernel(s) + ONE small exchange":

  mapreduce : local mapreduce -> the partials of all ranks -> fold in rank order -> g. On GPUs of one
              node the partials travel through peer memory (kf_peer_allgather: every rank stores its
              element into all ranks' mapped regions and waits, with a limit, for the others in its
              own); otherwise an allreduce (allgather + ordered fold for operators NCCL cannot reduce).
  scan      : local reduce -> allgather of the shard totals -> local scan seeded with the totals of
              the shards before it, which the scan kernel folds itself in rank order (12n bytes
              instead of the 16n of "scan, then fix up", and no kernel for the carry). `scan_many_`
              does this for several arrays with the allgathers running behind the local kernels. Non-commutative operators
              (AffineCompose) take the ordered route: local scan for the total, then the seeded scan.
  sort      : samples of the shard, allgather, identical splitter choice everywhere -> cut the shard
              into one run per destination -> all-to-all of the runs (NCCL, over NVLink) -> local
              onesweep sort of what arrived (keys only, so stable order is irrelevant and the result
              is bit-exact). The cut is "partition first" for 4- and 8-byte keys: destination ids
              (kf_bucket_ids) and ONE stable radix pass on those one-byte ids with the keys as the
              payload, about 0.4 of a full local sort; other key widths sort the shard first and
              cut it with kf_upper_bounds. On GPUs of one node the all-to-all is a PULL over NVLink:
              every rank partitions into an exchange buffer that the other ranks have mapped (CUDA
              IPC), and each rank copies its runs out of the peers' buffers with one asynchronous
              device-to-device copy per run (3 to 4 times the rate NCCL's send/recv all-to-all
              reached here); host tensors (the CPU tests) take `all_to_all_single`.

Remote data always lands in local HBM through NCCL before a kernel touches it. The local steps go
through `LocalOps`, whose default implementation calls the CUDA kernels; the CPU tests of the
exchange logic inject a host implementation instead (gloo backend).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _cabi as C
from . import ops
from .allocations import Scan1D, get_allocation
from .mapreduce import mapreduce_
from .scan import scan_ as _scan_
from .sort import sort_ as _sort_

SAMPLES_PER_RANK = 1024


class ShardGroup:
    """The ranks that share one sharded array (a torch.distributed process group)."""

    def __init__(self, group=None, peer_memory=None):
        """`peer_memory`: exchange shard totals and sample-sort runs through mapped peer memory (GPU
        ranks of one node) instead of the communication library. Default: on when the backend is NCCL."""
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self._scratch = {}
        self.peer_memory = (dist.get_backend(group) == "nccl") if peer_memory is None else bool(peer_memory)
        self._peer = None

    # ---- one-element allgather over peer memory (kf_peer_allgather) -----------------------------------
    def _peer_setup(self, device):
        import ctypes
        lib = C.load()
        nbytes = int(lib.kf_peer_region_bytes())
        with torch.cuda.device(device):
            mine = ctypes.c_void_p()
            C.check(lib.kf_xbuf_alloc(nbytes, ctypes.byref(mine)), "peer region")
            _as_tensor(mine.value, nbytes, torch.uint8, device).zero_()
            handle = (ctypes.c_ubyte * 64)()
            C.check(lib.kf_ipc_export(mine, handle), "peer region export")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=self.group)
            ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    ptrs.append(mine.value)
                    continue
                raw = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                ptr = ctypes.c_void_p()
                C.check(lib.kf_ipc_open(raw, ctypes.byref(ptr)), "peer region of rank %d" % r)
                ptrs.append(ptr.value)
            table = torch.tensor(ptrs, dtype=torch.int64, device=device)
            status = torch.zeros(256, dtype=torch.uint8, device=device)
            torch.cuda.synchronize()
        dist.barrier(group=self.group)  # every region is cleared and mapped before anybody writes into one
        self._peer = {"mine": mine.value, "ptrs": ptrs, "table": table, "status": status, "epoch": 0, "device": device}

    def peer_allgather(self, value, out=None):
        """`value`: one element (or a Float32 (a, b) pair) on the device. Returns the elements of all ranks
        in rank order, gathered by a kernel of the library over peer memory: no NCCL call, no host
        synchronisation. Every rank must call it in the same order (the epoch advances with each call)."""
        if self._peer is None:
            self._peer_setup(value.device)
        p = self._peer
        p["epoch"] = p["epoch"] % 0xFFFFFFFF + 1  # 1, 2, ..., never 0
        nb = value.numel() * value.element_size()
        if out is None:
            out = torch.empty(self.world * value.numel(), dtype=value.dtype, device=value.device)
        with torch.cuda.device(value.device):
            rc = C.load().kf_peer_allgather(p["table"].data_ptr(), p["mine"], self.world, self.rank, p["epoch"], value.data_ptr(), nb,
                                            out.data_ptr(), p["status"].data_ptr(), None, ops.stream_handle(value))
        C.check(rc, "peer_allgather")
        return out

    def check(self):
        """Synchronises and raises if an exchange kernel of this group gave up waiting for a rank."""
        if self._peer is not None:
            C.check(C.load().kf_check(self._peer["status"].data_ptr(), None), "sharded exchange")

    def _peer_release(self):
        if self._peer is None:
            return
        lib, p = C.load(), self._peer
        with torch.cuda.device(p["device"]):
            torch.cuda.synchronize()
            for r, ptr in enumerate(p["ptrs"]):
                if r != self.rank:
                    lib.kf_ipc_close(ptr)
            dist.barrier(group=self.group)
            lib.kf_xbuf_free(p["mine"])
        self._peer = None

    # ---- peer-memory exchange buffers (GPU ranks of one node) ---------------------------------------
    def exchange_buffers(self, nbytes, device):
        """This rank's exchange buffer of at least `nbytes` and the peers' mapped buffers, as raw device
        pointers (ints): (mine, [peer pointers by rank]). Collective: the ranks agree on the largest
        request first, so that all of them create (or keep) their buffers together. Buffers are created
        and mapped on first use and grow by re-creation."""
        import ctypes
        lib = C.load()
        want = torch.tensor([nbytes], dtype=torch.int64, device=device)
        dist.all_reduce(want, op=dist.ReduceOp.MAX, group=self.group)
        nbytes = int(want.item())
        have = getattr(self, "_xbuf", None)
        if have is not None and have["nbytes"] >= nbytes:
            return have["mine"], have["peers"]
        self.release_exchange_buffers()
        with torch.cuda.device(device):
            mine = ctypes.c_void_p()
            C.check(lib.kf_xbuf_alloc(nbytes, ctypes.byref(mine)), "exchange buffer")
            handle = (ctypes.c_ubyte * 64)()
            C.check(lib.kf_ipc_export(mine, handle), "exchange buffer export")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=self.group)
            peers = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    peers.append(mine.value)
                    continue
                raw = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                ptr = ctypes.c_void_p()
                C.check(lib.kf_ipc_open(raw, ctypes.byref(ptr)), "exchange buffer of rank %d" % r)
                peers.append(ptr.value)
        self._xbuf = {"nbytes": nbytes, "mine": mine.value, "peers": peers, "device": device}
        return mine.value, peers

    def release_exchange_buffers(self):
        """Unmaps the peers' buffers and frees this rank's (collective: all ranks call it together)."""
        have = getattr(self, "_xbuf", None)
        if have is None:
            return
        lib = C.load()
        with torch.cuda.device(have["device"]):
            torch.cuda.synchronize()
            for r, p in enumerate(have["peers"]):
                if r != self.rank:
                    lib.kf_ipc_close(p)
            dist.barrier(group=self.group)  # nobody frees a buffer that a peer still has mapped
            lib.kf_xbuf_free(have["mine"])
        self._xbuf = None

    def close(self):
        """Releases what the group holds on the device (collective)."""
        self.release_exchange_buffers()
        self._peer_release()
        self._scratch = {}

    def scratch(self, name, numel, dtype, device):
        """A small reusable tensor (partials, gathered totals): allocated once per (name, shape, type)."""
        key = (name, numel, dtype, device)
        t = self._scratch.get(key)
        if t is None:
            t = self._scratch[key] = torch.empty(numel, dtype=dtype, device=device)
        return t


class LocalOps:
    """Local (per-shard) steps on the GPU through libkf_b200.so."""

    def reduce(self, f, op, x, out=None):
        if out is None:
            out = torch.empty(1, dtype=x.dtype, device=x.device)
        return mapreduce_(f, op, out, x)

    def fold(self, op, partials, g=ops.identity):
        """op-reduction of a handful of partials (one per rank), then g."""
        out = torch.empty(1, dtype=partials.dtype, device=partials.device)
        return mapreduce_(ops.identity, op, out, partials, g=g)

    def scan_(self, f, op, dst, src, init=None, tmp=None):
        return _scan_(f, op, dst, src, init=init, tmp=tmp)

    def sort(self, x):
        return _sort_(torch.empty_like(x), x)

    def upper_bounds(self, sorted_keys, splitters):
        out = torch.empty(splitters.numel(), dtype=torch.int64, device=sorted_keys.device)
        with torch.cuda.device(sorted_keys.device):
            rc = C.load().kf_upper_bounds(ops.dtype_code(sorted_keys), sorted_keys.data_ptr(), sorted_keys.numel(),
                                          splitters.data_ptr(), splitters.numel(), out.data_ptr(),
                                          ops.stream_handle(sorted_keys))
        C.check(rc, "upper_bounds")
        return out

    def bucket_ids(self, x, splitters):
        """uint8 destination of every key: the number of splitters below it (in the sort's key order)."""
        out = torch.empty(x.numel(), dtype=torch.uint8, device=x.device)
        with torch.cuda.device(x.device):
            rc = C.load().kf_bucket_ids(ops.dtype_code(x), x.data_ptr(), x.numel(), splitters.data_ptr(),
                                        splitters.numel(), out.data_ptr(), ops.stream_handle(x))
        C.check(rc, "bucket_ids")
        return out

    def partition(self, ids, x, out=None):
        """x arranged by destination id (stable), and the sorted ids. `out` receives the arranged x."""
        vals, keys = _sort_(torch.empty_like(x) if out is None else out, x, keys=ids, keys_dst=torch.empty_like(ids))
        return vals, keys

    def take(self, x, positions):
        """x[positions] for a small index tensor (sample extraction). torch cannot index unsigned
        16/32/64-bit tensors, so the gather runs on the signed twin of the same bits."""
        return _bits_view(x)[positions].view(x.dtype)


_DEFAULT_OPS = LocalOps()
_NCCL_REDUCE = {C.OP_ADD: dist.ReduceOp.SUM, C.OP_MUL: dist.ReduceOp.PRODUCT, C.OP_MIN: dist.ReduceOp.MIN,
                C.OP_MAX: dist.ReduceOp.MAX}
_NCCL_DTYPES = {torch.float32, torch.float64, torch.int32, torch.int64, torch.uint8, torch.int8}


def _bits_view(t):
    """Unsigned 16/32/64-bit tensors as their signed twins (torch indexes and NCCL moves those)."""
    twin = {getattr(torch, "uint16", None): torch.int16, getattr(torch, "uint32", None): torch.int32,
            getattr(torch, "uint64", None): torch.int64}
    return t.view(twin[t.dtype]) if t.dtype in twin else t


def _wire_view(t):
    """What a collective carries: opaque bits. 2-byte integers travel as bytes (NCCL has no 16-bit
    integer type); returns the view and the number of wire elements per element."""
    t = _bits_view(t)
    if t.dtype == torch.int16:
        return t.view(torch.uint8), 2
    return t, 1


def all_gather_vec(group: ShardGroup, x):
    """Concatenation over ranks of equally sized 1-D tensors."""
    out = torch.empty(group.world * x.numel(), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(_wire_view(out)[0], _wire_view(x.contiguous())[0], group=group.group)
    return out


def gather_one(group: ShardGroup, value, out=None):
    """One element per rank (a shard total), in rank order, on every rank: through peer memory on GPUs of
    one node, else through the communication library."""
    if group.peer_memory and value.is_cuda and group.world <= 64 and value.numel() * value.element_size() <= 8:
        return group.peer_allgather(value, out=out)
    if out is None:
        return all_gather_vec(group, value)
    dist.all_gather_into_tensor(_wire_view(out)[0], _wire_view(value.contiguous())[0], group=group.group)
    return out


# ---- mapreduce -----------------------------------------------------------------------------------
def mapreduce(group: ShardGroup, f, op, x, *, g=ops.identity, local: LocalOps = _DEFAULT_OPS, to_cpu=True):
    """Global g(op-reduce f(x)) over all shards; every rank gets the value."""
    opcode = ops.op_code(op)
    if opcode == C.OP_AFFINE:
        raise C.ArgumentError("AffineCompose is not commutative: use scan")
    gcode = ops.post_code(g)
    part = local.reduce(f, op, x, out=group.scratch("partial", 1, x.dtype, x.device))
    if group.peer_memory and part.is_cuda and group.world <= 64:
        # partials of all ranks through peer memory, folded in rank order by one small kernel (with g):
        # deterministic, any operator, no communication-library call
        every = gather_one(group, part, out=group.scratch("partials", group.world, x.dtype, x.device))
        total = local.fold(op, every, g=g)
    elif opcode in _NCCL_REDUCE and part.dtype in _NCCL_DTYPES:
        dist.all_reduce(part, op=_NCCL_REDUCE[opcode], group=group.group)
        if gcode == C.POST_IDENTITY:
            total = part
        elif to_cpu:  # g on the host side of the read-back: no second kernel for one element
            v = part.cpu()[0].item()
            if gcode == C.POST_SQRT:
                return v ** 0.5
            raise C.ArgumentError("unknown post-map")
        else:
            total = local.fold(op, part, g=g)
    else:
        total = local.fold(op, all_gather_vec(group, part), g=g)
    return total.cpu()[0].item() if to_cpu else total


# ---- scan ----------------------------------------------------------------------------------------
def _unpack_scan_args(args):
    if len(args) == 3:
        return (ops.identity,) + tuple(args)
    return tuple(args)


def scan_(group: ShardGroup, *args, tmp=None, g=ops.identity, local: LocalOps = _DEFAULT_OPS):
    """Sharded `scan!([f,] op, dst, src)`: dst holds this rank's shard of the global inclusive scan."""
    f, op, dst, src = _unpack_scan_args(args)
    affine = isinstance(op, ops.AffineCompose)
    kw = {} if ops.post_code(g) == C.POST_IDENTITY else {"g": g}
    if group.world == 1:
        return local.scan_(f, op, dst, src, tmp=tmp, **kw)  # a single shard needs no carry
    if affine:
        # ordered route: the shard total is the last element of a local scan
        local.scan_(f, op, dst, src, tmp=tmp)
        if isinstance(dst, (tuple, list)):
            total = torch.stack([dst[0][-1], dst[1][-1]])
        else:
            total = dst[-1].clone()
        totals = gather_one(group, total)  # (a, b) pairs in rank order
        if group.rank == 0:
            return dst
        return local.scan_(f, op, dst, src, init=totals[: 2 * group.rank], tmp=tmp)
    total = local.reduce(f, op, src, out=group.scratch("partial", 1, src.dtype, src.device))
    totals = gather_one(group, total, out=group.scratch("totals", group.world, src.dtype, src.device))
    # the scan kernel folds the totals of the shards before this one itself (ninit = rank)
    init = totals[: group.rank] if group.rank > 0 else None
    return local.scan_(f, op, dst, src, init=init, tmp=tmp, **kw)


def scan_many_(group: ShardGroup, jobs, *, local: LocalOps = _DEFAULT_OPS):
    """Several sharded scans in one go: `jobs` are (op, dst, src) or (op, dst, src, tmp) tuples with
    elementwise operators (AffineCompose goes through `scan_`). Order of work: reduce job 0, exchange its
    total, reduce job 1, exchange its total, ..., then the seeded scans. On GPUs of one node the exchange
    is `kf_peer_allgather`, a kernel on the same stream (a few microseconds, no host involvement); with a
    communication library it is an asynchronous allgather that runs behind the next job's reduction."""
    if group.world == 1:
        return [local.scan_(ops.identity, j[0], j[1], j[2], tmp=j[3] if len(j) > 3 else None) for j in jobs]
    if any(isinstance(j[0], ops.AffineCompose) for j in jobs):
        raise C.ArgumentError("scan_many_ takes elementwise operators; use scan_ for AffineCompose")
    peer = group.peer_memory and jobs[0][2].is_cuda and group.world <= 64
    pending = []
    for i, j in enumerate(jobs):
        src = j[2]
        part = local.reduce(ops.identity, j[0], src, out=group.scratch("many_partial%d" % i, 1, src.dtype, src.device))
        totals = group.scratch("many_totals%d" % i, group.world, src.dtype, src.device)
        if peer:  # a kernel of the library on the same stream: nothing to wait for on the host side
            group.peer_allgather(part, out=totals)
            pending.append((None, totals))
        else:
            work = dist.all_gather_into_tensor(_wire_view(totals)[0], _wire_view(part)[0], group=group.group, async_op=True)
            pending.append((work, totals))
    outs = []
    for (work, totals), j in zip(pending, jobs):
        if work is not None:
            work.wait()
        # the scan kernel folds the totals of the shards before this one itself (ninit = rank)
        init = totals[: group.rank] if group.rank > 0 else None
        outs.append(local.scan_(ops.identity, j[0], j[1], j[2], init=init, tmp=j[3] if len(j) > 3 else None))
    return outs


# ---- sample sort ---------------------------------------------------------------------------------
class _RawCuda:
    """A device pointer dressed as a CUDA array, so that torch can alias the memory."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def _as_tensor(ptr, numel, dtype, device):
    """A torch tensor over `numel` elements at a raw device pointer (no ownership)."""
    if numel == 0:
        return torch.empty(0, dtype=dtype, device=device)
    nbytes = numel * torch.empty(0, dtype=dtype).element_size()
    return torch.as_tensor(_RawCuda(ptr, nbytes), device=device).view(dtype)


def _pull_runs(group, inbox, peers, count_matrix, elem_bytes):
    """Copies the runs addressed to this rank out of every rank's exchange buffer into `inbox` (in rank
    order), one asynchronous device-to-device copy per run, spread over a few streams; the peers' own
    streams are not involved. Ends with a stream-ordered barrier: a rank may overwrite its exchange buffer
    (the next sort) only after every peer has pulled from it."""
    lib = C.load()
    world, rank = group.world, group.rank
    cur = torch.cuda.current_stream(inbox.device)
    streams = getattr(group, "_pull_streams", None)
    if streams is None:
        streams = group._pull_streams = [torch.cuda.Stream(inbox.device) for _ in range(min(4, max(1, world - 1)))]
    for st in streams:
        st.wait_stream(cur)
    offsets = torch.cumsum(count_matrix, dim=1) - count_matrix  # [source][destination]: start of the run in the source
    dst_off = 0
    with torch.cuda.device(inbox.device):
        for k in range(world):
            src_rank = (rank + k) % world          # start with the local run, then walk the ring: spreads the load
            cnt = int(count_matrix[src_rank, rank])
            dst_off = int(count_matrix[:src_rank, rank].sum())
            if cnt == 0:
                continue
            st = streams[k % len(streams)]
            rc = lib.kf_copy_d2d(inbox.data_ptr() + dst_off * elem_bytes,
                                 peers[src_rank] + int(offsets[src_rank, rank]) * elem_bytes, cnt * elem_bytes, st.cuda_stream)
            C.check(rc, "exchange copy")
    for st in streams:
        cur.wait_stream(st)
    # stream-ordered (no host synchronisation): completes once every rank has enqueued it behind its pulls
    dist.all_reduce(group.scratch("pull_fence", 1, torch.int32, inbox.device), group=group.group)


def choose_splitters(sorted_samples, world: int):
    """world-1 splitters from the globally sorted samples: every world-th quantile."""
    per = sorted_samples.numel() // world
    pos = torch.arange(1, world, device=sorted_samples.device) * per
    return _bits_view(sorted_samples)[pos].view(sorted_samples.dtype)


def sample_positions(n: int, s: int, device):
    """s positions in [0, n): one per stratum of n/s elements, at a low-discrepancy offset inside it
    (so that periodic data does not alias with the stride)."""
    i = torch.arange(s, device=device, dtype=torch.float64)
    jitter = torch.remainder(i * 0.6180339887498949 + 0.5, 1.0)
    return ((i + jitter) * (n / s)).to(torch.int64).clamp_(0, max(n - 1, 0))


def sort(group: ShardGroup, x, *, local: LocalOps = _DEFAULT_OPS, samples_per_rank: int = SAMPLES_PER_RANK,
         partition_first=None):
    """Sample sort of the sharded keys `x`. Returns (sorted_chunk, counts): rank r holds the r-th
    contiguous piece of the globally sorted array; `counts` (host list) are the piece lengths.
    `partition_first` (default: for 4- and 8-byte keys) cuts the unsorted shard with one radix pass
    instead of sorting it first."""
    world, rank = group.world, group.rank
    n = x.numel()
    if world == 1:
        return local.sort(x), [n]
    if partition_first is None:
        partition_first = x.element_size() in (4, 8) and world <= 256
    s = samples_per_rank
    # On GPUs the runs are PULLED out of the peers' exchange buffers; `mine` then lives in this rank's one.
    pull = x.is_cuda and local is _DEFAULT_OPS
    peers = None
    if pull:
        my_ptr, peers = group.exchange_buffers(max(n, 1) * x.element_size(), x.device)
        xbuf = _as_tensor(my_ptr, n, x.dtype, x.device)
    if partition_first:
        # 1. samples of the unsorted shard (4x oversampled: they are not regular samples of a sorted run)
        s = 4 * samples_per_rank
        samples = local.take(x, sample_positions(n, s, x.device)) if n > 0 else torch.zeros(s, dtype=x.dtype, device=x.device)
        splitters = choose_splitters(local.sort(all_gather_vec(group, samples)), world)
        # 2. destination of every key, then one stable pass on the one-byte destinations with the keys as
        #    the payload. (A single pass that finds the destination itself, by binary search in the
        #    splitters at each of its three digit uses, was built and measured: 2.48 ms against
        #    0.37 + 1.48 ms at 2^28 keys and 7 splitters, so the two-step cut stays.)
        if pull:
            mine, ids = local.partition(local.bucket_ids(x, splitters), x, out=xbuf)
        else:
            mine, ids = local.partition(local.bucket_ids(x, splitters), x)
        dest = torch.arange(world - 1, dtype=torch.uint8, device=x.device)
        cuts = local.upper_bounds(ids, dest)
    else:
        # 1. regular samples of the sorted shard
        mine = _sort_(xbuf, x) if pull else local.sort(x)
        pos = ((torch.arange(s, device=x.device, dtype=torch.float64) + 0.5) * (n / s)).to(torch.int64).clamp_(0, max(n - 1, 0))
        samples = local.take(mine, pos) if n > 0 else torch.zeros(s, dtype=x.dtype, device=x.device)
        splitters = choose_splitters(local.sort(all_gather_vec(group, samples)), world)
        # 2. cut the sorted shard: run j goes to rank j
        cuts = local.upper_bounds(mine, splitters)
    bounds = torch.cat([torch.zeros(1, dtype=torch.int64, device=x.device), cuts,
                        torch.full((1,), n, dtype=torch.int64, device=x.device)])
    send_counts = bounds[1:] - bounds[:-1]
    # The gathered counts depend on every rank's cut, hence on every rank's arranged shard being complete:
    # once they are on the host, all exchange buffers may be read.
    count_matrix = all_gather_vec(group, send_counts).view(world, world).cpu()
    send = [int(v) for v in count_matrix[rank]]
    recv = [int(v) for v in count_matrix[:, rank]]
    # 3. all-to-all of the runs
    inbox = torch.empty(sum(recv), dtype=x.dtype, device=x.device)
    if pull:
        _pull_runs(group, inbox, peers, count_matrix, x.element_size())
    else:
        wire_in, per = _wire_view(inbox)
        dist.all_to_all_single(wire_in, _wire_view(mine)[0], output_split_sizes=[per * v for v in recv],
                               input_split_sizes=[per * v for v in send], group=group.group)
    # 4. one local sort of what arrived
    out = local.sort(inbox) if inbox.numel() else inbox
    counts = [int(v) for v in count_matrix.sum(dim=0)]
    return out, counts


# ---- host-buffer pipeline (end-to-end path) --------------------------------------------------------
class HostScanPipeline:
    """`scan!` for arrays that live in pinned HOST memory.

    The arrays are cut into chunks that flow through a small ring of device staging slots: chunk c is
    copied in on one stream, scanned on a second stream with `init` = the last output element of
    chunk c-1 (still in its slot), and copied out on a third, so both PCIe directions and the kernel
    overlap. Several arrays given to `scan_host_many` form ONE stream of chunks (the carry restarts
    at every array), so the pipeline fills and drains once per call, not once per array. Device
    memory: 2 * slots * chunk_bytes, whatever the array sizes; slots are guarded by events.
    """

    def __init__(self, kf_module, max_n: int, chunks: int = 0, device=None, chunk_bytes: int = 32 << 20, slots: int = 4):
        self.kf = kf_module
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.max_n = max_n
        if chunks:  # sized by a chunk count for the largest array (8-byte elements), as earlier versions were
            chunk_bytes = max(1 << 20, -(-(max_n * 8) // chunks))
        self.chunk_bytes = (chunk_bytes + 255) // 256 * 256
        self.slots = max(2, slots)
        self.stage_in = [torch.empty(self.chunk_bytes, dtype=torch.uint8, device=self.device) for _ in range(self.slots)]
        self.stage_out = [torch.empty(self.chunk_bytes, dtype=torch.uint8, device=self.device) for _ in range(self.slots)]
        self.in_free = [None] * self.slots   # event: the scan has read stage_in[k]
        self.out_free = [None] * self.slots  # event: the copy-out has read stage_out[k]
        self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        self.counter = 0
        self._tmp = {}

    def scan_host(self, op, dst_host, src_host, f=ops.identity):
        return self.scan_host_many([(op, dst_host, src_host, f)])[0]

    def scan_host_many(self, jobs):
        """jobs: (op, dst_host, src_host[, f]) tuples, scanned independently, pipelined as one stream."""
        cur = torch.cuda.current_stream(self.device)
        for st in (self.s_in, self.s_cmp, self.s_out):
            st.wait_stream(cur)
        outs = []
        for job in jobs:
            op, dst_host, src_host = job[0], job[1], job[2]
            f = job[3] if len(job) > 3 else ops.identity
            n = src_host.numel()
            if n > self.max_n or src_host.element_size() > 8:
                raise C.ArgumentError("HostScanPipeline was sized for %d elements of at most 8 bytes" % self.max_n)
            if dst_host.numel() != n or dst_host.dtype != src_host.dtype:
                raise C.ArgumentError("dst and src must match in length and element type")
            dt, es = src_host.dtype, src_host.element_size()
            per = self.chunk_bytes // es
            carry = None
            lo = 0
            while lo < n:
                hi = min(n, lo + per)
                k = self.counter % self.slots
                self.counter += 1
                d_in = self.stage_in[k][: (hi - lo) * es].view(dt)
                d_out = self.stage_out[k][: (hi - lo) * es].view(dt)
                key = (dt, hi - lo)
                if key not in self._tmp:
                    self._tmp[key] = get_allocation(Scan1D, f, op, d_in)
                with torch.cuda.stream(self.s_in):
                    if self.in_free[k] is not None:
                        self.s_in.wait_event(self.in_free[k])
                    d_in.copy_(src_host[lo:hi], non_blocking=True)
                    arrived = self.s_in.record_event()
                with torch.cuda.stream(self.s_cmp):
                    self.s_cmp.wait_event(arrived)
                    if self.out_free[k] is not None:
                        self.s_cmp.wait_event(self.out_free[k])
                    _scan_(f, op, d_out, d_in, init=carry, tmp=self._tmp[key])
                    scanned = self.s_cmp.record_event()
                self.in_free[k] = scanned
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(scanned)
                    dst_host[lo:hi].copy_(d_out, non_blocking=True)
                    self.out_free[k] = self.s_out.record_event()
                carry = d_out[hi - lo - 1: hi - lo]  # read by the next chunk's scan, long before the slot is reused
                lo = hi
            outs.append(dst_host)
        cur.wait_stream(self.s_out)
        return outs
