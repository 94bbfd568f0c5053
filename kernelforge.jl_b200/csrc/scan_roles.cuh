// Persistent look-back scan for sm_100a that never waits for the look-back: every tile is read
// twice, K tiles apart. The first read (from HBM, by the bulk-copy engine into a shared-memory
// ring) only feeds a reduction, so the tile's AGGREGATE is published K tile-times before the tile
// is scanned; the second read (plain 128-bit loads) finds the tile in L2, which comfortably holds
// the K * (number of SMs) tiles in between. HBM traffic stays at one read and one write per
// element, and the latency of the descriptor round trips (1.5-2 us each when the memory system is
// saturated) is covered by those K tile-times instead of by tiles parked in shared memory.
//
// One CTA per SM, three kinds of warps; the CTA's j-th tile is "step j":
//
//   loader   (one lane)  takes a ticket per step, records (tile id, first element, count) in the
//       step ring and starts the tile's bulk load into data buffer j mod NBUF as soon as the
//       scanners have released it. The buffers are released right after the reduction, so all of
//       them serve as prefetch depth.
//
//   scanners (THREADS threads), every warp on its own, without CTA barriers:
//       for j = 0, 1, ...:  issue the loads of S(j);  R(j + K);  finish S(j)
//     R(s)  wait for the buffer, reduce this warp's 32*VECS slots, release the buffer, leave the
//           warp total in the step ring, arrive on `totals[s]`.
//     S(s)  128-bit loads of the warp's slots (striped: lane l holds slots v*32 + l, so loads and
//           stores are fully coalesced), wait for `base[s]`, scan in registers with shuffles,
//           combine with the tile's exclusive prefix and the warp's prefix, streaming stores.
//
//   resolvers (NRES warps; resolver q owns steps q, q + NRES, ...):
//     1  when `totals[s]` completes: scan the warp totals (one shuffle scan), store the warps'
//        exclusive prefixes, publish the tile AGGREGATE in the global descriptor array.
//     2  once step s + LAG has been reduced (so that the predecessors have normally published): the
//        step's exclusive prefix = the inclusive prefix of this resolver's PREVIOUS step combined with
//        the AGGREGATES of the tiles in between (about NRES * gridDim.x of them), read DEPTH coalesced
//        rows of 32 descriptors per round trip. Nobody's inclusive prefix is ever read from global
//        memory, so resolving a tile depends on no other CTA having resolved anything. The resolver
//        stores the exclusive prefix and arrives on `base[s]`. A window with a descriptor that is not
//        yet published is simply read again; step 1 of later steps is never held up by that.
//
// Dependencies only ever point to smaller tile ids (tickets are handed out in order, every CTA is
// resident, and reductions depend on nothing but loads), so the protocol cannot deadlock. Every
// wait is bounded and abort-aware: a wait that runs out records KF_ERR_TIMEOUT, raises the CTA's
// abort flag and poisons the tiles the CTA holds; a poisoned descriptor makes later tiles give up.
//
// Only whole tiles of 16-byte aligned arrays take the vector paths; the short head tile of a
// misaligned view and the ragged last tile use element-wise accesses inside the same loop.
//
// Floating point: the aggregate comes from the reduction and the outputs from the scan, which
// associate the additions differently; the carried prefix and the tile's own last output may
// differ in the last bits, as the outputs of any two summation orders do. Integer results are exact.
#pragma once

#include "scan_tma.cuh"

namespace kf {

template <typename Arrays, typename T, int THREADS, int VECS, int NBUF, int K> struct ScanRolesSmem {
    static constexpr int WARPS = THREADS / 32;
    static constexpr int NSTEP = NBUF + K + 1;  // steps that can be alive at once: loaded, reduced, waiting for S
    static constexpr int ARR_BYTES = THREADS * VECS * 16;
    static constexpr int BUF_BYTES = Arrays::NARR * ARR_BYTES;
    static constexpr size_t kData = (size_t)NBUF * BUF_BYTES;
    // 8-byte words behind the data: full, empty [NBUF] (mbarriers); per step slot [NSTEP]: totals,
    // base (mbarriers), ticket, start, count, tile total, tile exclusive prefix; warp totals and
    // warp exclusive prefixes [NSTEP][WARPS]. Then 4-byte words: abort flag, steps armed, end step.
    static constexpr size_t kWords = 2 * NBUF + 7 * NSTEP + 2 * (size_t)NSTEP * WARPS;
    static constexpr size_t kBytes = kData + 8 * kWords + 16;
};

// Bounded wait that also gives up when the CTA's abort flag is raised. Returns true when the
// barrier phase completed.
__device__ __forceinline__ bool mbar_wait_or_abort(u64 *bar, u32 parity, const int *s_abort) {
    for (u32 spins = 0; spins < kSpinLimit; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & 31) == 31) {
            if (*reinterpret_cast<const volatile int *>(s_abort)) return false;
            __nanosleep(32);
        }
    }
    return false;
}
__device__ __forceinline__ bool mbar_test_wait(u64 *bar, u32 parity) {
    u32 ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(smem_addr(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
// The same for a whole warp (all 32 lanes must call it): one answer for every lane, so that the
// warp-wide shuffles that follow never miss a lane.
__device__ __forceinline__ bool mbar_wait_or_abort_warp(u64 *bar, u32 parity, const int *s_abort) {
    return __all_sync(0xFFFFFFFFu, mbar_wait_or_abort(bar, parity, s_abort));
}

// Combination of the values of all lanes in ASCENDING lane order (lane 0 is the leftmost operand),
// valid in every lane.
template <typename T, typename Op> __device__ __forceinline__ T warp_fold_ascending(T x, u32 lane) {
    if constexpr (Op::commutative) {
        return warp_fold_descending<T, Op>(x, lane);
    } else {
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            T y = shfl_up(x, d);
            y = lane >= (u32)d ? y : Op::template identity<T>();
            x = Op::template apply<T>(y, x);
        }
        return shfl_idx(x, 31);
    }
}

template <typename T, typename Op, typename Access, typename Arrays, int THREADS, int VECS, int NBUF, int K, int DEPTH, int NRES, int LAG,
          bool PACKED = false>
__global__ void __launch_bounds__(THREADS + 32 + 32 * NRES) scan_kernel_roles(Access acc, Arrays arr, ScanArgs args) {
    // PACKED: one-byte elements under `+` (wrap-around, so signed and unsigned alike) with f = g =
    // identity stay packed, four elements per register: sums by dp4a, prefixes in two 16-bit lanes per
    // word (byte_sum16 / byte_prefix16). It is an instantiation of its own because the per-element
    // code needs a register per BYTE (64 to 128 of them), costs 11.6 instructions per element and is
    // issue-bound at 0.68 of the copy rate.
    static_assert(!PACKED || (sizeof(T) == 1 && std::is_same<Op, OpAdd>::value && Arrays::NARR == 1), "PACKED is the byte-add form");
    using SM = ScanRolesSmem<Arrays, T, THREADS, VECS, NBUF, K>;
    constexpr int EPV = Arrays::EPV;
    constexpr int NARR = Arrays::NARR;
    constexpr int WARPS = THREADS / 32;
    constexpr int NSTEP = SM::NSTEP;
    constexpr u64 TILE = (u64)THREADS * VECS * EPV;
    static_assert(NBUF >= 1 && K >= 1, "ring too small");
    static_assert(sizeof(T) <= 8, "totals are staged as 8-byte words");
    static_assert(WARPS + 1 + NRES <= 32, "scanners + loader + resolvers must fit in one CTA");
    static_assert(NRES >= 1 && NRES <= NSTEP, "a resolver must have finished step s-NSTEP before it tests step s");
    static_assert(LAG < K && LAG < NSTEP, "the reductions run only K steps in front of the step being scanned");

    extern __shared__ __align__(128) unsigned char smem[];
    u64 *words = reinterpret_cast<u64 *>(smem + SM::kData);
    u64 *s_full = words;                    // [NBUF]  loader -> scanners: tile data (or nothing, for element-wise tiles) is in the buffer
    u64 *s_empty = words + NBUF;            // [NBUF]  scanners -> loader: buffer may be refilled
    u64 *s_totals = words + 2 * NBUF;       // [NSTEP] scanners -> resolver: all warp totals of the step are stored
    u64 *s_base = s_totals + NSTEP;         // [NSTEP] resolver -> scanners: the step's exclusive prefix is stored
    u64 *s_ticket = s_base + NSTEP;         // [NSTEP] tile id of the step (>= ntiles: end marker)
    u64 *s_start = s_ticket + NSTEP;        // [NSTEP] first element of the tile
    u64 *s_count = s_start + NSTEP;         // [NSTEP] elements in the tile
    u64 *s_tile_total = s_count + NSTEP;    // [NSTEP]
    u64 *s_tile_excl = s_tile_total + NSTEP;  // [NSTEP]
    u64 *s_warp_total = s_tile_excl + NSTEP;                  // [NSTEP][WARPS]
    u64 *s_warp_excl = s_warp_total + (size_t)NSTEP * WARPS;  // [NSTEP][WARPS]
    int *s_abort = reinterpret_cast<int *>(words + SM::kWords);
    u32 *s_issued = reinterpret_cast<u32 *>(s_abort + 1);
    u32 *s_end = s_issued + 1;  // step that carries the end marker (0xFFFFFFFF until the loader knows)
    auto slot_ref = [](u64 *w) -> T & { return *reinterpret_cast<T *>(w); };

    const u32 tid = threadIdx.x, lane = lane_id(), warp = tid >> 5;
    const u64 first = args.head > 0 ? 1 : 0;

    if (tid == 0) {
        for (int b = 0; b < NBUF; ++b) {
            mbar_init(&s_full[b], 1);
            mbar_init(&s_empty[b], WARPS);
        }
        for (int q = 0; q < NSTEP; ++q) {
            mbar_init(&s_totals[q], WARPS);
            mbar_init(&s_base[q], 1);
        }
        *s_abort = ld_relaxed_u32(&args.header[kStatusWord]) != 0u;
        *s_issued = 0;
        *s_end = 0xFFFFFFFFu;
        fence_async_proxy();  // barrier init visible to the bulk-copy engine
    }
    __syncthreads();

    // A wait that ran out (not one that was aborted) is this CTA's own failure: record it.
    auto wait_failed = [&](u32 where) {
        if (*reinterpret_cast<volatile int *>(s_abort) == 0) {
            record_error(args.header, KF_ERR_TIMEOUT, where);
            *reinterpret_cast<volatile int *>(s_abort) = 2;
        }
    };

    if (warp == WARPS) {
        // ======================= loader =========================================================
        if (lane == 0) {
            u32 pending = atomicAdd(&args.header[kTicketBase], 1u);
            for (u32 j = 0;; ++j) {
                const u32 b = j % NBUF, q = j % NSTEP;
                // buffer b free again means every warp has reduced step j-NBUF, hence finished S(j-NBUF-K-1):
                // step slot q (last used by step j-NSTEP) is free as well
                if (j >= (u32)NBUF && !mbar_wait_or_abort(&s_empty[b], ((j / NBUF) - 1) & 1, s_abort)) {
                    wait_failed(0xFFFFFFFEu);
                    break;
                }
                if (*reinterpret_cast<volatile int *>(s_abort)) break;
                const u64 t = pending;
                u64 start = 0, count = 0;
                if (t < args.ntiles) {
                    if (t < first) {
                        count = args.head;
                    } else {
                        start = args.head + (t - first) * TILE;
                        count = args.n - start < TILE ? args.n - start : TILE;
                    }
                }
                s_ticket[q] = t;
                s_start[q] = start;
                s_count[q] = count;
                *reinterpret_cast<volatile u32 *>(s_issued) = j + 1;
                if (t >= args.ntiles) {
                    *reinterpret_cast<volatile u32 *>(s_end) = j;
                    mbar_arrive(&s_full[b]);  // the end marker travels through the ring like a tile
                    break;
                }
                pending = atomicAdd(&args.header[kTicketBase], 1u);  // used one step from now
                if (count == TILE) {
                    const u64 off = start * Arrays::elem_bytes;
                    unsigned char *buf = smem + (size_t)b * SM::BUF_BYTES;
                    mbar_expect_tx(&s_full[b], (u32)SM::BUF_BYTES);
#pragma unroll
                    for (int a = 0; a < NARR; ++a)
                        bulk_load(buf + a * SM::ARR_BYTES, arr.src[a] + off, (u32)SM::ARR_BYTES, &s_full[b]);
                } else {
                    mbar_arrive(&s_full[b]);  // element-wise tile: nothing to load
                }
            }
        }
    } else if (warp > WARPS) {
        // ======================= resolvers ======================================================
        // Resolver q carries its own running prefix over the steps q, q + NRES, ...: the exclusive
        // prefix of a step is the inclusive prefix of the resolver's previous step combined with the
        // AGGREGATES of the tiles in between (about NRES * gridDim.x of them). Nobody's inclusive prefix
        // is ever read, so resolving a tile does not depend on any other CTA having resolved anything.
        u32 j = warp - (WARPS + 1);  // next step of this resolver to aggregate
        u32 r = j;                   // next step of this resolver to resolve
        bool more = true, ok = true;
        bool fresh = true;        // the look-back of step r has not started
        bool gate_seen = false;   // the gate of step r has opened
        u64 R = 0;                // tile id of step r
        long long hi = 0, lo = 0; // tiles lo..hi are still to be folded (nearest first)
        long long prev_tile = -1; // tile of this resolver's previous step
        T prev_incl = Op::template identity<T>();  // and its inclusive prefix
        bool have_prev = false;
        T acc_r = Op::template identity<T>();
        u32 spins = 0, idle = 0;
        while (ok) {
            // ---- step 1: aggregate of step j, when the scanners are done with it. Never blocks. --------
            if (more) {
                const u32 q = j % NSTEP, par = (j / NSTEP) & 1;
                const bool ready = __all_sync(0xFFFFFFFFu, mbar_test_wait(&s_totals[q], par));
                if (!ready) {
                    // steps after the end marker never come
                    if (__any_sync(0xFFFFFFFFu, *reinterpret_cast<volatile u32 *>(s_end) < j)) more = false;
                    else if (r >= j || (LAG > 0 && !gate_seen)) {  // nothing to do but wait
                        if (++idle > kSpinLimit) {
                            if (lane == 0) wait_failed(0xFFFFFFFCu);
                            break;
                        }
                        if ((idle & 15) == 15 && __any_sync(0xFFFFFFFFu, *reinterpret_cast<volatile int *>(s_abort) != 0)) break;
                        __nanosleep(40);
                    }
                }
                if (ready) {
                    const u64 tile = s_ticket[q];
                    if (tile >= args.ntiles) {
                        more = false;
                    } else {
                        T incl = lane < (u32)WARPS ? slot_ref(&s_warp_total[q * WARPS + lane]) : Op::template identity<T>();
#pragma unroll
                        for (int d = 1; d < 32; d <<= 1) {
                            T up = shfl_up(incl, d);
                            up = lane >= (u32)d ? up : Op::template identity<T>();
                            incl = Op::template apply<T>(up, incl);
                        }
                        T before = shfl_up(incl, 1);
                        before = lane == 0 ? Op::template identity<T>() : before;
                        if (lane < (u32)WARPS) slot_ref(&s_warp_excl[q * WARPS + lane]) = before;
                        const T total = shfl_idx(incl, 31);
                        if (lane == 0) {
                            slot_ref(&s_tile_total[q]) = total;
                            // (test hook: a muted tile keeps its aggregate to itself)
                            if (!(args.mute_tile && tile + 1 == (u64)args.mute_tile)) Desc<T>::publish(args.desc, tile, kAggregate, total);
                        }
                        j += NRES;
                        idle = 0;
                    }
                }
            }
            // ---- step 2: one round trip of the look-back of step r ------------------------------------
            // gate: step r + LAG (any resolver's) has been reduced, or the tiles end before it
            bool gate = r < j;
            if (LAG > 0 && gate && !gate_seen) {
                const u32 g = r + LAG;
                gate = __any_sync(0xFFFFFFFFu, *reinterpret_cast<volatile u32 *>(s_end) <= g) ||
                       __all_sync(0xFFFFFFFFu, mbar_test_wait(&s_totals[g % NSTEP], (g / NSTEP) & 1));
                gate_seen = gate;
            }
            if (gate) {
                const u32 rq = r % NSTEP;
                if (fresh) {
                    R = s_ticket[rq];
                    hi = (long long)R - 1;
                    lo = prev_tile + 1;
                    acc_r = Op::template identity<T>();
                    spins = 0;
                    fresh = false;
                }
                bool resolved = hi < lo;
                if (!resolved) {
                    // Row d of the window holds tiles hi - 32*d - lane (nearest first; a row is 256 contiguous
                    // bytes, one coalesced load). Tiles before `lo` are already part of prev_incl.
                    u32 st[DEPTH];
                    T val[DEPTH];
#pragma unroll
                    for (int d = 0; d < DEPTH; ++d) {
                        const long long t = hi - (long long)(d * 32 + lane);
                        val[d] = Op::template identity<T>();
                        st[d] = t >= lo ? Desc<T>::read(args.desc, (u64)t, val[d]) : (u32)kAggregate;
                        if (t < lo) val[d] = Op::template identity<T>();
                    }
                    bool missing = false, poisoned = false;
#pragma unroll
                    for (int d = 0; d < DEPTH; ++d) {
                        missing = missing || st[d] == kInvalid;
                        poisoned = poisoned || st[d] == kPoison;
                    }
                    missing = __any_sync(0xFFFFFFFFu, missing);
                    poisoned = __any_sync(0xFFFFFFFFu, poisoned);
                    if (poisoned) {
                        ok = false;
                    } else if (missing) {  // a predecessor has not published yet: come back
                        ++spins;
                        if (spins > args.spin_limit) {
                            if (lane == 0) wait_failed((u32)R);
                            ok = false;
                        } else if ((spins & 15) == 15 && *reinterpret_cast<volatile int *>(s_abort)) {
                            ok = false;
                        } else if (spins > 8) {
                            __nanosleep(spins > 64 ? 256 : 32);
                        }
                    } else {
                        T window;  // tiles max(lo, hi - 32*DEPTH + 1) .. hi, in array order
                        if constexpr (Op::commutative) {
                            T acc_l = val[0];
#pragma unroll
                            for (int d = 1; d < DEPTH; ++d) acc_l = Op::template apply<T>(val[d], acc_l);
                            window = warp_fold_descending<T, Op>(acc_l, lane);
                        } else {
                            window = warp_fold_descending<T, Op>(val[0], lane);
#pragma unroll
                            for (int d = 1; d < DEPTH; ++d) window = Op::template apply<T>(warp_fold_descending<T, Op>(val[d], lane), window);
                        }
                        acc_r = Op::template apply<T>(window, acc_r);
                        hi -= 32 * DEPTH;
                        spins = 0;
                        resolved = hi < lo;
                    }
                }
                if (resolved) {
                    T excl = acc_r;
                    if (have_prev) excl = Op::template apply<T>(prev_incl, acc_r);
                    else if (args.init && args.ninit) excl = Op::template apply<T>(fold_init<T, Op>(args), acc_r);
                    prev_incl = Op::template apply<T>(excl, slot_ref(&s_tile_total[rq]));
                    prev_tile = (long long)R;
                    have_prev = true;
                    if (lane == 0) {
                        slot_ref(&s_tile_excl[rq]) = excl;
                        mbar_arrive(&s_base[rq]);
                    }
                    r += NRES;
                    fresh = true;
                    gate_seen = false;
                }
            } else if (!more && r >= j) {
                break;
            }
        }
        if (!ok && lane == 0 && *reinterpret_cast<volatile int *>(s_abort) == 0) *reinterpret_cast<volatile int *>(s_abort) = 1;
    } else {
        // ======================= scanners =======================================================
        const u32 warp_slot0 = warp * 32 * VECS;

        // R(s): 0 = reduced, 1 = end of tiles, 2 = gave up
        auto reduce_step = [&](u32 s) -> int {
            const u32 b = s % NBUF, q = s % NSTEP;
            if (!mbar_wait_or_abort_warp(&s_full[b], (s / NBUF) & 1, s_abort)) {
                if (lane == 0) wait_failed(0xFFFFFFFBu);
                return 2;
            }
            const u64 tile = s_ticket[q];
            if (tile >= args.ntiles) {
                if (lane == 0) mbar_arrive(&s_totals[q]);  // the resolver learns of the end the same way
                return 1;
            }
            const u64 start = s_start[q], count = s_count[q];
            const unsigned char *buf = smem + (size_t)b * SM::BUF_BYTES;
            T rowsum[VECS];
            if (count == TILE) {
#pragma unroll
                for (int v = 0; v < VECS; ++v) {
                    uint4 raw[NARR];
                    T e[EPV];
                    const u32 slot = warp_slot0 + v * 32 + lane;
#pragma unroll
                    for (int a = 0; a < NARR; ++a) raw[a] = *reinterpret_cast<const uint4 *>(buf + a * SM::ARR_BYTES + slot * 16);
                    if constexpr (PACKED) {
                        rowsum[v] = (T)byte_sum16(raw[0]);
                    } else {
                        Arrays::unpack(raw, e);
                        if (args.f != KF_MAP_IDENTITY) {
#pragma unroll
                            for (int k = 0; k < EPV; ++k) e[k] = map_elem<T>(args.f, e[k]);
                        }
                        rowsum[v] = e[0];
#pragma unroll
                        for (int k = 1; k < EPV; ++k) rowsum[v] = Op::template apply<T>(rowsum[v], e[k]);
                    }
                }
            } else {
#pragma unroll
                for (int v = 0; v < VECS; ++v) {
                    rowsum[v] = Op::template identity<T>();
#pragma unroll
                    for (int k = 0; k < EPV; ++k) {
                        const u64 off = (u64)(warp_slot0 + v * 32 + lane) * EPV + k;
                        const T x = off < count ? map_elem<T>(args.f, acc.load_elem(start + off)) : Op::template identity<T>();
                        rowsum[v] = Op::template apply<T>(rowsum[v], x);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[b]);  // this warp has read its part of the buffer
            T total;
            if constexpr (Op::commutative) {
                T mine = rowsum[0];
#pragma unroll
                for (int v = 1; v < VECS; ++v) mine = Op::template apply<T>(mine, rowsum[v]);
                total = warp_fold_ascending<T, Op>(mine, lane);
            } else {  // element order is (row, lane, component)
                total = warp_fold_ascending<T, Op>(rowsum[0], lane);
#pragma unroll
                for (int v = 1; v < VECS; ++v) total = Op::template apply<T>(total, warp_fold_ascending<T, Op>(rowsum[v], lane));
            }
            if (lane == 0) {
                slot_ref(&s_warp_total[q * WARPS + warp]) = total;
                mbar_arrive(&s_totals[q]);
            }
            return 0;
        };

        bool more = true, go = true;
#pragma unroll 1
        for (u32 s = 0; s < (u32)K && more; ++s) {
            const int rr = reduce_step(s);
            more = rr == 0;
            go = rr != 2;
        }
#pragma unroll 1
        for (u32 s = 0; go; ++s) {
            // ---- S(s), first half: the loads (they hit L2) ------------------------------------------
            const u32 q = s % NSTEP;
            const u64 tile = s_ticket[q];  // bound: the loader reuses the slot only after every warp finished S(s)
            if (tile >= args.ntiles) break;
            const u64 start = s_start[q], count = s_count[q];
            const bool fast = count == TILE;
            if constexpr (PACKED) {
                // the ragged last tile builds its vectors from single bytes (zeros past the end)
                uint4 rv[VECS];
#pragma unroll
                for (int v = 0; v < VECS; ++v) {
                    const u64 off0 = (u64)(warp_slot0 + v * 32 + lane) * 16;
                    if (fast) {
                        rv[v] = ld_v4(arr.src[0] + start + off0);
                    } else {
                        u32 w[4] = {0, 0, 0, 0};
#pragma unroll
                        for (int k = 0; k < 16; ++k)
                            if (off0 + k < count) w[k >> 2] |= (u32)(uint8_t)acc.load_elem(start + off0 + k) << (8 * (k & 3));
                        rv[v] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
                if (more) {
                    const int rr = reduce_step(s + K);
                    more = rr == 0;
                    if (rr == 2) break;
                }
                T tot[VECS][1], slot_excl[VECS];
#pragma unroll
                for (int v = 0; v < VECS; ++v) tot[v][0] = (T)byte_sum16(rv[v]);
                (void)warp_tile_scan<T, Op, VECS, 1>(tot, slot_excl, lane);
                if (!mbar_wait_or_abort_warp(&s_base[q], (s / NSTEP) & 1, s_abort)) {
                    if (lane == 0) wait_failed(0xFFFFFFFAu);
                    break;
                }
                const T base = Op::template apply<T>(slot_ref(&s_tile_excl[q]), slot_ref(&s_warp_excl[q * WARPS + warp]));
#pragma unroll
                for (int v = 0; v < VECS; ++v) {
                    const u64 off0 = (u64)(warp_slot0 + v * 32 + lane) * 16;
                    const uint4 o = byte_prefix16(rv[v], (u32)(uint8_t)Op::template apply<T>(base, slot_excl[v]));
                    if (fast) {
                        st_stream_v4(arr.dst[0] + start + off0, o);
                    } else {
                        const u32 w[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                        for (int k = 0; k < 16; ++k)
                            if (off0 + k < count) acc.store_elem(start + off0 + k, (T)(w[k >> 2] >> (8 * (k & 3))));
                    }
                }
                continue;
            }
            T e[VECS][EPV];
            if (fast) {
#pragma unroll
                for (int v = 0; v < VECS; ++v) {
                    uint4 raw[NARR];
#pragma unroll
                    for (int a = 0; a < NARR; ++a)
                        raw[a] = ld_v4(arr.src[a] + start * Arrays::elem_bytes + (size_t)(warp_slot0 + v * 32 + lane) * 16);
                    Arrays::unpack(raw, e[v]);
                }
            } else {
#pragma unroll
                for (int v = 0; v < VECS; ++v)
#pragma unroll
                    for (int k = 0; k < EPV; ++k) {
                        const u64 off = (u64)(warp_slot0 + v * 32 + lane) * EPV + k;
                        e[v][k] = off < count ? acc.load_elem(start + off) : Op::template identity<T>();
                    }
            }
            // ---- R(s + K) ------------------------------------------------------------------------------
            if (more) {
                const int rr = reduce_step(s + K);
                more = rr == 0;
                if (rr == 2) break;
            }
            // ---- S(s), second half -----------------------------------------------------------------------
            if (args.f != KF_MAP_IDENTITY) {
#pragma unroll
                for (int v = 0; v < VECS; ++v)
#pragma unroll
                    for (int k = 0; k < EPV; ++k) {
                        const u64 off = (u64)(warp_slot0 + v * 32 + lane) * EPV + k;
                        e[v][k] = off < count ? map_elem<T>(args.f, e[v][k]) : Op::template identity<T>();
                    }
            }
            T slot_excl[VECS];
            (void)warp_tile_scan<T, Op, VECS, EPV>(e, slot_excl, lane);
            if (!mbar_wait_or_abort_warp(&s_base[q], (s / NSTEP) & 1, s_abort)) {
                if (lane == 0) wait_failed(0xFFFFFFFAu);
                break;
            }
            const T base = Op::template apply<T>(slot_ref(&s_tile_excl[q]), slot_ref(&s_warp_excl[q * WARPS + warp]));
            // (the post-map g is a uniform switch around the whole store loop: g = identity carries no
            // per-element branch)
            auto emit = [&](auto with_g) {
                constexpr bool WITH_G = decltype(with_g)::value;
#pragma unroll
                for (int v = 0; v < VECS; ++v) {
                    const T p = Op::template apply<T>(base, slot_excl[v]);
#pragma unroll
                    for (int k = 0; k < EPV; ++k) {
                        e[v][k] = Op::template apply<T>(p, e[v][k]);
                        if constexpr (WITH_G) e[v][k] = post_elem<T>(args.g, e[v][k]);
                    }
                    if (fast) {
                        uint4 raw[NARR];
                        Arrays::pack(e[v], raw);
#pragma unroll
                        for (int a = 0; a < NARR; ++a)
                            st_stream_v4(arr.dst[a] + start * Arrays::elem_bytes + (size_t)(warp_slot0 + v * 32 + lane) * 16, raw[a]);
                    } else {
#pragma unroll
                        for (int k = 0; k < EPV; ++k) {
                            const u64 off = (u64)(warp_slot0 + v * 32 + lane) * EPV + k;
                            if (off < count) acc.store_elem(start + off, e[v][k]);
                        }
                    }
                }
            };
            if (args.g == KF_POST_IDENTITY) emit(std::false_type{});
            else emit(std::true_type{});
        }
    }

    // ---- leave: no bulk load of this CTA may still be in flight ----------------------------------------
    __syncthreads();
    if (tid == 0 && *reinterpret_cast<volatile int *>(s_abort)) {
        // Wait (bounded) for every load the loader started and poison the tiles this CTA holds so that
        // nobody waits for them.
        const u32 issued = *reinterpret_cast<volatile u32 *>(s_issued);
        const u32 lo_load = issued > (u32)NBUF ? issued - NBUF : 0;
        for (u32 j = lo_load; j < issued; ++j) (void)mbar_wait(&s_full[j % NBUF], (j / NBUF) & 1);
        const u32 lo = issued > (u32)NSTEP ? issued - NSTEP : 0;
        for (u32 j = lo; j < issued; ++j) {
            const u64 t = s_ticket[j % NSTEP];
            if (t < args.ntiles) Desc<T>::publish(args.desc, t, kPoison, Op::template identity<T>());
        }
    }
}

}  // namespace kf
