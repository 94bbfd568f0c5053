// Persistent, warp-specialised variant of the look-back scan for sm_100a. Tiles are staged into a
// shared-memory ring by the bulk-copy engine (TMA, cp.async.bulk) so that HBM reads stay in flight
// whatever the compute warps are doing; a tile crosses shared memory exactly once and every global
// round trip of the look-back protocol is taken off the critical path. One CTA-wide barrier per tile.
//
// The grid fills the GPU once (CTAs per SM x SM count); each CTA pulls tile tickets until they run
// out. A CTA is THREADS consumer threads plus one producer warp:
//
//   producer (one lane)  for each ring slot in turn: wait until the consumers have released it
//       (mbarrier `empty`), bind the ticket requested one step earlier to it (the atomic's latency
//       is hidden), start the tile's bulk load (completion on mbarrier `full`), request the next
//       ticket. Runs up to NBUF tiles ahead of the consumers.
//
//   consumers, iteration k (tile t_k; AHEAD >= 1 tiles are scanned ahead of the one being finished
//   and wait in a register ring, so the loop is unrolled AHEAD+1 times):
//     A  wait for `full` of tile t_k+AHEAD, read its slots from shared memory into registers
//        (striped, conflict-free 128-bit loads), release the ring buffer, scan in registers; each
//        warp leaves its total in shared memory.
//     B1 each warp summarises its window of t_k's predecessor descriptors from a SNAPSHOT it read one
//        iteration ago (a descriptor read takes 1-2 us under full streaming load).
//     -- the one barrier --
//     A' tile aggregate and warp prefixes of t_k+AHEAD; thread 0 publishes the AGGREGATE. Because
//        every CTA publishes aggregates AHEAD tiles before it resolves them, predecessors have
//        normally published when a tile looks back, and no look-back waits on another look-back.
//     B2 every warp folds the summaries into t_k's exclusive prefix (block-wide look-back: WARPS
//        windows of 32 tiles at once); thread 0 publishes t_k's inclusive PREFIX. If a predecessor
//        had not published when the snapshot was taken, the CTA polls the live descriptors.
//     C  add the prefix to t_k's registers and write the result to global memory with coalesced
//        128-bit streaming stores; then read the snapshot for t_k+1.
//
// Only whole tiles whose arrays sit on a 16-byte boundary take the bulk path; the short head tile
// of a misaligned view and the ragged last tile use element-wise global accesses inside the same
// loop. Every wait (mbarrier, look-back) is bounded and reports KF_ERR_TIMEOUT.
#pragma once

#include "scan_impl.cuh"

namespace kf {

__device__ __forceinline__ u32 smem_addr(const void *p) { return (u32)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(u64 *bar, u32 count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(u64 *bar, u32 bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(u64 *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(u64 *bar, u32 parity) {
    u32 ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(smem_addr(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
// Bounded wait; false when it ran out.
__device__ __forceinline__ bool mbar_wait(u64 *bar, u32 parity) {
    for (u32 spins = 0; spins < kSpinLimit; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if (spins > 64) __nanosleep(64);
    }
    return false;
}
// global -> shared bulk copy, completion (bytes) signalled on the mbarrier.
__device__ __forceinline__ void bulk_load(void *dst_smem, const void *src_gmem, u32 bytes, u64 *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}
// shared -> global bulk copy, tracked by the thread's bulk async-group.
__device__ __forceinline__ void bulk_store(void *dst_gmem, const void *src_smem, u32 bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem), "r"(smem_addr(src_smem)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Array views for the bulk path: NARR arrays, each contributing one 16-byte vector per slot.
template <typename T> struct PlainArrays {
    static constexpr int NARR = 1;
    static constexpr int EPV = 16 / sizeof(T);
    const char *src[1];
    char *dst[1];
    static constexpr int elem_bytes = sizeof(T);  // bytes per element in each array
    __device__ __forceinline__ static void unpack(const uint4 (&raw)[1], T (&e)[EPV]) { memcpy(e, &raw[0], 16); }
    __device__ __forceinline__ static void pack(const T (&e)[EPV], uint4 (&raw)[1]) { memcpy(&raw[0], e, 16); }
};
struct AffineSoaArrays {
    static constexpr int NARR = 2;
    static constexpr int EPV = 4;
    const char *src[2];
    char *dst[2];
    static constexpr int elem_bytes = 4;
    __device__ __forceinline__ static void unpack(const uint4 (&raw)[2], Affine (&e)[4]) {
        float a[4], b[4];
        memcpy(a, &raw[0], 16);
        memcpy(b, &raw[1], 16);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            e[k].a = a[k];
            e[k].b = b[k];
        }
    }
    __device__ __forceinline__ static void pack(const Affine (&e)[4], uint4 (&raw)[2]) {
        float a[4], b[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            a[k] = e[k].a;
            b[k] = e[k].b;
        }
        memcpy(&raw[0], a, 16);
        memcpy(&raw[1], b, 16);
    }
};

template <typename Arrays, typename T, int THREADS, int VECS, int NBUF, int AHEAD> struct ScanRingSmem {
    static constexpr int WARPS = THREADS / 32;
    static constexpr int ARR_BYTES = THREADS * VECS * 16;
    static constexpr int BUF_BYTES = Arrays::NARR * ARR_BYTES;
    static constexpr size_t kData = (size_t)NBUF * BUF_BYTES;
    static constexpr size_t kScratch = (size_t)WARPS * VECS * 32 * 8;  // per-warp scan scratch (8 bytes per slot total)
    // 8-byte words behind data and scratch: full / empty mbarriers, tickets, tile totals [NBUF each];
    // warp totals [2][WARPS]; warp prefixes [AHEAD+1][WARPS]; look-back values [2][WARPS]; then 4-byte
    // words: look-back info [2][WARPS], abort flag, tiles issued.
    static constexpr size_t kWords = 4 * NBUF + (5 + AHEAD) * WARPS;
    static constexpr size_t kBytes = kData + kScratch + 8 * kWords + 4 * (2 * WARPS + 2) + 16;
};

template <typename T, typename Op, typename Access, typename Arrays, int THREADS, int VECS, int NBUF, int AHEAD, bool IN_REGS>
__global__ void __launch_bounds__(THREADS + 32) scan_kernel_ring(Access acc, Arrays arr, ScanArgs args) {
    using SM = ScanRingSmem<Arrays, T, THREADS, VECS, NBUF, AHEAD>;
    constexpr int EPV = Arrays::EPV;
    constexpr int NARR = Arrays::NARR;
    constexpr int WARPS = THREADS / 32;
    constexpr int RING = AHEAD + 1;  // tiles scanned ahead or being finished (held in registers if IN_REGS)
    constexpr int RREGS = IN_REGS ? RING : 1;
    static_assert(IN_REGS || NBUF >= AHEAD + 2, "tiles that wait in the ring need a buffer each");
    constexpr u64 TILE = (u64)THREADS * VECS * EPV;
    constexpr int W8 = 8 / sizeof(T);  // index stride that keeps 8-byte spacing for small T
    static_assert(NBUF >= 2 && AHEAD >= 1, "ring too small");
    static_assert(sizeof(T) <= 8, "totals are staged as 8-byte words");

    extern __shared__ __align__(128) unsigned char smem[];
    T *s_scratch = reinterpret_cast<T *>(smem + SM::kData);
    u64 *words = reinterpret_cast<u64 *>(smem + SM::kData + SM::kScratch);
    u64 *s_full = words;                                                       // [NBUF]
    u64 *s_empty = words + NBUF;                                               // [NBUF]
    u64 *s_ticket = words + 2 * NBUF;                                          // [NBUF] tile ids
    T *s_total = reinterpret_cast<T *>(words + 3 * NBUF);                      // [NBUF] tile aggregates
    T *s_warp_total = reinterpret_cast<T *>(words + 4 * NBUF);                 // [2][WARPS]
    T *s_warp_excl = reinterpret_cast<T *>(words + 4 * NBUF + 2 * WARPS);      // [AHEAD+1][WARPS]
    T *s_lb_val = reinterpret_cast<T *>(words + 4 * NBUF + (3 + AHEAD) * WARPS);  // [2][WARPS]
    u32 *s_lb_info = reinterpret_cast<u32 *>(words + SM::kWords);             // [2][WARPS]
    int *s_abort = reinterpret_cast<int *>(s_lb_info + 2 * WARPS);
    u32 *s_issued = reinterpret_cast<u32 *>(s_abort + 1);                      // ring steps the producer has armed

    const u32 tid = threadIdx.x, lane = lane_id(), warp = tid >> 5;
    const u64 first = args.head > 0 ? 1 : 0;

    auto tile_start = [&](u64 tile) -> u64 { return tile < first ? 0 : args.head + (tile - first) * TILE; };
    auto tile_count = [&](u64 tile) -> u64 {
        if (tile < first) return args.head;
        const u64 s = args.head + (tile - first) * TILE;
        return args.n - s < TILE ? args.n - s : TILE;
    };

#ifdef KF_SCAN_TRACE
    if (tid == 0 && blockIdx.x == 0) {
        args.trace[args.ntiles * 16 + 0] = (u64)clock64();
        args.trace[args.ntiles * 16 + 1] = kf_now();
    }
#endif
    if (tid == 0) {
        for (int b = 0; b < NBUF; ++b) {
            mbar_init(&s_full[b], 1);
            mbar_init(&s_empty[b], WARPS);
        }
        *s_abort = ld_relaxed_u32(&args.header[kStatusWord]) != 0u;
        *s_issued = 0;
        fence_async_proxy();  // barrier init visible to the bulk-copy engine
    }
    __syncthreads();

    bool wait_failed = false;
    if (warp == WARPS) {
        // ======================= producer =======================================================
        if (lane == 0) {
            u32 pending = atomicAdd(&args.header[kTicketBase], 1u);
            for (u32 j = 0;; ++j) {
                const u32 b = j % NBUF;
                if (j >= (u32)NBUF) {
                    bool freed = false, aborted = false;
                    for (u32 spins = 0; spins < kSpinLimit && !freed && !aborted; ++spins) {
                        freed = mbar_try_wait(&s_empty[b], ((j / NBUF) - 1) & 1);
                        if (!freed && (spins & 63) == 63) {
                            aborted = *reinterpret_cast<volatile int *>(s_abort) != 0;
                            __nanosleep(64);
                        }
                    }
                    if (aborted) break;
                    if (!freed) {
                        wait_failed = true;
                        break;
                    }
                }
                if (*reinterpret_cast<volatile int *>(s_abort)) break;
                const u64 t = pending;
                s_ticket[b] = t;
                *reinterpret_cast<volatile u32 *>(s_issued) = j + 1;
                if (t >= args.ntiles) {
                    mbar_arrive(&s_full[b]);  // the end marker travels through the ring like a tile
                    break;
                }
                pending = atomicAdd(&args.header[kTicketBase], 1u);  // used one step from now
                if (tile_count(t) == TILE) {
                    const u64 off = tile_start(t) * Arrays::elem_bytes;
                    unsigned char *buf = smem + (size_t)b * SM::BUF_BYTES;
                    mbar_expect_tx(&s_full[b], (u32)SM::BUF_BYTES);
#pragma unroll
                    for (int a = 0; a < NARR; ++a)
                        bulk_load(buf + a * SM::ARR_BYTES, arr.src[a] + off, (u32)SM::ARR_BYTES, &s_full[b]);
                } else {
                    mbar_arrive(&s_full[b]);  // element-wise tile: nothing to load
                }
            }
            if (wait_failed) {
                record_error(args.header, KF_ERR_TIMEOUT, 0xFFFFFFFEu);
                *reinterpret_cast<volatile int *>(s_abort) = 1;
            }
        }
    } else {
        // ======================= consumers ======================================================
        const u32 warp_slot0 = warp * 32 * VECS;
        T *my_scratch = s_scratch + (size_t)warp * VECS * 32;
        T regs[RREGS][VECS][EPV];  // IN_REGS: tiles scanned ahead, inclusive within the warp
        const u32 rot = blocked_rot<VECS>(lane);
        u64 tiles[RING];          // their tile ids (>= ntiles: none)
#pragma unroll
        for (int r = 0; r < RING; ++r) tiles[r] = ~0ull;

        // Phase A, part 1, for the CTA's j-th tile: ring buffer -> registers, release the buffer,
        // scan, leave the warp total in s_warp_total[j & 1]. 0 = done, 1 = end of tiles, 2 = wait ran out.
        auto phase_a = [&](u32 j, T (&e)[VECS][EPV], u64 &tile_out) -> int {
            const u32 b = j % NBUF;
            if (!mbar_wait(&s_full[b], (j / NBUF) & 1)) {
                *reinterpret_cast<volatile int *>(s_abort) = 2;  // seen by every thread after the next barrier
                return 2;
            }
            const u64 tile = s_ticket[b];
            tile_out = tile;
            if (tile >= args.ntiles) return 1;
            const u64 start = tile_start(tile), count = tile_count(tile);
            unsigned char *buf = smem + (size_t)b * SM::BUF_BYTES;
            // IN_REGS: striped slots (v*32 + lane), kept in registers until phase C.
            // else   : blocked slots (lane*VECS + m) touched in rotated order, written back to the buffer.
            auto slot_of = [&](int v) -> u32 {
                return IN_REGS ? warp_slot0 + v * 32 + lane : warp_slot0 + lane * VECS + ((v + rot) & (VECS - 1));
            };
            if (count == TILE) {
#pragma unroll
                for (int v = 0; v < VECS; ++v) {
                    uint4 raw[NARR];
                    const u32 slot = slot_of(v);
#pragma unroll
                    for (int a = 0; a < NARR; ++a) raw[a] = *reinterpret_cast<const uint4 *>(buf + a * SM::ARR_BYTES + slot * 16);
                    Arrays::unpack(raw, e[v]);
                }
            } else {
#pragma unroll
                for (int v = 0; v < VECS; ++v)
#pragma unroll
                    for (int k = 0; k < EPV; ++k) {
                        const u64 off = (u64)slot_of(v) * EPV + k;
                        e[v][k] = off < count ? acc.load_elem(start + off) : Op::template identity<T>();
                    }
            }
            if constexpr (IN_REGS) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_empty[b]);  // this warp has its part of the buffer in registers
            }
            if (args.f != KF_MAP_IDENTITY) {
#pragma unroll
                for (int v = 0; v < VECS; ++v)
#pragma unroll
                    for (int k = 0; k < EPV; ++k) {
                        const u64 off = (u64)slot_of(v) * EPV + k;
                        e[v][k] = off < count ? map_elem<T>(args.f, e[v][k]) : Op::template identity<T>();
                    }
            }
            T carry;
            if constexpr (IN_REGS) {
                carry = warp_tile_scan_via_smem<T, Op, VECS, EPV>(e, my_scratch, lane);
            } else {
                carry = warp_tile_scan_blocked<T, Op, VECS, EPV>(e, rot, lane);
#pragma unroll
                for (int v = 0; v < VECS; ++v) {  // inclusive within the warp, back into the ring buffer
                    uint4 raw[NARR];
                    Arrays::pack(e[v], raw);
                    const u32 slot = slot_of(v);
#pragma unroll
                    for (int a = 0; a < NARR; ++a) *reinterpret_cast<uint4 *>(buf + a * SM::ARR_BYTES + slot * 16) = raw[a];
                }
            }
            if (lane == 0) s_warp_total[((j & 1) * WARPS + warp) * W8] = carry;
            return 0;
        };
        // Phase A, part 2 (after the barrier): this warp's prefix within the tile, the tile aggregate.
        // `tile` comes from the caller's registers: the producer may already have rebound the ring slot.
        auto phase_a_finish = [&](u32 j, u64 tile) {
            const T mine = lane < (u32)WARPS ? s_warp_total[((j & 1) * WARPS + lane) * W8] : Op::template identity<T>();
            // descending fold wants the earliest operand in the highest lane: mirror the lanes
            const T mirrored = shfl_idx(mine, 31 - (int)lane);
            const T tile_total = warp_fold_descending<T, Op>(mirrored, lane);
            const T before = (31 - lane) < warp ? mirrored : Op::template identity<T>();
            const T warp_excl = warp_fold_descending<T, Op>(before, lane);
            if (lane == 0) s_warp_excl[((j % RING) * WARPS + warp) * W8] = warp_excl;
            if (tid == 0) {
                s_total[(j % RING) * W8] = tile_total;
                if (tile > 0 && tile < args.ntiles) Desc<T>::publish(args.desc, tile, kAggregate, tile_total);
            }
        };

        // ---- prologue: scan the first AHEAD tiles ahead --------------------------------------------
        bool more = true;  // tiles left to scan ahead
#pragma unroll
        for (int j = 0; j < AHEAD; ++j) {
            if (more && !wait_failed) {
                const int r = phase_a((u32)j, regs[IN_REGS ? j : 0], tiles[j]);
                more = r == 0;
                cta_sync<THREADS>();
                wait_failed = *reinterpret_cast<volatile int *>(s_abort) == 2;
                if (r == 0 && !wait_failed) phase_a_finish((u32)j, tiles[j]);
            }
        }
        u32 st_next = kInvalid;  // snapshot of the descriptors before the CTA's next tile, one per lane
        T v_next = T();
        if (!wait_failed && tiles[0] < args.ntiles) st_next = lookback_read<T>(args, tiles[0], warp, lane, v_next);

        bool done = wait_failed;
        for (u32 it0 = 0; !done; it0 += RING) {
#pragma unroll
            for (int u = 0; u < RING; ++u) {
                if (done) break;
                const u32 it = it0 + u;
                constexpr int dummy = 0;
                (void)dummy;
                const int ua = (u + AHEAD) % RING;  // register slot of the tile scanned ahead now
                const u64 tile = tiles[u];
                if (tile >= args.ntiles) {
                    done = true;
                    break;
                }
#ifdef KF_SCAN_TRACE
                KF_TRACE(0, kf_now());
#endif
                int ra = 1;
                if (more) {
                    ra = phase_a(it + AHEAD, regs[IN_REGS ? ua : 0], tiles[ua]);
                    more = ra == 0;
                } else {
                    tiles[ua] = ~0ull;
                }
#ifdef KF_SCAN_TRACE
                KF_TRACE(1, kf_now());
#endif
                u32 *info = s_lb_info + (it & 1) * WARPS;
                T *val = s_lb_val + (it & 1) * WARPS * W8;
                lookback_summarise<T, Op>(tile, st_next, v_next, warp, lane, info, val);
                cta_sync<THREADS>();
#ifdef KF_SCAN_TRACE
                KF_TRACE(2, kf_now());
#endif
                {
                    const int ab = *reinterpret_cast<volatile int *>(s_abort);  // same answer in every thread: the barrier orders it
                    if (ab) {
                        wait_failed = ab == 2;
                        done = true;
                        break;
                    }
                }
                if (ra == 0) phase_a_finish(it + AHEAD, tiles[ua]);
                T excl = Op::template identity<T>();
                bool all_agg = false;
                int how = lookback_finish<T, Op, WARPS>(lane, info, val, excl, all_agg);
#ifdef KF_SCAN_TRACE
                if (args.block_order & 8) how = 1;  // lab knob: never poll (wrong results, timing only)
                KF_TRACE(6, (u64)how);
#endif
                const T my_total = s_total[(it % RING) * W8];  // read by thread 0 only where it matters
                if (how == 1) {
                    if (tile == 0 && args.init) excl = *reinterpret_cast<const T *>(args.init);
                    if (tid == 0) Desc<T>::publish(args.desc, tile, kPrefix, Op::template apply<T>(excl, my_total));
                } else if (how == 0) {
                    // a predecessor had not published when the snapshot was taken: poll the live descriptors
                    cta_sync<THREADS>();  // everyone is done reading the summaries the poll will overwrite
                    if (!resolve_tile_prefix_block<T, Op, WARPS, false, THREADS>(args, tile, my_total, warp, lane, s_abort,
                                                                                 info, val, excl)) {
                        done = true;
                        break;
                    }
                } else {
                    if (tid == 0) {
                        Desc<T>::publish(args.desc, tile, kPoison, Op::template identity<T>());
                        *reinterpret_cast<volatile int *>(s_abort) = 1;
                    }
                    done = true;
                    break;
                }
#ifdef KF_SCAN_TRACE
                KF_TRACE(3, kf_now());
#endif
                // ---- phase C: add the prefix to the tile held in registers and write it out --------------
                const u64 start = tile_start(tile), count = tile_count(tile);
                const bool fast = count == TILE;
                const T base = Op::template apply<T>(excl, s_warp_excl[((it % RING) * WARPS + warp) * W8]);
                const u32 bc = it % NBUF;
#pragma unroll
                for (int v = 0; v < VECS; ++v) {
                    T e[EPV];
                    if constexpr (IN_REGS) {
#pragma unroll
                        for (int k = 0; k < EPV; ++k) e[k] = regs[u][v][k];
                    } else {  // striped read of the locally scanned tile: the stores below stay coalesced
                        uint4 raw[NARR];
                        const unsigned char *buf = smem + (size_t)bc * SM::BUF_BYTES;
#pragma unroll
                        for (int a = 0; a < NARR; ++a)
                            raw[a] = *reinterpret_cast<const uint4 *>(buf + a * SM::ARR_BYTES + (warp_slot0 + v * 32 + lane) * 16);
                        Arrays::unpack(raw, e);
                    }
#pragma unroll
                    for (int k = 0; k < EPV; ++k) e[k] = Op::template apply<T>(base, e[k]);
                    if (fast) {
                        uint4 raw[NARR];
                        Arrays::pack(e, raw);
#pragma unroll
                        for (int a = 0; a < NARR; ++a)
                            st_stream_v4(arr.dst[a] + start * Arrays::elem_bytes + (size_t)(warp_slot0 + v * 32 + lane) * 16, raw[a]);
                    } else {
#pragma unroll
                        for (int k = 0; k < EPV; ++k) {
                            const u64 off = (u64)(warp_slot0 + v * 32 + lane) * EPV + k;
                            if (off < count) acc.store_elem(start + off, e[k]);
                        }
                    }
                }
                if constexpr (!IN_REGS) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&s_empty[bc]);  // this warp is done with the buffer
                }
                // ---- snapshot of the next tile's predecessors, consumed one iteration from now -----------
                {
                    const u64 tile_next = tiles[(u + 1) % RING];
                    if (tile_next < args.ntiles) st_next = lookback_read<T>(args, tile_next, warp, lane, v_next);
                }
#ifdef KF_SCAN_TRACE
                KF_TRACE(7, kf_now());
#endif
            }
        }
        if (tid == 0) {
            if (wait_failed) record_error(args.header, KF_ERR_TIMEOUT, 0xFFFFFFFFu);
            if (*reinterpret_cast<volatile int *>(s_abort)) {
                // tiles scanned ahead but never resolved: nobody may wait for them
#pragma unroll
                for (int r = 0; r < RING; ++r)
                    if (tiles[r] < args.ntiles) Desc<T>::publish(args.desc, tiles[r], kPoison, Op::template identity<T>());
            }
        }
    }

    // ---- leave: no bulk load of this CTA may still be in flight ----------------------------------------
    __syncthreads();
#ifdef KF_SCAN_TRACE
    if (tid == 0 && blockIdx.x == 0) {
        args.trace[args.ntiles * 16 + 2] = (u64)clock64();
        args.trace[args.ntiles * 16 + 3] = kf_now();
    }
#endif
    if (tid == 0 && *reinterpret_cast<volatile int *>(s_abort)) {
        // Wait (bounded) for every load the producer started and poison the tiles this CTA holds so
        // that nobody waits for them.
        const u32 issued = *reinterpret_cast<volatile u32 *>(s_issued);
        const u32 lo = issued > (u32)NBUF ? issued - NBUF : 0;
        for (u32 j = lo; j < issued; ++j) {
            const u32 b = j % NBUF;
            (void)mbar_wait(&s_full[b], (j / NBUF) & 1);
            const u64 t = s_ticket[b];
            if (t < args.ntiles) Desc<T>::publish(args.desc, t, kPoison, Op::template identity<T>());
        }
    }
}

}  // namespace kf
