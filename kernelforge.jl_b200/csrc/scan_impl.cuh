// Single-pass inclusive scan with decoupled look-back for sm_100a.
//
// Layout of one tile (THREADS threads, VECS slots per thread, EPV elements per 16-byte slot):
// warp w owns the contiguous run of 32*VECS slots starting at slot w*32*VECS, and lane l holds
// slots j*32 + l (j = 0..VECS-1) of that run. Every load and store instruction of a warp
// therefore touches 512 contiguous bytes (fully coalesced 128-bit accesses) and the element
// order is (warp, j, lane, component) with no shared-memory transpose: a thread scans the
// components of each slot, the warp scans slot totals with shuffles (VECS independent scans),
// and a running carry chains the VECS rows. Operand order is preserved throughout, so
// non-commutative operators are allowed.
//
// Tiles are handed out by an atomic ticket, so a tile's predecessors are always already running.
// Each tile publishes its aggregate, looks back over its predecessors' descriptors with one warp
// (32 descriptors per poll), then publishes its inclusive prefix. A descriptor is one 64-bit word
// {status:32 | value:32} for elements up to 4 bytes, or one such word per 32 bits of a wider element
// (two for 8-byte elements, eight for a Float64 quaternion): each word validates itself and a reader
// retries until all carry the same status, so no fence separates value and flag. Every wait is
// bounded; a tile that gives up records KF_ERR_TIMEOUT in the workspace header and publishes a
// poison status that makes its successors return too.
//
// Semantics follow scan_kernel_packed! / scan_kernel! of KernelForge.jl
// (src/scan/scan_kernel.jl:310-478, 94-299): inclusive, f applied on load, left-to-right order.
#pragma once

#include "common.cuh"

#include <type_traits>

namespace kf {

enum : u32 { kInvalid = 0, kAggregate = 1, kPrefix = 2, kPoison = 3 };

// ---- descriptors ------------------------------------------------------------------------------
template <typename T> struct Desc {
    static constexpr int WORDS = sizeof(T) <= 4 ? 1 : (int)(sizeof(T) / 4);

    static __device__ __forceinline__ void publish(u64 *desc, u64 tile, u32 status, T v) {
        if constexpr (WORDS == 1) {
            u32 bits = 0;
            memcpy(&bits, &v, sizeof(T));
            st_relaxed_u64(desc + tile, ((u64)status << 32) | bits);
        } else {
            u32 h[WORDS];
            memcpy(h, &v, sizeof(T));
#pragma unroll
            for (int i = 0; i < WORDS; ++i) st_relaxed_u64(desc + WORDS * tile + i, ((u64)status << 32) | h[i]);
        }
    }
    // Returns the status (kInvalid when not yet published or when the words disagree).
    static __device__ __forceinline__ u32 read(const u64 *desc, u64 tile, T &v) {
        if constexpr (WORDS == 1) {
            const u64 w = ld_relaxed_u64(desc + tile);
            const u32 bits = (u32)w;
            memcpy(&v, &bits, sizeof(T));
            return (u32)(w >> 32);
        } else {
            u32 h[WORDS];
            u32 st = 0;
            bool same = true;
#pragma unroll
            for (int i = 0; i < WORDS; ++i) {
                const u64 w = ld_relaxed_u64(desc + WORDS * tile + i);
                h[i] = (u32)w;
                const u32 si = (u32)(w >> 32);
                if (i == 0) st = si;
                else same = same && si == st;
            }
            memcpy(&v, h, sizeof(T));
            return same ? st : (u32)kInvalid;
        }
    }
};

// ---- slot access policies ---------------------------------------------------------------------
// Plain array of T (also the interleaved (a, b) pair form of the affine scan).
template <typename T> struct PlainAccess {
    static constexpr int EPV = 16 / sizeof(T);
    const T *src;
    T *dst;
    __device__ __forceinline__ void load_slot(u64 slot_elem0, T (&e)[EPV]) const {
        uint4 v = ld_v4(src + slot_elem0);
        memcpy(e, &v, 16);
    }
    __device__ __forceinline__ void store_slot(u64 slot_elem0, const T (&e)[EPV]) const {
        uint4 v;
        memcpy(&v, e, 16);
        st_stream_v4(dst + slot_elem0, v);
    }
    __device__ __forceinline__ T load_elem(u64 i) const { return src[i]; }
    __device__ __forceinline__ void store_elem(u64 i, T v) const { dst[i] = v; }
};

// Affine pairs stored as two Float32 arrays. A slot is 4 pairs: one 16-byte vector of each array.
struct AffineSoaAccess {
    static constexpr int EPV = 4;
    const float *a_src, *b_src;
    float *a_dst, *b_dst;
    __device__ __forceinline__ void load_slot(u64 i0, Affine (&e)[EPV]) const {
        uint4 va = ld_v4(a_src + i0), vb = ld_v4(b_src + i0);
        float a[4], b[4];
        memcpy(a, &va, 16);
        memcpy(b, &vb, 16);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            e[k].a = a[k];
            e[k].b = b[k];
        }
    }
    __device__ __forceinline__ void store_slot(u64 i0, const Affine (&e)[EPV]) const {
        float a[4], b[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            a[k] = e[k].a;
            b[k] = e[k].b;
        }
        uint4 va, vb;
        memcpy(&va, a, 16);
        memcpy(&vb, b, 16);
        st_stream_v4(a_dst + i0, va);
        st_stream_v4(b_dst + i0, vb);
    }
    __device__ __forceinline__ Affine load_elem(u64 i) const {
        Affine x;
        x.a = a_src[i];
        x.b = b_src[i];
        return x;
    }
    __device__ __forceinline__ void store_elem(u64 i, Affine v) const {
        a_dst[i] = v.a;
        b_dst[i] = v.b;
    }
};

// Quaternions as an array of structs. Float32 components: a slot is FOUR consecutive quaternions of one
// lane (64 bytes), which the lane scans serially, so that only the slot totals go through the warp scan
// (measured at n = 2^24: 0.375 ms against 0.457 ms with one quaternion per slot); a lane's vectors are
// 64 bytes apart from its neighbour's, so these loads go through L1. Float64 components: one quaternion
// (two 16-byte vectors) per slot, streaming accesses (0.865 ms against 0.944 ms with four per slot).
template <typename F> struct QuatAccess {
    static constexpr int EPV = sizeof(F) == 4 ? 4 : 1;
    using Q = Quat<F>;
    static constexpr int NV = (int)(EPV * sizeof(Q) / 16);  // 16-byte vectors per slot
    const Q *src;
    Q *dst;
    __device__ __forceinline__ void load_slot(u64 i0, Q (&e)[EPV]) const {
        uint4 v[NV];
        const uint4 *p = reinterpret_cast<const uint4 *>(src + i0);
#pragma unroll
        for (int k = 0; k < NV; ++k) v[k] = EPV == 1 ? ld_v4(p + k) : p[k];
        memcpy(&e[0], v, sizeof(v));
    }
    __device__ __forceinline__ void store_slot(u64 i0, const Q (&e)[EPV]) const {
        uint4 v[NV];
        memcpy(v, &e[0], sizeof(v));
        uint4 *p = reinterpret_cast<uint4 *>(dst + i0);
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            if (EPV == 1) st_stream_v4(p + k, v[k]);
            else p[k] = v[k];
        }
    }
    __device__ __forceinline__ Q load_elem(u64 i) const {
        const F *p = reinterpret_cast<const F *>(src + i);
        Q q;
        q.w = p[0];
        q.x = p[1];
        q.y = p[2];
        q.z = p[3];
        return q;
    }
    __device__ __forceinline__ void store_elem(u64 i, Q q) const {
        F *p = reinterpret_cast<F *>(dst + i);
        p[0] = q.w;
        p[1] = q.x;
        p[2] = q.y;
        p[3] = q.z;
    }
};

template <typename T> __device__ __forceinline__ T map_elem(int f, T x) { return apply_map<T>(f, x); }
template <> __device__ __forceinline__ Affine map_elem<Affine>(int, Affine x) { return x; }
template <> __device__ __forceinline__ Quat<float> map_elem<Quat<float>>(int, Quat<float> x) { return x; }
template <> __device__ __forceinline__ Quat<double> map_elem<Quat<double>>(int, Quat<double> x) { return x; }

struct ScanArgs {
    u64 n;          // elements
    u64 head;       // elements before the first 16-byte boundary (tile 0 when > 0)
    u64 ntiles;
    u64 *desc;      // Desc<T>::WORDS words per tile
    u32 *header;    // workspace header (status, ticket)
    const void *init;  // optional left seed: `ninit` elements, folded left to right, or nullptr
    int vec_ok;     // all arrays share their 16-byte misalignment: full tiles use 128-bit accesses
    int f;
    int g;          // kf_post applied to every output element (the carried prefix stays unmapped)
    u32 ninit;
    u32 spin_limit; // polls before a look-back gives up
    u32 mute_tile;  // test hook: 1 + index of a tile that publishes nothing (0 = none)
};

template <typename T> __device__ __forceinline__ T post_elem(int g, T x) { return apply_post<T>(g, x); }
template <> __device__ __forceinline__ Affine post_elem<Affine>(int, Affine x) { return x; }
template <> __device__ __forceinline__ Quat<float> post_elem<Quat<float>>(int, Quat<float> x) { return x; }
template <> __device__ __forceinline__ Quat<double> post_elem<Quat<double>>(int, Quat<double> x) { return x; }

// The seed of the scan: init[0] op init[1] op ... (identity when there is none). A sharded scan passes
// the totals of all shards and `ninit` = its rank, so the carry needs no kernel of its own.
template <typename T, typename Op> __device__ __forceinline__ T fold_init(const ScanArgs &args) {
    T acc = Op::template identity<T>();
    if (args.init) {
        const T *p = reinterpret_cast<const T *>(args.init);
        for (u32 i = 0; i < args.ninit; ++i) acc = i == 0 ? p[0] : Op::template apply<T>(acc, p[i]);
    }
    return acc;
}


// Sixteen packed bytes: their sum (the low 8 bits are the wrap-around sum), and their inclusive
// wrap-around prefix sums on top of a carried-in byte `b`. A word {b0,b1,b2,b3} is split into its even
// and odd bytes as two 16-bit lanes each; lane sums stay below 2^16, so nothing carries between lanes:
//   lo = {b0, b2}, hi = {b1, b3};  lo * 0x00010001 = {b0, b0+b2};
//   even prefixes {p0, p2} = {b0, b0+b2} + {0, b1} + b;  odd prefixes {p1, p3} = {b0, b0+b2} + {b1, b1+b3} + b.
__device__ __forceinline__ u32 byte_sum16(uint4 r) {
    u32 s = __dp4a(r.x, 0x01010101u, 0u);
    s = __dp4a(r.y, 0x01010101u, s);
    s = __dp4a(r.z, 0x01010101u, s);
    return __dp4a(r.w, 0x01010101u, s);
}
__device__ __forceinline__ uint4 byte_prefix16(uint4 r, u32 b) {
    u32 carry = b | (b << 16);  // the carried-in byte in both lanes
    u32 w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const u32 lo = __byte_perm(w[i], 0u, 0x4240u);  // {b0, 0, b2, 0}
        const u32 hi = __byte_perm(w[i], 0u, 0x4341u);  // {b1, 0, b3, 0}
        const u32 s_lo = lo * 0x00010001u + carry;
        const u32 even = (hi << 16) + s_lo;
        const u32 odd = hi * 0x00010001u + s_lo;
        w[i] = __byte_perm(even, odd, 0x6240u);          // {p0, p1, p2, p3}, low bytes of the lanes
        carry = __byte_perm(odd, 0u, 0x4242u);           // p3 in both lanes
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// Scans the VECS x EPV elements a thread holds (in place, inclusive within each slot) and the slot
// totals across the warp. On return e[j][k] is inclusive within its slot, slot_excl[j] is the
// combination of everything the warp holds before slot j of this lane, and the return value is
// the warp total (valid in every lane).
template <typename T, typename Op, int VECS, int EPV>
__device__ __forceinline__ T warp_tile_scan(T (&e)[VECS][EPV], T (&slot_excl)[VECS], u32 lane) {
    T incl[VECS];
#pragma unroll
    for (int j = 0; j < VECS; ++j) {
#pragma unroll
        for (int k = 1; k < EPV; ++k) e[j][k] = Op::template apply<T>(e[j][k - 1], e[j][k]);
        incl[j] = e[j][EPV - 1];
    }
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
#pragma unroll
        for (int j = 0; j < VECS; ++j) {  // VECS independent shuffles per step, no branches
            T up = shfl_up(incl[j], d);
            up = lane >= (u32)d ? up : Op::template identity<T>();
            incl[j] = Op::template apply<T>(up, incl[j]);
        }
    }
    // Exclusive prefix of each slot within the warp: carry over rows j, then lanes before mine.
    T carry = Op::template identity<T>();
#pragma unroll
    for (int j = 0; j < VECS; ++j) {
        T prev = shfl_up(incl[j], 1);
        prev = lane == 0 ? Op::template identity<T>() : prev;
        slot_excl[j] = Op::template apply<T>(carry, prev);
        carry = Op::template apply<T>(carry, shfl_idx(incl[j], 31));
    }
    return carry;
}

// CTA-wide barrier, or a named barrier over the first BAR_THREADS threads when part of the CTA
// (a producer warp) must not take part.
template <int BAR_THREADS> __device__ __forceinline__ void cta_sync() {
    if constexpr (BAR_THREADS == 0) __syncthreads();
    else asm volatile("bar.sync 1, %0;" ::"n"(BAR_THREADS) : "memory");
}

// What one warp's window of 32 predecessor descriptors looks like, for the block-wide look-back.
enum : u32 { kLbAllAgg = 0, kLbHasPrefix = 1, kLbNotReady = 2, kLbPoison = 3 };

// Combination of the values of lanes 0..31 in DESCENDING lane order (lane 31 is the leftmost
// operand), valid in every lane. Look-back windows are laid out with the nearest predecessor in
// lane 0, so descending lane order is array order. Commutative operators use a butterfly (or one
// redux.sync for 32-bit integer add/min/max/and/or/xor); the others keep the ordered tree.
template <typename T, typename Op> __device__ __forceinline__ T warp_fold_descending(T x, u32 lane) {
    if constexpr (Op::commutative) {
        if constexpr (sizeof(T) == 4 && !IsFloat<T>::value && !std::is_same<Op, OpMul>::value) {
            if constexpr (std::is_same<Op, OpAdd>::value) return (T)__reduce_add_sync(0xFFFFFFFFu, (unsigned)x);
            else if constexpr (std::is_same<Op, OpAnd>::value) return (T)__reduce_and_sync(0xFFFFFFFFu, (unsigned)x);
            else if constexpr (std::is_same<Op, OpOr>::value) return (T)__reduce_or_sync(0xFFFFFFFFu, (unsigned)x);
            else if constexpr (std::is_same<Op, OpXor>::value) return (T)__reduce_xor_sync(0xFFFFFFFFu, (unsigned)x);
            else if constexpr (std::is_same<Op, OpMin>::value) return (T)__reduce_min_sync(0xFFFFFFFFu, x);
            else return (T)__reduce_max_sync(0xFFFFFFFFu, x);
        } else {
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) x = Op::template apply<T>(x, shfl_xor(x, d));
            return x;
        }
    } else {
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            T y = shfl_down(x, d);
            y = lane + d < 32 ? y : Op::template identity<T>();
            x = Op::template apply<T>(y, x);
        }
        return shfl_idx(x, 0);
    }
}

// Block-wide look-back, first half: every warp summarises its window of 32 predecessor descriptors
// (one per lane, read earlier: warp w covers tiles tile-1-32w .. tile-32-32w) into s_info[warp] /
// s_val[warp]. A barrier must separate it from the second half.
template <typename T, typename Op>
__device__ __forceinline__ void lookback_summarise(u64 tile, u32 st, T v, u32 warp, u32 lane, u32 *s_info, T *s_val) {
    const long long mine = (long long)tile - 1 - (long long)(warp * 32 + lane);
    if (mine < 0) st = kPrefix;  // positions before tile 0 read as "prefix = identity"
    const u32 poison = __ballot_sync(0xFFFFFFFFu, st == kPoison);
    const u32 pfx = __ballot_sync(0xFFFFFFFFu, st == kPrefix);
    const u32 inv = __ballot_sync(0xFFFFFFFFu, st == kInvalid);
    const int last = pfx ? (__ffs(pfx) - 1) : 31;  // nearest tile of the window with an inclusive prefix
    const u32 need = last == 31 ? 0xFFFFFFFFu : ((2u << last) - 1u);
    const T x = ((int)lane <= last && mine >= 0) ? v : Op::template identity<T>();
    const T folded = warp_fold_descending<T, Op>(x, lane);
    if (lane == 0) {
        s_info[warp] = poison ? kLbPoison : ((inv & need) ? kLbNotReady : (pfx ? kLbHasPrefix : kLbAllAgg));
        s_val[warp] = folded;
    }
}
// Second half, run by every warp on the same summaries: 1 = resolved (`excl`, valid in every thread,
// combines everything back to and including the nearest prefix); 0 = the caller has to poll
// (someone was not ready, or no prefix within 32*WARPS tiles; for the latter `excl` holds the
// aggregates of the whole block window); 2 = a predecessor was poisoned.
template <typename T, typename Op, int WARPS>
__device__ __forceinline__ int lookback_finish(u32 lane, const u32 *s_info, const T *s_val, T &excl, bool &all_aggregates) {
    static_assert(WARPS <= 32, "one lane per warp in the final fold");
    const u32 info = lane < (u32)WARPS ? s_info[lane] : (u32)kLbAllAgg;
    const T val = lane < (u32)WARPS ? s_val[lane] : Op::template identity<T>();
    const u32 not_agg = __ballot_sync(0xFFFFFFFFu, info != kLbAllAgg);
    all_aggregates = not_agg == 0;
    const int stop = all_aggregates ? 31 : __ffs(not_agg) - 1;
    const u32 why = all_aggregates ? (u32)kLbAllAgg : __shfl_sync(0xFFFFFFFFu, info, stop);
    if (why == kLbPoison) return 2;
    if (why == kLbNotReady) return 0;
    const T y = (int)lane <= stop ? val : Op::template identity<T>();
    excl = warp_fold_descending<T, Op>(y, lane);
    return all_aggregates ? 0 : 1;
}

// Block-wide look-back with polling: the CTA's WARPS warps read WARPS consecutive windows of 32
// predecessor descriptors in the same round trip, so a tile whose nearest inclusive prefix is
// hundreds of tiles back still resolves in one poll instead of walking 32 tiles per round trip.
// Called by every thread that takes part in barrier BAR_THREADS (it synchronises). On success the
// exclusive prefix is returned in every thread and thread 0 has published the tile's inclusive
// prefix; on failure (bounded wait ran out, or a poisoned predecessor) thread 0 has published
// poison, recorded the error and raised *s_abort, and the function returns false after a barrier.
// `s_info` / `s_val` hold one entry per warp. PUBLISH_AGG = false when the caller has already
// published the tile's aggregate.
template <typename T> __device__ __forceinline__ u32 lookback_read(const ScanArgs &args, u64 base_tile, u32 warp, u32 lane, T &v) {
    const long long mine = (long long)base_tile - 1 - (long long)(warp * 32 + lane);
    v = T();
    return mine >= 0 ? Desc<T>::read(args.desc, (u64)mine, v) : (u32)kPrefix;
}

template <typename T, typename Op, int WARPS, bool PUBLISH_AGG, int BAR_THREADS>
__device__ __forceinline__ bool resolve_tile_prefix_block(const ScanArgs &args, u64 tile, T tile_total, u32 warp, u32 lane,
                                                          int *s_abort, u32 *s_info, T *s_val, T &excl_out) {
    const u32 tid = threadIdx.x;
    if (tile == 0) {
        const T excl = fold_init<T, Op>(args);
        if (tid == 0) Desc<T>::publish(args.desc, tile, kPrefix, Op::template apply<T>(excl, tile_total));
        excl_out = excl;
        return true;
    }
    if (PUBLISH_AGG && tid == 0) Desc<T>::publish(args.desc, tile, kAggregate, tile_total);
    T acc = Op::template identity<T>();
    u64 base = tile;  // the window covers tiles base-1 .. base-32*WARPS
    u32 spins = 0;
    int how;
    bool timed_out = false;
    while (true) {
        T v;
        const u32 st = lookback_read<T>(args, base, warp, lane, v);
        lookback_summarise<T, Op>(base, st, v, warp, lane, s_info, s_val);
        cta_sync<BAR_THREADS>();
        T part = Op::template identity<T>();
        bool all_agg = false;
        how = lookback_finish<T, Op, WARPS>(lane, s_info, s_val, part, all_agg);
        cta_sync<BAR_THREADS>();  // summaries may be overwritten from here on
        if (how == 1 || all_agg) acc = Op::template apply<T>(part, acc);
        if (how != 0) break;
        if (all_agg) {
            base -= 32 * WARPS;  // nothing but aggregates in sight: keep walking back
            spins = 0;
        } else {
            if (++spins > args.spin_limit) {
                timed_out = true;
                how = 2;
                break;
            }
            if (spins > 4) __nanosleep(spins > 64 ? 256 : 32);
        }
    }
    if (how == 1) {
        if (tid == 0) Desc<T>::publish(args.desc, tile, kPrefix, Op::template apply<T>(acc, tile_total));
        excl_out = acc;
        return true;
    }
    if (tid == 0) {
        if (timed_out) record_error(args.header, KF_ERR_TIMEOUT, (u32)tile);
        Desc<T>::publish(args.desc, tile, kPoison, Op::template identity<T>());
        *s_abort = 1;
    }
    cta_sync<BAR_THREADS>();
    return false;
}

template <typename T, typename Op, typename Access, int THREADS, int VECS>
__global__ void __launch_bounds__(THREADS) scan_kernel(Access acc, ScanArgs args) {
    constexpr int EPV = Access::EPV;
    constexpr int WARPS = THREADS / 32;
    constexpr u64 TILE = (u64)THREADS * VECS * EPV;

    __shared__ T s_warp_total[WARPS];
    __shared__ u64 s_tile;
    __shared__ int s_abort;
    __shared__ u32 s_lb_info[WARPS];
    __shared__ T s_lb_val[WARPS];

    const u32 tid = threadIdx.x, lane = lane_id(), warp = tid >> 5;

    if (tid == 0) {
        s_tile = (u64)atomicAdd(&args.header[kTicketBase], 1u);
        s_abort = ld_relaxed_u32(&args.header[kStatusWord]) != 0u;
    }
    __syncthreads();
    const u64 tile = s_tile;
    if (tile >= args.ntiles) return;
    if (s_abort) {  // an earlier tile failed: pass the poison on so nobody waits for this tile
        if (tid == 0) Desc<T>::publish(args.desc, tile, kPoison, Op::template identity<T>());
        return;
    }
    if (args.mute_tile && tile + 1 == (u64)args.mute_tile) return;  // test hook: a tile that never publishes

    // Tile extent. With a misaligned base, tile 0 is the short scalar head.
    const u64 first = args.head > 0 ? 1 : 0;
    u64 start, count;
    if (tile < first) {
        start = 0;
        count = args.head;
    } else {
        start = args.head + (tile - first) * TILE;
        count = args.n - start < TILE ? args.n - start : TILE;
    }
    const bool fast = args.vec_ok && count == TILE;
    const u64 warp_slot0 = (u64)warp * 32 * VECS;  // first slot of this warp, within the tile

    // ---- load + map -------------------------------------------------------------------------
    T e[VECS][EPV];
    if (fast) {
#pragma unroll
        for (int j = 0; j < VECS; ++j) acc.load_slot(start + (warp_slot0 + (u64)j * 32 + lane) * EPV, e[j]);
#pragma unroll
        for (int j = 0; j < VECS; ++j)
#pragma unroll
            for (int k = 0; k < EPV; ++k) e[j][k] = map_elem<T>(args.f, e[j][k]);
    } else {
#pragma unroll
        for (int j = 0; j < VECS; ++j)
#pragma unroll
            for (int k = 0; k < EPV; ++k) {
                const u64 off = (warp_slot0 + (u64)j * 32 + lane) * EPV + k;
                e[j][k] = off < count ? map_elem<T>(args.f, acc.load_elem(start + off)) : Op::template identity<T>();
            }
    }

    // ---- thread-local scan of each slot, warp scan of slot totals ----------------------------
    T slot_excl[VECS];
    const T carry = warp_tile_scan<T, Op, VECS, EPV>(e, slot_excl, lane);
    if (lane == 0) s_warp_total[warp] = carry;
    __syncthreads();

    // ---- warp prefix within the tile and the tile aggregate ----------------------------------
    T warp_excl = Op::template identity<T>();
    T tile_total = Op::template identity<T>();
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
        const T t = s_warp_total[w];
        warp_excl = Op::template apply<T>(warp_excl, w < (int)warp ? t : Op::template identity<T>());
        tile_total = Op::template apply<T>(tile_total, t);
    }

    // ---- publish, look back, publish ---------------------------------------------------------
    T tile_excl;
    if (!resolve_tile_prefix_block<T, Op, WARPS, true, 0>(args, tile, tile_total, warp, lane, &s_abort, s_lb_info, s_lb_val, tile_excl)) return;

    // ---- apply the prefix and store -----------------------------------------------------------
    // (the post-map g is a uniform switch around the whole store loop, so that the common g = identity
    // path carries no per-element branch)
    const T base = Op::template apply<T>(tile_excl, warp_excl);
    auto emit = [&](auto with_g) {
        constexpr bool WITH_G = decltype(with_g)::value;
        if (fast) {
#pragma unroll
            for (int j = 0; j < VECS; ++j) {
                const T p = Op::template apply<T>(base, slot_excl[j]);
#pragma unroll
                for (int k = 0; k < EPV; ++k) {
                    e[j][k] = Op::template apply<T>(p, e[j][k]);
                    if constexpr (WITH_G) e[j][k] = post_elem<T>(args.g, e[j][k]);
                }
                acc.store_slot(start + (warp_slot0 + (u64)j * 32 + lane) * EPV, e[j]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < VECS; ++j) {
                const T p = Op::template apply<T>(base, slot_excl[j]);
#pragma unroll
                for (int k = 0; k < EPV; ++k) {
                    const u64 off = (warp_slot0 + (u64)j * 32 + lane) * EPV + k;
                    T v = Op::template apply<T>(p, e[j][k]);
                    if constexpr (WITH_G) v = post_elem<T>(args.g, v);
                    if (off < count) acc.store_elem(start + off, v);
                }
            }
        }
    };
    if (args.g == KF_POST_IDENTITY) emit(std::false_type{});
    else emit(std::true_type{});
}

}  // namespace kf
