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
// {status:32 | value:32} for elements up to 4 bytes, or two such words {status | low half},
// {status | high half} for 8-byte elements: each word validates itself and a reader retries
// until both carry the same status, so no fence separates value and flag. Every wait is
// bounded; a tile that gives up records KF_ERR_TIMEOUT in the workspace header and publishes a
// poison status that makes its successors return too.
//
// Semantics follow scan_kernel_packed! / scan_kernel! of KernelForge.jl
// (src/scan/scan_kernel.jl:310-478, 94-299): inclusive, f applied on load, left-to-right order.
#pragma once

#include "common.cuh"

namespace kf {

enum : u32 { kInvalid = 0, kAggregate = 1, kPrefix = 2, kPoison = 3 };

// ---- descriptors ------------------------------------------------------------------------------
template <typename T> struct Desc {
    static constexpr int WORDS = sizeof(T) <= 4 ? 1 : 2;

    static __device__ __forceinline__ void publish(u64 *desc, u64 tile, u32 status, T v) {
        if constexpr (WORDS == 1) {
            u32 bits = 0;
            memcpy(&bits, &v, sizeof(T));
            st_relaxed_u64(desc + tile, ((u64)status << 32) | bits);
        } else {
            u32 h[2];
            memcpy(h, &v, 8);
            st_relaxed_u64(desc + 2 * tile, ((u64)status << 32) | h[0]);
            st_relaxed_u64(desc + 2 * tile + 1, ((u64)status << 32) | h[1]);
        }
    }
    // Returns the status (kInvalid when not yet published or when the two halves disagree).
    static __device__ __forceinline__ u32 read(const u64 *desc, u64 tile, T &v) {
        if constexpr (WORDS == 1) {
            const u64 w = ld_relaxed_u64(desc + tile);
            const u32 bits = (u32)w;
            memcpy(&v, &bits, sizeof(T));
            return (u32)(w >> 32);
        } else {
            const u64 w0 = ld_relaxed_u64(desc + 2 * tile);
            const u64 w1 = ld_relaxed_u64(desc + 2 * tile + 1);
            u32 h[2] = {(u32)w0, (u32)w1};
            memcpy(&v, h, 8);
            const u32 s0 = (u32)(w0 >> 32), s1 = (u32)(w1 >> 32);
            return s0 == s1 ? s0 : (u32)kInvalid;
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

template <typename T> __device__ __forceinline__ T map_elem(int f, T x) { return apply_map<T>(f, x); }
template <> __device__ __forceinline__ Affine map_elem<Affine>(int, Affine x) { return x; }

struct ScanArgs {
    u64 n;          // elements
    u64 head;       // elements before the first 16-byte boundary (tile 0 when > 0)
    u64 ntiles;
    u64 *desc;      // Desc<T>::WORDS words per tile
    u32 *header;    // workspace header (status, ticket)
    const void *init;  // optional left seed (one element) or nullptr
    int vec_ok;     // all arrays share their 16-byte misalignment: full tiles use 128-bit accesses
    int f;
};

// Look-back over the descriptors of tiles [0, tile), by one full warp. Returns false if the wait
// ran out or a predecessor was poisoned. On success `excl` (valid in every lane) is the
// combination of all predecessors in order.
template <typename T, typename Op>
__device__ __forceinline__ bool lookback(const u64 *desc, u64 tile, u32 lane, T &excl, bool &timed_out) {
    T acc = Op::template identity<T>();
    long long cur = (long long)tile - 1;
    u32 spins = 0;
    timed_out = false;
    while (true) {
        const long long mine = cur - (long long)lane;
        T v = Op::template identity<T>();
        u32 st = kPrefix;  // lanes before tile 0 read as "prefix = identity"
        if (mine >= 0) st = Desc<T>::read(desc, (u64)mine, v);
        const u32 poison = __ballot_sync(0xFFFFFFFFu, st == kPoison);
        if (poison) return false;
        const u32 pfx = __ballot_sync(0xFFFFFFFFu, st == kPrefix);
        const u32 inv = __ballot_sync(0xFFFFFFFFu, st == kInvalid);
        const int last = pfx ? (__ffs(pfx) - 1) : 31;  // nearest tile with a full prefix
        const u32 need = last == 31 ? 0xFFFFFFFFu : ((2u << last) - 1u);
        if (inv & need) {
            if (++spins > kSpinLimit) {
                timed_out = true;
                return false;
            }
            if (spins > 8) __nanosleep(spins > 64 ? 256 : 32);
            continue;
        }
        // Ordered fold of lanes 0..last: a higher lane is an earlier tile, i.e. the left operand.
        T x = (int)lane <= last ? v : Op::template identity<T>();
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            T y = shfl_down(x, d);
            if (lane + d < 32) x = Op::template apply<T>(y, x);
        }
        x = shfl_idx(x, 0);
        acc = Op::template apply<T>(x, acc);
        if (pfx) break;
        cur -= 32;
    }
    excl = acc;
    return true;
}

template <typename T, typename Op, typename Access, int THREADS, int VECS>
__global__ void __launch_bounds__(THREADS) scan_kernel(Access acc, ScanArgs args) {
    constexpr int EPV = Access::EPV;
    constexpr int WARPS = THREADS / 32;
    constexpr u64 TILE = (u64)THREADS * VECS * EPV;

    __shared__ T s_warp_total[WARPS];
    __shared__ T s_tile_excl;
    __shared__ u64 s_tile;
    __shared__ int s_abort;

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
        for (int j = 0; j < VECS; ++j) {  // VECS independent shuffles per step
            T up = shfl_up(incl[j], d);
            if (lane >= (u32)d) incl[j] = Op::template apply<T>(up, incl[j]);
        }
    }
    // Exclusive prefix of each slot within the warp: carry over rows j, then lanes before mine.
    T slot_excl[VECS];
    T carry = Op::template identity<T>();
#pragma unroll
    for (int j = 0; j < VECS; ++j) {
        T prev = shfl_up(incl[j], 1);
        if (lane == 0) prev = Op::template identity<T>();
        slot_excl[j] = Op::template apply<T>(carry, prev);
        carry = Op::template apply<T>(carry, shfl_idx(incl[j], 31));
    }
    if (lane == 0) s_warp_total[warp] = carry;
    __syncthreads();

    // ---- warp prefix within the tile and the tile aggregate ----------------------------------
    T warp_excl = Op::template identity<T>();
    T tile_total = Op::template identity<T>();
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
        const T t = s_warp_total[w];
        if (w < (int)warp) warp_excl = Op::template apply<T>(warp_excl, t);
        tile_total = Op::template apply<T>(tile_total, t);
    }

    // ---- publish, look back, publish ---------------------------------------------------------
    if (warp == 0) {
        T excl = Op::template identity<T>();
        bool ok = true, timed_out = false;
        if (tile == 0) {
            if (args.init) excl = *reinterpret_cast<const T *>(args.init);
        } else {
            if (lane == 0) Desc<T>::publish(args.desc, tile, kAggregate, tile_total);
            ok = lookback<T, Op>(args.desc, tile, lane, excl, timed_out);
        }
        if (lane == 0) {
            if (ok) {
                Desc<T>::publish(args.desc, tile, kPrefix, Op::template apply<T>(excl, tile_total));
                s_tile_excl = excl;
            } else {
                if (timed_out) record_error(args.header, KF_ERR_TIMEOUT, (u32)tile);
                Desc<T>::publish(args.desc, tile, kPoison, Op::template identity<T>());
                s_abort = 1;
            }
        }
    }
    __syncthreads();
    if (s_abort) return;

    // ---- apply the prefix and store -----------------------------------------------------------
    const T base = Op::template apply<T>(s_tile_excl, warp_excl);
    if (fast) {
#pragma unroll
        for (int j = 0; j < VECS; ++j) {
            const T p = Op::template apply<T>(base, slot_excl[j]);
#pragma unroll
            for (int k = 0; k < EPV; ++k) e[j][k] = Op::template apply<T>(p, e[j][k]);
            acc.store_slot(start + (warp_slot0 + (u64)j * 32 + lane) * EPV, e[j]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < VECS; ++j) {
            const T p = Op::template apply<T>(base, slot_excl[j]);
#pragma unroll
            for (int k = 0; k < EPV; ++k) {
                const u64 off = (warp_slot0 + (u64)j * 32 + lane) * EPV + k;
                if (off < count) acc.store_elem(start + off, Op::template apply<T>(p, e[j][k]));
            }
        }
    }
}

// ---- host-side geometry shared by the workspace query and the launch ---------------------------
struct ScanVariant {
    int threads, vecs;
};
static const ScanVariant kScanVariants[] = {{256, 4}, {512, 4}, {512, 2}, {1024, 2}};
constexpr int kNumScanVariants = 4;

struct ScanPlan {
    int variant;
    u64 tile;     // elements per tile
    u64 ntiles;   // upper bound used for sizing (includes a possible head tile)
    int words;    // descriptor words per tile
};

int scan_plan(int elem_bytes, int epv, u64 n, const kf_launch_cfg *cfg, ScanPlan *plan);

template <typename T, typename Op, typename Access>
int scan_launch(int variant, const Access &acc, const ScanArgs &args, cudaStream_t s) {
    const unsigned grid = (unsigned)args.ntiles;
    switch (variant) {
    case 0: scan_kernel<T, Op, Access, 256, 4><<<grid, 256, 0, s>>>(acc, args); break;
    case 1: scan_kernel<T, Op, Access, 512, 4><<<grid, 512, 0, s>>>(acc, args); break;
    case 2: scan_kernel<T, Op, Access, 512, 2><<<grid, 512, 0, s>>>(acc, args); break;
    case 3: scan_kernel<T, Op, Access, 1024, 2><<<grid, 1024, 0, s>>>(acc, args); break;
    default: return KF_ERR_UNSUPPORTED;
    }
    KF_CUDA_TRY(cudaGetLastError());
    return KF_OK;
}

// One translation unit per element type instantiates this (keeps the build parallel).
template <typename T>
int scan_dispatch_ops(int op, int variant, const PlainAccess<T> &acc, const ScanArgs &args, cudaStream_t s) {
    switch (op) {
    case KF_OP_ADD: return scan_launch<T, OpAdd>(variant, acc, args, s);
    case KF_OP_MUL: return scan_launch<T, OpMul>(variant, acc, args, s);
    case KF_OP_MIN: return scan_launch<T, OpMin>(variant, acc, args, s);
    case KF_OP_MAX: return scan_launch<T, OpMax>(variant, acc, args, s);
    default: break;
    }
    if constexpr (!IsFloat<T>::value) {
        switch (op) {
        case KF_OP_AND: return scan_launch<T, OpAnd>(variant, acc, args, s);
        case KF_OP_OR: return scan_launch<T, OpOr>(variant, acc, args, s);
        case KF_OP_XOR: return scan_launch<T, OpXor>(variant, acc, args, s);
        default: break;
        }
    }
    return KF_ERR_UNSUPPORTED;
}

// Defined in scan_inst_*.cu
int scan_dispatch_u8(int op, int variant, const void *src, void *dst, const ScanArgs &args, cudaStream_t s);
int scan_dispatch_i8(int op, int variant, const void *src, void *dst, const ScanArgs &args, cudaStream_t s);
int scan_dispatch_u16(int op, int variant, const void *src, void *dst, const ScanArgs &args, cudaStream_t s);
int scan_dispatch_i16(int op, int variant, const void *src, void *dst, const ScanArgs &args, cudaStream_t s);
int scan_dispatch_u32(int op, int variant, const void *src, void *dst, const ScanArgs &args, cudaStream_t s);
int scan_dispatch_i32(int op, int variant, const void *src, void *dst, const ScanArgs &args, cudaStream_t s);
int scan_dispatch_u64(int op, int variant, const void *src, void *dst, const ScanArgs &args, cudaStream_t s);
int scan_dispatch_i64(int op, int variant, const void *src, void *dst, const ScanArgs &args, cudaStream_t s);
int scan_dispatch_f32(int op, int variant, const void *src, void *dst, const ScanArgs &args, cudaStream_t s);
int scan_dispatch_f64(int op, int variant, const void *src, void *dst, const ScanArgs &args, cudaStream_t s);
int scan_dispatch_affine_aos(int variant, const float *src, float *dst, const ScanArgs &args, cudaStream_t s);
int scan_dispatch_affine_soa(int variant, const float *a_src, const float *b_src, float *a_dst, float *b_dst,
                             const ScanArgs &args, cudaStream_t s);

#define KF_SCAN_INSTANTIATE(NAME, T)                                                                     \
    namespace kf {                                                                                       \
    int scan_dispatch_##NAME(int op, int variant, const void *src, void *dst, const ScanArgs &args,      \
                             cudaStream_t s) {                                                           \
        PlainAccess<T> acc{(const T *)src, (T *)dst};                                                    \
        return scan_dispatch_ops<T>(op, variant, acc, args, s);                                          \
    }                                                                                                    \
    }

}  // namespace kf
