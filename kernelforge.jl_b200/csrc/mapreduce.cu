// Full (1-D) mapreduce for sm_100a: dst[0] = g(op-reduce_i f(src[i])).
//
// One launch of a persistent grid (a multiple of the SM count). Each CTA walks the input in
// grid-strided strips of THREADS*UNROLL 16-byte vectors with UNROLL independent 128-bit
// streaming loads in flight per thread, folds its strip-local values in registers, reduces
// across the CTA with shuffles (redux.sync for 32-bit integer ops) and writes one partial.
// The last CTA to finish (atomic completion counter in the workspace header) folds the partials
// in index order and applies g, so no CTA ever waits on another and the result is
// deterministic for a given launch configuration.
//
// Follows the semantics of mapreduce1d_kernel! (src/mapreduce/1D/mapreduce1d_kernel.jl:5-94 of
// KernelForge.jl): accumulate in the element type, strided order (op must be commutative), g
// applied once at the end.
#include "mapreduce_impl.cuh"

namespace kf {

template <typename T, typename Op, int THREADS, int UNROLL>
__global__ void __launch_bounds__(THREADS)
mapreduce_kernel(const T *__restrict__ src, u64 n, T *dst, T *partials, u32 *header, int f, int g) {
    constexpr int EPV = 16 / sizeof(T);  // elements per 16-byte vector
    __shared__ T smem[THREADS / 32];
    __shared__ bool is_last;

    const u32 tid = threadIdx.x;
    // Peel to a 16-byte boundary: [0, head) scalar, then nvec whole vectors, then a scalar tail.
    const u64 mis = ((uintptr_t)src & 15u) / sizeof(T);
    u64 head = mis ? (EPV - mis) : 0;
    if (head > n) head = n;
    const u64 nvec = (n - head) / EPV;
    const u64 tail_start = head + nvec * EPV;
    const uint4 *vsrc = reinterpret_cast<const uint4 *>(src + head);

    T acc[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) acc[u] = Op::template identity<T>();

    constexpr u64 STRIP = (u64)THREADS * UNROLL;
    const u64 stride = (u64)gridDim.x * STRIP;
    u64 base = (u64)blockIdx.x * STRIP;
    // One-byte elements under `+` without a map stay packed: the sum of a word's four bytes is one dp4a,
    // and the 32-bit running sums agree with the element-type (wrap-around) sum modulo 256, for signed
    // and unsigned bytes alike. The per-element code below needs an instruction pair per byte and is
    // issue-bound at 0.65 of the copy rate.
    if constexpr (sizeof(T) == 1 && std::is_same<Op, OpAdd>::value) {
        if (f == KF_MAP_IDENTITY) {
            u32 pacc[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) pacc[u] = 0;
            for (; base + STRIP <= nvec; base += stride) {
                uint4 v[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) v[u] = ld_stream_v4(vsrc + base + (u64)u * THREADS + tid);
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    pacc[u] = __dp4a(v[u].x, 0x01010101u, pacc[u]);
                    pacc[u] = __dp4a(v[u].y, 0x01010101u, pacc[u]);
                    pacc[u] = __dp4a(v[u].z, 0x01010101u, pacc[u]);
                    pacc[u] = __dp4a(v[u].w, 0x01010101u, pacc[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) acc[u] = (T)pacc[u];
        }
    }
    // Whole strips: no bounds checks, UNROLL loads issued back to back.
    for (; base + STRIP <= nvec; base += stride) {
        uint4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) v[u] = ld_stream_v4(vsrc + base + (u64)u * THREADS + tid);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            T e[EPV];
            memcpy(e, &v[u], 16);
            T t = apply_map<T>(f, e[0]);
#pragma unroll
            for (int k = 1; k < EPV; ++k) t = Op::template apply<T>(t, apply_map<T>(f, e[k]));
            acc[u] = Op::template apply<T>(acc[u], t);
        }
    }
    // Ragged last strip (at most one per CTA).
    if (base < nvec) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const u64 idx = base + (u64)u * THREADS + tid;
            if (idx < nvec) {
                uint4 v = ld_stream_v4(vsrc + idx);
                T e[EPV];
                memcpy(e, &v, 16);
#pragma unroll
                for (int k = 0; k < EPV; ++k) acc[u] = Op::template apply<T>(acc[u], apply_map<T>(f, e[k]));
            }
        }
    }
    // Scalar head and tail (fewer than EPV elements each) go to CTA 0.
    if (blockIdx.x == 0) {
        if (tid < head) acc[0] = Op::template apply<T>(acc[0], apply_map<T>(f, src[tid]));
        const u64 t = tail_start + tid;
        if (t < n) acc[0] = Op::template apply<T>(acc[0], apply_map<T>(f, src[t]));
    }

    T v = acc[0];
#pragma unroll
    for (int u = 1; u < UNROLL; ++u) v = Op::template apply<T>(v, acc[u]);
    v = block_reduce<Op, T, THREADS>(v, smem);

    // The kernel is chained behind the one that clears the workspace header (programmatic dependent
    // launch): everything above only reads the input, so it may run while that kernel is still in flight;
    // the header (completion counter, status) is first touched here.
    grid_dep_wait();
    if (tid == 0) {
        partials[blockIdx.x] = v;
        __threadfence();  // partial visible device-wide before the counter moves
        const u32 done = atomicAdd(&header[kTicketBase], 1u);
        is_last = (done == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();  // order the partial reads after the counter observation

    // Last CTA: fold the partials in index order (thread-strided, then the same CTA reduction).
    T r = Op::template identity<T>();
    for (u32 i = tid; i < gridDim.x; i += THREADS) {
        T x = *((const volatile T *)(partials + i));  // written by other CTAs: no cached read
        r = Op::template apply<T>(r, x);
    }
    r = block_reduce<Op, T, THREADS>(r, smem);
    if (tid == 0) dst[0] = apply_post<T>(g, r);
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------

// Clears the 256-byte workspace header (completion counter, status words).
__global__ void zero_header_kernel(u32 *header) { header[threadIdx.x] = 0; }

struct MrVariant {
    int threads, unroll;
};
static const MrVariant kMrVariants[] = {{256, 4}, {512, 4}, {256, 8}};
constexpr int kNumMrVariants = 3;

// Persistent-grid size: the table's (or the default) CTAs per SM, but never more CTAs than there
// are strips of input: fewer CTAs mean fewer partials for the last CTA to fold.
static int mr_clamp_blocks(u64 blocks, int threads, int unroll, u64 n_bytes) {
    const u64 strip_bytes = (u64)threads * unroll * 16;
    u64 need = (n_bytes + strip_bytes - 1) / strip_bytes;
    if (need < 1) need = 1;
    if (blocks > need) blocks = need;
    return (int)blocks;
}

int mapreduce_resolve(int dtype, u64 n, const kf_launch_cfg *cfg, int *variant, int *blocks) {
    kf_launch_cfg t;
    const int eb = dtype_bytes(dtype);
    if (eb == 0) return KF_ERR_INVALID_ARG;
    kf_launch_table_lookup(KF_PRIM_MAPREDUCE, eb, n, &t);
    if (cfg) {
        if (cfg->threads) t.threads = cfg->threads;
        if (cfg->items) t.items = cfg->items;
        if (cfg->blocks) t.blocks = cfg->blocks;
    }
    int v = -1;
    for (int i = 0; i < kNumMrVariants; ++i)
        if (kMrVariants[i].threads == t.threads && kMrVariants[i].unroll == t.items) v = i;
    if (v < 0) return KF_ERR_UNSUPPORTED;
    int b;
    if (cfg && cfg->blocks > 0) {
        b = cfg->blocks;  // explicit override: taken as given
    } else {
        const u64 dflt = t.blocks > 0 ? (u64)t.blocks : (u64)device_sm_count() * (2048 / t.threads);
        b = mr_clamp_blocks(dflt, t.threads, t.items, n * (u64)eb);
    }
    if (b < 1 || b > (1 << 20)) return KF_ERR_INVALID_ARG;
    *variant = v;
    *blocks = b;
    return KF_OK;
}

template <typename T, typename Op>
static int launch_mr(int variant, int blocks, const void *src, u64 n, void *dst, void *partials, u32 *header,
                     int f, int g, cudaStream_t s) {
    const T *in = (const T *)src;
    T *out = (T *)dst;
    T *part = (T *)partials;
    switch (variant) {
    case 0: KF_CUDA_TRY(launch_chained(mapreduce_kernel<T, Op, 256, 4>, (unsigned)blocks, 256u, 0, s, in, n, out, part, header, f, g)); note_launch(); break;
    case 1: KF_CUDA_TRY(launch_chained(mapreduce_kernel<T, Op, 512, 4>, (unsigned)blocks, 512u, 0, s, in, n, out, part, header, f, g)); note_launch(); break;
    case 2: KF_CUDA_TRY(launch_chained(mapreduce_kernel<T, Op, 256, 8>, (unsigned)blocks, 256u, 0, s, in, n, out, part, header, f, g)); note_launch(); break;
    default: return KF_ERR_UNSUPPORTED;
    }
    KF_CUDA_TRY(cudaGetLastError());
    return KF_OK;
}

template <typename T>
static int dispatch_mr_op(int op, int variant, int blocks, const void *src, u64 n, void *dst, void *partials,
                          u32 *header, int f, int g, cudaStream_t s) {
    switch (op) {
    case KF_OP_ADD: return launch_mr<T, OpAdd>(variant, blocks, src, n, dst, partials, header, f, g, s);
    case KF_OP_MUL: return launch_mr<T, OpMul>(variant, blocks, src, n, dst, partials, header, f, g, s);
    case KF_OP_MIN: return launch_mr<T, OpMin>(variant, blocks, src, n, dst, partials, header, f, g, s);
    case KF_OP_MAX: return launch_mr<T, OpMax>(variant, blocks, src, n, dst, partials, header, f, g, s);
    default: break;
    }
    if constexpr (!IsFloat<T>::value) {
        switch (op) {
        case KF_OP_AND: return launch_mr<T, OpAnd>(variant, blocks, src, n, dst, partials, header, f, g, s);
        case KF_OP_OR: return launch_mr<T, OpOr>(variant, blocks, src, n, dst, partials, header, f, g, s);
        case KF_OP_XOR: return launch_mr<T, OpXor>(variant, blocks, src, n, dst, partials, header, f, g, s);
        default: break;
        }
    }
    return KF_ERR_UNSUPPORTED;
}

}  // namespace kf

using namespace kf;

extern "C" size_t kf_mapreduce_workspace_bytes(int32_t dtype, uint64_t n, const kf_launch_cfg *cfg) {
    int variant, blocks;
    if (mapreduce_resolve(dtype, n, cfg, &variant, &blocks) != KF_OK) return 0;
    return kHeaderBytes + align_up((size_t)blocks * dtype_bytes(dtype), 256);
}

extern "C" int32_t kf_mapreduce(int32_t f, int32_t op, int32_t g, int32_t dtype, const void *src, uint64_t n,
                                void *dst, void *ws, size_t ws_bytes, const kf_launch_cfg *cfg,
                                kf_stream_t stream) {
    if (n == 0) return KF_ERR_EMPTY_REDUCTION;
    if (!src || !dst || !ws) return KF_ERR_INVALID_ARG;
    if (f < KF_MAP_IDENTITY || f > KF_MAP_ABS) return KF_ERR_UNSUPPORTED;
    if (g < KF_POST_IDENTITY || g > KF_POST_SQRT) return KF_ERR_UNSUPPORTED;
    const int eb = dtype_bytes(dtype);
    if (eb == 0) return KF_ERR_INVALID_ARG;
    if (((uintptr_t)src % eb) || ((uintptr_t)dst % eb) || ((uintptr_t)ws % 256)) return KF_ERR_INVALID_ARG;
    if (g == KF_POST_SQRT && dtype != KF_F32 && dtype != KF_F64) return KF_ERR_UNSUPPORTED;
    int variant, blocks;
    int rc = mapreduce_resolve(dtype, n, cfg, &variant, &blocks);
    if (rc != KF_OK) return rc;
    const size_t need = kHeaderBytes + align_up((size_t)blocks * eb, 256);
    if (ws_bytes < need) return KF_ERR_WORKSPACE_TOO_SMALL;
    KF_LOGF("mapreduce f=%d op=%d g=%d dtype=%d n=%llu: %dx%d, %d CTAs", f, op, g, dtype, (unsigned long long)n,
            kMrVariants[variant].threads, kMrVariants[variant].unroll, blocks);

    cudaStream_t s = (cudaStream_t)stream;
    u32 *header = (u32 *)ws;
    void *partials = (char *)ws + kHeaderBytes;
    // a kernel of the library instead of a memset node, so that the reduction can be chained behind it
    zero_header_kernel<<<1, kHeaderBytes / 4, 0, s>>>(header); note_launch();
    switch (dtype) {
    case KF_U8: return dispatch_mr_op<uint8_t>(op, variant, blocks, src, n, dst, partials, header, f, g, s);
    case KF_I8: return dispatch_mr_op<int8_t>(op, variant, blocks, src, n, dst, partials, header, f, g, s);
    case KF_U16: return dispatch_mr_op<uint16_t>(op, variant, blocks, src, n, dst, partials, header, f, g, s);
    case KF_I16: return dispatch_mr_op<int16_t>(op, variant, blocks, src, n, dst, partials, header, f, g, s);
    case KF_U32: return dispatch_mr_op<uint32_t>(op, variant, blocks, src, n, dst, partials, header, f, g, s);
    case KF_I32: return dispatch_mr_op<int32_t>(op, variant, blocks, src, n, dst, partials, header, f, g, s);
    case KF_U64: return dispatch_mr_op<u64>(op, variant, blocks, src, n, dst, partials, header, f, g, s);
    case KF_I64: return dispatch_mr_op<long long>(op, variant, blocks, src, n, dst, partials, header, f, g, s);
    case KF_F32: return dispatch_mr_op<float>(op, variant, blocks, src, n, dst, partials, header, f, g, s);
    case KF_F64: return dispatch_mr_op<double>(op, variant, blocks, src, n, dst, partials, header, f, g, s);
    default: return KF_ERR_INVALID_ARG;
    }
}
