// Tuple form of the full mapreduce for sm_100a: dst[0] = g(op-reduce_i fn(x1[i], ..., xk[i])), the
// dot-product family. Same structure as the one-array kernel (mapreduce.cu): a persistent grid,
// grid-strided strips with UNROLL independent 128-bit streaming loads per array in flight per
// thread, shuffle / redux.sync reductions, one partial per CTA, the last CTA to finish folds the
// partials in index order. HBM-bound: k * n * sizeof(T) bytes.
//
// Follows the tuple methods of mapreduce1d! (src/mapreduce/1D/mapreduce1d.jl:177-288 of
// KernelForge.jl): accumulate in the element type, strided order, g applied once at the end.
#include "mapreduce_impl.cuh"

namespace kf {

template <typename T, int NSRC> struct MultiSrc {
    const T *p[NSRC];
};

template <typename T, int NSRC> __device__ __forceinline__ T apply_mapn(int fn, const T (&x)[NSRC]) {
    if (fn == KF_MAPN_SQDIFF) {
        const T d = (T)(x[0] - x[1]);
        return (T)(d * d);
    }
    if (fn == KF_MAPN_WSQ) return (T)((T)(x[0] * x[1]) * x[1]);
    T r = x[0];
#pragma unroll
    for (int a = 1; a < NSRC; ++a) r = (T)(r * x[a]);
    return r;
}

template <typename T, typename Op, int NSRC, int THREADS, int UNROLL>
__global__ void __launch_bounds__(THREADS)
mapreduce_multi_kernel(MultiSrc<T, NSRC> src, u64 n, u64 head, int vec_ok, T *dst, T *partials, u32 *header, int fn, int g) {
    constexpr int EPV = 16 / sizeof(T);
    __shared__ T smem[THREADS / 32];
    __shared__ bool is_last;
    const u32 tid = threadIdx.x;

    T acc[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) acc[u] = Op::template identity<T>();

    auto fold_elem = [&](T &a, u64 i) {
        T x[NSRC];
#pragma unroll
        for (int s = 0; s < NSRC; ++s) x[s] = src.p[s][i];
        a = Op::template apply<T>(a, apply_mapn<T, NSRC>(fn, x));
    };

    if (vec_ok) {
        // [0, head) scalar, then nvec whole vectors (every array is 16-byte aligned there), then a scalar tail
        const u64 nvec = (n - head) / EPV;
        const u64 tail_start = head + nvec * EPV;
        constexpr u64 STRIP = (u64)THREADS * UNROLL;
        const u64 stride = (u64)gridDim.x * STRIP;
        for (u64 base = (u64)blockIdx.x * STRIP; base < nvec; base += stride) {
            uint4 v[UNROLL][NSRC];
            bool ok[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const u64 idx = base + (u64)u * THREADS + tid;
                ok[u] = idx < nvec;
                if (ok[u]) {
#pragma unroll
                    for (int s = 0; s < NSRC; ++s) v[u][s] = ld_stream_v4(reinterpret_cast<const uint4 *>(src.p[s] + head) + idx);
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                if (ok[u]) {
                    T e[NSRC][EPV];
#pragma unroll
                    for (int s = 0; s < NSRC; ++s) memcpy(e[s], &v[u][s], 16);
#pragma unroll
                    for (int k = 0; k < EPV; ++k) {
                        T x[NSRC];
#pragma unroll
                        for (int s = 0; s < NSRC; ++s) x[s] = e[s][k];
                        acc[u] = Op::template apply<T>(acc[u], apply_mapn<T, NSRC>(fn, x));
                    }
                }
            }
        }
        if (blockIdx.x == 0) {
            if (tid < head) fold_elem(acc[0], tid);
            const u64 t = tail_start + tid;
            if (t < n) fold_elem(acc[0], t);
        }
    } else {
        const u64 stride = (u64)gridDim.x * THREADS;
        for (u64 i = (u64)blockIdx.x * THREADS + tid; i < n; i += stride) fold_elem(acc[0], i);
    }

    T v = acc[0];
#pragma unroll
    for (int u = 1; u < UNROLL; ++u) v = Op::template apply<T>(v, acc[u]);
    v = block_reduce<Op, T, THREADS>(v, smem);

    if (tid == 0) {
        partials[blockIdx.x] = v;
        __threadfence();  // partial visible device-wide before the counter moves
        const u32 done = atomicAdd(&header[kTicketBase], 1u);
        is_last = (done == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();  // order the partial reads after the counter observation

    T r = Op::template identity<T>();
    for (u32 i = tid; i < gridDim.x; i += THREADS) {
        T x = *((const volatile T *)(partials + i));  // written by other CTAs: no cached read
        r = Op::template apply<T>(r, x);
    }
    r = block_reduce<Op, T, THREADS>(r, smem);
    if (tid == 0) dst[0] = apply_post<T>(g, r);
}

template <typename T, typename Op, int NSRC>
static int launch_multi(int blocks, const void *const *srcs, u64 n, void *dst, void *partials, u32 *header, int fn, int g,
                        cudaStream_t s) {
    constexpr int THREADS = 256, UNROLL = 4;
    constexpr int EPV = 16 / sizeof(T);
    MultiSrc<T, NSRC> m;
    const uintptr_t mis = (uintptr_t)srcs[0] & 15u;
    bool same = true;
    for (int a = 0; a < NSRC; ++a) {
        m.p[a] = static_cast<const T *>(srcs[a]);
        same = same && (((uintptr_t)srcs[a] & 15u) == mis);
    }
    u64 head = mis ? (u64)(EPV - mis / sizeof(T)) : 0;
    if (head > n) head = n;
    mapreduce_multi_kernel<T, Op, NSRC, THREADS, UNROLL><<<blocks, THREADS, 0, s>>>(m, n, head, same ? 1 : 0, (T *)dst, (T *)partials,
                                                                                   header, fn, g); note_launch();
    KF_CUDA_TRY(cudaGetLastError());
    return KF_OK;
}

template <typename T, typename Op>
static int dispatch_multi_n(int nsrc, int blocks, const void *const *srcs, u64 n, void *dst, void *partials, u32 *header, int fn,
                            int g, cudaStream_t s) {
    switch (nsrc) {
    case 2: return launch_multi<T, Op, 2>(blocks, srcs, n, dst, partials, header, fn, g, s);
    case 3: return launch_multi<T, Op, 3>(blocks, srcs, n, dst, partials, header, fn, g, s);
    case 4: return launch_multi<T, Op, 4>(blocks, srcs, n, dst, partials, header, fn, g, s);
    default: return KF_ERR_UNSUPPORTED;
    }
}

template <typename T>
static int dispatch_multi_op(int op, int nsrc, int blocks, const void *const *srcs, u64 n, void *dst, void *partials, u32 *header,
                             int fn, int g, cudaStream_t s) {
    switch (op) {
    case KF_OP_ADD: return dispatch_multi_n<T, OpAdd>(nsrc, blocks, srcs, n, dst, partials, header, fn, g, s);
    case KF_OP_MUL: return dispatch_multi_n<T, OpMul>(nsrc, blocks, srcs, n, dst, partials, header, fn, g, s);
    case KF_OP_MIN: return dispatch_multi_n<T, OpMin>(nsrc, blocks, srcs, n, dst, partials, header, fn, g, s);
    case KF_OP_MAX: return dispatch_multi_n<T, OpMax>(nsrc, blocks, srcs, n, dst, partials, header, fn, g, s);
    default: return KF_ERR_UNSUPPORTED;
    }
}

}  // namespace kf

using namespace kf;

extern "C" int32_t kf_mapreduce_multi(int32_t fn, int32_t op, int32_t g, int32_t dtype, const void *const *srcs, int32_t nsrc,
                                      uint64_t n, void *dst, void *ws, size_t ws_bytes, const kf_launch_cfg *cfg,
                                      kf_stream_t stream) {
    if (n == 0) return KF_ERR_EMPTY_REDUCTION;
    if (!srcs || !dst || !ws) return KF_ERR_INVALID_ARG;
    if (nsrc < 2 || nsrc > 4) return KF_ERR_UNSUPPORTED;
    if (fn < KF_MAPN_PROD || fn > KF_MAPN_WSQ) return KF_ERR_UNSUPPORTED;
    if (fn != KF_MAPN_PROD && nsrc != 2) return KF_ERR_UNSUPPORTED;
    if (g < KF_POST_IDENTITY || g > KF_POST_SQRT) return KF_ERR_UNSUPPORTED;
    const int eb = dtype_bytes(dtype);
    if (eb == 0) return KF_ERR_INVALID_ARG;
    for (int a = 0; a < nsrc; ++a)
        if (!srcs[a] || ((uintptr_t)srcs[a] % eb)) return KF_ERR_INVALID_ARG;
    if (((uintptr_t)dst % eb) || ((uintptr_t)ws % 256)) return KF_ERR_INVALID_ARG;
    if (g == KF_POST_SQRT && dtype != KF_F32 && dtype != KF_F64) return KF_ERR_UNSUPPORTED;
    int variant, blocks;
    int rc = mapreduce_resolve(dtype, n, cfg, &variant, &blocks);
    if (rc != KF_OK) return rc;
    const size_t need = kHeaderBytes + align_up((size_t)blocks * eb, 256);
    if (ws_bytes < need) return KF_ERR_WORKSPACE_TOO_SMALL;

    cudaStream_t s = (cudaStream_t)stream;
    u32 *header = (u32 *)ws;
    void *partials = (char *)ws + kHeaderBytes;
    KF_CUDA_TRY(cudaMemsetAsync(header, 0, kHeaderBytes, s));
    switch (dtype) {
    case KF_U8: return dispatch_multi_op<uint8_t>(op, nsrc, blocks, srcs, n, dst, partials, header, fn, g, s);
    case KF_I8: return dispatch_multi_op<int8_t>(op, nsrc, blocks, srcs, n, dst, partials, header, fn, g, s);
    case KF_U16: return dispatch_multi_op<uint16_t>(op, nsrc, blocks, srcs, n, dst, partials, header, fn, g, s);
    case KF_I16: return dispatch_multi_op<int16_t>(op, nsrc, blocks, srcs, n, dst, partials, header, fn, g, s);
    case KF_U32: return dispatch_multi_op<uint32_t>(op, nsrc, blocks, srcs, n, dst, partials, header, fn, g, s);
    case KF_I32: return dispatch_multi_op<int32_t>(op, nsrc, blocks, srcs, n, dst, partials, header, fn, g, s);
    case KF_U64: return dispatch_multi_op<u64>(op, nsrc, blocks, srcs, n, dst, partials, header, fn, g, s);
    case KF_I64: return dispatch_multi_op<long long>(op, nsrc, blocks, srcs, n, dst, partials, header, fn, g, s);
    case KF_F32: return dispatch_multi_op<float>(op, nsrc, blocks, srcs, n, dst, partials, header, fn, g, s);
    case KF_F64: return dispatch_multi_op<double>(op, nsrc, blocks, srcs, n, dst, partials, header, fn, g, s);
    default: return KF_ERR_INVALID_ARG;
    }
}
