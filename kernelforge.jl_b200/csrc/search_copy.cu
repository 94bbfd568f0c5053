// The callers one step out of the reduction path, for sm_100a: first extremal element (argmax /
// argmin), first / last element satisfying a comparison (findfirst / findlast), and the vectorised
// copy and fill that double as roofline calibration kernels. All are HBM-bound streaming kernels
// built like the mapreduce kernel: persistent grids, 128-bit streaming accesses, shuffle
// reductions, a last-CTA fold or one atomic per CTA.
//
// Semantics follow KernelForge.jl: argmax1d (src/search/argmax.jl:8-86, kernel
// src/search/argmax_kernel.jl:1-148: `rel` is a strict comparison, ties go to the smallest index),
// findfirst / findlast (src/search/findfirst.jl:3-110), vcopy! / setvalue! (src/copy/copy.jl:1-55).
// Indices are 0-based here. findfirst reports "not found" as UINT64_MAX; findlast stores found indices
// as index + 1, so that 0 means "not found".
#include "mapreduce_impl.cuh"

#include <cstdlib>

namespace kf {

// ---- argmax ---------------------------------------------------------------------------------------
template <typename T> struct Best {
    T v;
    u64 i;  // ~0: nothing seen yet
};
// Is a better than b? Strict relation first, then the smaller index among equals; "nothing seen"
// loses against anything.
template <typename T, bool GREATER> __device__ __forceinline__ bool better(const Best<T> &a, const Best<T> &b) {
    if (a.i == ~0ull) return false;
    if (b.i == ~0ull) return true;
    const bool rel = GREATER ? (a.v > b.v) : (a.v < b.v);
    if constexpr (IsFloat<T>::value) {
        if (b.v != b.v) return a.v == a.v || a.i < b.i;  // a NaN loses against any number, and against an earlier NaN
    }
    return rel || (a.v == b.v && a.i < b.i);
}
// Does the value a beat the value b under the strict relation? (A NaN b loses against any number, so
// that a NaN only survives where nothing else was seen, and then the earliest one does.)
template <typename T, bool GREATER> __device__ __forceinline__ bool value_wins(T a, T b) {
    const bool rel = GREATER ? (a > b) : (a < b);
    if constexpr (IsFloat<T>::value) return rel || (b != b && a == a);
    else return rel;
}
template <typename T, bool GREATER> __device__ __forceinline__ Best<T> warp_best(Best<T> b) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        Best<T> o;
        o.v = shfl_down(b.v, d);
        o.i = shfl_down(b.i, d);
        if (better<T, GREATER>(o, b)) b = o;
    }
    return b;
}
template <typename T, bool GREATER, int THREADS> __device__ __forceinline__ Best<T> block_best(Best<T> b, T *sv, u64 *si) {
    const u32 lane = lane_id(), warp = threadIdx.x >> 5;
    b = warp_best<T, GREATER>(b);
    if (lane == 0) {
        sv[warp] = b.v;
        si[warp] = b.i;
    }
    __syncthreads();
    if (warp == 0) {
        b.v = lane < THREADS / 32 ? sv[lane] : T();
        b.i = lane < THREADS / 32 ? si[lane] : ~0ull;
        b = warp_best<T, GREATER>(b);
    }
    __syncthreads();
    return b;  // valid in thread 0
}

template <typename T, bool GREATER, int THREADS, int UNROLL>
__global__ void __launch_bounds__(THREADS)
argmax_kernel(const T *__restrict__ src, u64 n, T *out_value, u64 *out_index, T *pv, u64 *pi, u32 *header, int f) {
    constexpr int EPV = 16 / sizeof(T);
    __shared__ T sv[THREADS / 32];
    __shared__ u64 si[THREADS / 32];
    __shared__ bool is_last;
    const u32 tid = threadIdx.x;
    const u64 mis = ((uintptr_t)src & 15u) / sizeof(T);
    u64 head = mis ? (EPV - mis) : 0;
    if (head > n) head = n;
    const u64 nvec = (n - head) / EPV;
    const u64 tail_start = head + nvec * EPV;
    const uint4 *vsrc = reinterpret_cast<const uint4 *>(src + head);

    // Hot loop: per thread the best VALUE seen and the index of the vector that holds it. A thread visits
    // its vectors in increasing index order, so the strict relation keeps the earliest one; the element
    // inside the vector is looked up once, after the loop. (Tracking a 64-bit element index per element
    // made this kernel issue-bound at half the copy rate.)
    T bestv = T();
    u64 best_vec = 0;
    bool seen = false;
    constexpr u64 STRIP = (u64)THREADS * UNROLL;
    const u64 stride = (u64)gridDim.x * STRIP;
    for (u64 base = (u64)blockIdx.x * STRIP; base < nvec; base += stride) {
        uint4 v[UNROLL];
        bool ok[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const u64 idx = base + (u64)u * THREADS + tid;
            ok[u] = idx < nvec;
            if (ok[u]) v[u] = ld_stream_v4(vsrc + idx);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (ok[u]) {
                T e[EPV];
                memcpy(e, &v[u], 16);
                T m = apply_map<T>(f, e[0]);
#pragma unroll
                for (int k = 1; k < EPV; ++k) {
                    const T x = apply_map<T>(f, e[k]);
                    m = value_wins<T, GREATER>(x, m) ? x : m;
                }
                if (!seen || value_wins<T, GREATER>(m, bestv)) {
                    bestv = m;
                    best_vec = base + (u64)u * THREADS + tid;
                    seen = true;
                }
            }
        }
    }
    Best<T> best;
    best.v = bestv;
    best.i = ~0ull;
    if (seen) {  // the first element of that vector that carries the best value (a NaN: the vector's first)
        const uint4 v = ld_stream_v4(vsrc + best_vec);
        T e[EPV];
        memcpy(e, &v, 16);
        int kbest = 0;
#pragma unroll
        for (int k = EPV - 1; k >= 0; --k)
            if (apply_map<T>(f, e[k]) == bestv) kbest = k;
        best.i = head + best_vec * EPV + (u64)kbest;
    }
    auto see = [&](T x, u64 i) {
        Best<T> c;
        c.v = apply_map<T>(f, x);
        c.i = i;
        if (better<T, GREATER>(c, best)) best = c;
    };
    if (blockIdx.x == 0) {
        if (tid < head) see(src[tid], tid);
        const u64 t = tail_start + tid;
        if (t < n) see(src[t], t);
    }
    best = block_best<T, GREATER, THREADS>(best, sv, si);
    if (tid == 0) {
        pv[blockIdx.x] = best.v;
        pi[blockIdx.x] = best.i;
        __threadfence();
        const u32 done = atomicAdd(&header[kTicketBase], 1u);
        is_last = (done == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    Best<T> r;
    r.v = T();
    r.i = ~0ull;
    for (u32 b = tid; b < gridDim.x; b += THREADS) {
        Best<T> c;
        c.v = *((const volatile T *)(pv + b));
        c.i = *((const volatile u64 *)(pi + b));
        if (better<T, GREATER>(c, r)) r = c;
    }
    r = block_best<T, GREATER, THREADS>(r, sv, si);
    if (tid == 0) {
        out_index[0] = r.i;
        if (out_value) out_value[0] = r.v;
    }
}

// ---- findfirst / findlast ---------------------------------------------------------------------------
enum { kPredGt = 0, kPredLt = 1, kPredGe = 2, kPredLe = 3, kPredEq = 4, kPredNe = 5 };
template <typename T> __device__ __forceinline__ bool pred_holds(int pred, T x, T y) {
    switch (pred) {
    case kPredGt: return x > y;
    case kPredLt: return x < y;
    case kPredGe: return x >= y;
    case kPredLe: return x <= y;
    case kPredEq: return x == y;
    default: return x != y;
    }
}
// result[0]: first -> smallest matching index (starts at ~0), last -> largest matching index + 1
// (starts at 0). CTAs walk chunks of THREADS * UNROLL 16-byte vectors in search order. Every thread
// carries a copy of result[0] that it refreshes once per chunk, one chunk ahead (the load travels
// with the data loads, nobody waits for it and there is no barrier): a thread stops as soon as that
// copy shows a match that precedes all of its remaining chunks. A stale copy only delays the stop.
template <typename T, int THREADS, int UNROLL>
__global__ void __launch_bounds__(THREADS) find_kernel(const T *__restrict__ src, u64 n, int pred, T operand, int last, u64 *result) {
    constexpr int EPV = 16 / sizeof(T);
    constexpr u64 CHUNK = (u64)THREADS * UNROLL;  // vectors
    const u32 tid = threadIdx.x;
    const u64 mis = ((uintptr_t)src & 15u) / sizeof(T);
    u64 head = mis ? (EPV - mis) : 0;
    if (head > n) head = n;
    const u64 nvec = (n - head) / EPV;
    const u64 tail_start = head + nvec * EPV;
    const uint4 *vsrc = reinterpret_cast<const uint4 *>(src + head);
    const u64 none = last ? 0 : ~0ull;
    auto publish = [&](u64 mine) {  // one atomic per warp that found something
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            const u64 o = shfl_down(mine, d);
            mine = last ? (o > mine ? o : mine) : (o < mine ? o : mine);
        }
        if (lane_id() == 0 && mine != none) {
            if (last) atomicMax((unsigned long long *)result, (unsigned long long)mine);
            else atomicMin((unsigned long long *)result, (unsigned long long)mine);
        }
    };
    if (blockIdx.x == 0) {  // the scalar head and tail (fewer than EPV elements each)
        u64 mine = none;
        const u64 t = tail_start + tid;
        if (t < n && pred_holds<T>(pred, src[t], operand)) mine = last ? t + 1 : t;
        if (tid < head && pred_holds<T>(pred, src[tid], operand)) mine = (last && mine != none) ? mine : (last ? tid + 1 : tid);
        publish(mine);
    }
    const u64 nchunks = (nvec + CHUNK - 1) / CHUNK;
    u64 seen = ld_relaxed_u64(result);
    for (u64 c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const u64 chunk = last ? nchunks - 1 - c : c;
        const u64 v0 = chunk * CHUNK;
        const u64 e_lo = head + v0 * EPV, e_hi = head + (v0 + CHUNK) * EPV;  // element range of the chunk (e_hi may pass the end)
        if (last ? (seen > e_hi) : (seen < e_lo)) return;  // a match beyond this chunk (in search order) exists
        const u64 seen_next = ld_relaxed_u64(result);
        uint4 v[UNROLL];
        bool ok[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const u64 idx = v0 + (u64)u * THREADS + tid;
            ok[u] = idx < nvec;
            if (ok[u]) v[u] = ld_stream_v4(vsrc + idx);
        }
        u64 mine = none;
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (ok[u]) {
                T e[EPV];
                memcpy(e, &v[u], 16);
                u32 hits = 0;
#pragma unroll
                for (int k = 0; k < EPV; ++k) hits |= pred_holds<T>(pred, e[k], operand) ? (1u << k) : 0u;
                if (hits) {
                    const u64 i0 = head + (v0 + (u64)u * THREADS + tid) * EPV;
                    if (last) {
                        const u64 cand = i0 + (31 - __clz(hits)) + 1;
                        mine = cand > mine ? cand : mine;
                    } else {
                        const u64 cand = i0 + (__ffs(hits) - 1);
                        mine = cand < mine ? cand : mine;
                    }
                }
            }
        }
        if (__any_sync(0xFFFFFFFFu, mine != none)) publish(mine);
        seen = seen_next;
    }
}

// ---- copy / fill -----------------------------------------------------------------------------------
template <int THREADS, int UNROLL>
__global__ void __launch_bounds__(THREADS) vcopy_kernel(const unsigned char *__restrict__ src, unsigned char *dst, u64 nbytes, u64 head) {
    // [0, head) bytes, then whole 16-byte vectors (both arrays aligned there), then the tail bytes
    const u64 nvec = (nbytes - head) / 16;
    const uint4 *vs = reinterpret_cast<const uint4 *>(src + head);
    uint4 *vd = reinterpret_cast<uint4 *>(dst + head);
    constexpr u64 STRIP = (u64)THREADS * UNROLL;
    const u64 stride = (u64)gridDim.x * STRIP;
    for (u64 base = (u64)blockIdx.x * STRIP; base < nvec; base += stride) {
        uint4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const u64 i = base + (u64)u * THREADS + threadIdx.x;
            if (i < nvec) v[u] = ld_stream_v4(vs + i);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const u64 i = base + (u64)u * THREADS + threadIdx.x;
            if (i < nvec) st_stream_v4(vd + i, v[u]);
        }
    }
    if (blockIdx.x == 0) {
        if (threadIdx.x < head) dst[threadIdx.x] = src[threadIdx.x];
        const u64 t = head + nvec * 16 + threadIdx.x;
        if (threadIdx.x < 16 && t < nbytes) dst[t] = src[t];
    }
}
// Arrays that do not share their 16-byte misalignment: element-wise (bytes).
__global__ void bcopy_kernel(const unsigned char *__restrict__ src, unsigned char *dst, u64 nbytes) {
    const u64 stride = (u64)gridDim.x * blockDim.x;
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < nbytes; i += stride) dst[i] = src[i];
}
// dst = repeated 16-byte pattern (the value replicated; element sizes divide 16). `phase` is the
// byte offset of dst[0] inside the pattern.
template <int THREADS>
__global__ void __launch_bounds__(THREADS) fill_kernel(unsigned char *dst, u64 nbytes, u64 head, uint4 pattern) {
    const u64 nvec = (nbytes - head) / 16;
    uint4 *vd = reinterpret_cast<uint4 *>(dst + head);
    const u64 stride = (u64)gridDim.x * THREADS;
    for (u64 i = (u64)blockIdx.x * THREADS + threadIdx.x; i < nvec; i += stride) vd[i] = pattern;
    if (blockIdx.x == 0) {
        // head and tail bytes: byte k of the array is byte (k - head) mod 16 of the pattern
        unsigned char pb[16];
        memcpy(pb, &pattern, 16);
        if (threadIdx.x < head) dst[threadIdx.x] = pb[(16 + threadIdx.x - head) & 15];
        const u64 t = head + nvec * 16 + threadIdx.x;
        if (threadIdx.x < 16 && t < nbytes) dst[t] = pb[threadIdx.x];
    }
}

static int stream_grid(u64 nbytes, int threads, int unroll) {
    const u64 strip = (u64)threads * unroll * 16;
    u64 need = (nbytes + strip - 1) / strip;
    const u64 cap = (u64)device_sm_count() * 8;
    if (need > cap) need = cap;
    return (int)(need < 1 ? 1 : need);
}

template <typename T>
static int launch_argmax(bool greater, int blocks, const void *src, u64 n, void *ov, u64 *oi, void *pv, u64 *pi, u32 *header, int f,
                         cudaStream_t s) {
    // 8 loads in flight per thread: 6270 GB/s at n = 2^28 Float32, against 5560 with 4
    if (greater) argmax_kernel<T, true, 256, 8><<<blocks, 256, 0, s>>>((const T *)src, n, (T *)ov, oi, (T *)pv, pi, header, f);
    else argmax_kernel<T, false, 256, 8><<<blocks, 256, 0, s>>>((const T *)src, n, (T *)ov, oi, (T *)pv, pi, header, f);
    note_launch();
    KF_CUDA_TRY(cudaGetLastError());
    return KF_OK;
}

template <typename T>
static int launch_find(const void *src, u64 n, int pred, const void *operand, int last, u64 *result, cudaStream_t s) {
    T y;
    memcpy(&y, operand, sizeof(T));
    // 8 loads in flight per thread and 16 CTAs per SM: 6590 GB/s for a predicate nothing satisfies at
    // n = 2^28 Float32 (4 loads, 8 CTAs: 5550)
    constexpr int THREADS = 256, UNROLL = 8;
    const u64 chunk_bytes = (u64)THREADS * UNROLL * 16;
    u64 nchunks = (n * sizeof(T) + chunk_bytes - 1) / chunk_bytes;
    if (nchunks < 1) nchunks = 1;
    u64 blocks = (u64)device_sm_count() * 16;
    if (blocks > nchunks) blocks = nchunks;
    find_kernel<T, THREADS, UNROLL><<<(unsigned)blocks, THREADS, 0, s>>>((const T *)src, n, pred, y, last, result); note_launch();
    KF_CUDA_TRY(cudaGetLastError());
    return KF_OK;
}

}  // namespace kf

using namespace kf;

static size_t argmax_blocks(uint64_t n, int eb) { return (size_t)stream_grid(n * (uint64_t)eb, 256, 8); }

extern "C" size_t kf_argmax_workspace_bytes(int32_t dtype, uint64_t n) {
    const int eb = dtype_bytes(dtype);
    if (eb == 0) return 0;
    const size_t b = argmax_blocks(n, eb);
    return kHeaderBytes + align_up(b * 8, 256) + align_up(b * 8, 256);
}

extern "C" int32_t kf_argmax(int32_t f, int32_t greater, int32_t dtype, const void *src, uint64_t n, void *out_value,
                             uint64_t *out_index, void *ws, size_t ws_bytes, kf_stream_t stream) {
    if (n == 0) return KF_ERR_EMPTY_REDUCTION;
    if (!src || !out_index || !ws) return KF_ERR_INVALID_ARG;
    if (f < KF_MAP_IDENTITY || f > KF_MAP_ABS) return KF_ERR_UNSUPPORTED;
    const int eb = dtype_bytes(dtype);
    if (eb == 0) return KF_ERR_INVALID_ARG;
    if (((uintptr_t)src % eb) || ((uintptr_t)ws % 256) || ((uintptr_t)out_index % 8) || (out_value && ((uintptr_t)out_value % eb)))
        return KF_ERR_INVALID_ARG;
    if (ws_bytes < kf_argmax_workspace_bytes(dtype, n)) return KF_ERR_WORKSPACE_TOO_SMALL;
    const int blocks = (int)argmax_blocks(n, eb);
    cudaStream_t s = (cudaStream_t)stream;
    u32 *header = (u32 *)ws;
    void *pv = (char *)ws + kHeaderBytes;
    u64 *pi = (u64 *)((char *)pv + align_up((size_t)blocks * 8, 256));
    KF_CUDA_TRY(cudaMemsetAsync(header, 0, kHeaderBytes, s));
    const bool g = greater != 0;
    switch (dtype) {
    case KF_U8: return launch_argmax<uint8_t>(g, blocks, src, n, out_value, (u64 *)out_index, pv, pi, header, f, s);
    case KF_I8: return launch_argmax<int8_t>(g, blocks, src, n, out_value, (u64 *)out_index, pv, pi, header, f, s);
    case KF_U16: return launch_argmax<uint16_t>(g, blocks, src, n, out_value, (u64 *)out_index, pv, pi, header, f, s);
    case KF_I16: return launch_argmax<int16_t>(g, blocks, src, n, out_value, (u64 *)out_index, pv, pi, header, f, s);
    case KF_U32: return launch_argmax<uint32_t>(g, blocks, src, n, out_value, (u64 *)out_index, pv, pi, header, f, s);
    case KF_I32: return launch_argmax<int32_t>(g, blocks, src, n, out_value, (u64 *)out_index, pv, pi, header, f, s);
    case KF_U64: return launch_argmax<u64>(g, blocks, src, n, out_value, (u64 *)out_index, pv, pi, header, f, s);
    case KF_I64: return launch_argmax<long long>(g, blocks, src, n, out_value, (u64 *)out_index, pv, pi, header, f, s);
    case KF_F32: return launch_argmax<float>(g, blocks, src, n, out_value, (u64 *)out_index, pv, pi, header, f, s);
    case KF_F64: return launch_argmax<double>(g, blocks, src, n, out_value, (u64 *)out_index, pv, pi, header, f, s);
    default: return KF_ERR_INVALID_ARG;
    }
}

extern "C" int32_t kf_find(int32_t pred, int32_t last, int32_t dtype, const void *src, uint64_t n, const void *operand,
                           uint64_t *out_index, kf_stream_t stream) {
    if (!out_index || !operand || (n && !src)) return KF_ERR_INVALID_ARG;
    if (pred < kPredGt || pred > kPredNe) return KF_ERR_UNSUPPORTED;
    const int eb = dtype_bytes(dtype);
    if (eb == 0 || ((uintptr_t)src % eb) || ((uintptr_t)out_index % 8)) return KF_ERR_INVALID_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    KF_CUDA_TRY(cudaMemsetAsync(out_index, last ? 0x00 : 0xFF, 8, s));
    if (n == 0) return KF_OK;
    switch (dtype) {
    case KF_U8: return launch_find<uint8_t>(src, n, pred, operand, last, (u64 *)out_index, s);
    case KF_I8: return launch_find<int8_t>(src, n, pred, operand, last, (u64 *)out_index, s);
    case KF_U16: return launch_find<uint16_t>(src, n, pred, operand, last, (u64 *)out_index, s);
    case KF_I16: return launch_find<int16_t>(src, n, pred, operand, last, (u64 *)out_index, s);
    case KF_U32: return launch_find<uint32_t>(src, n, pred, operand, last, (u64 *)out_index, s);
    case KF_I32: return launch_find<int32_t>(src, n, pred, operand, last, (u64 *)out_index, s);
    case KF_U64: return launch_find<u64>(src, n, pred, operand, last, (u64 *)out_index, s);
    case KF_I64: return launch_find<long long>(src, n, pred, operand, last, (u64 *)out_index, s);
    case KF_F32: return launch_find<float>(src, n, pred, operand, last, (u64 *)out_index, s);
    case KF_F64: return launch_find<double>(src, n, pred, operand, last, (u64 *)out_index, s);
    default: return KF_ERR_INVALID_ARG;
    }
}

extern "C" int32_t kf_vcopy(void *dst, const void *src, uint64_t nbytes, kf_stream_t stream) {
    if (nbytes == 0) return KF_OK;
    if (!dst || !src) return KF_ERR_INVALID_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const uintptr_t ms = (uintptr_t)src & 15u, md = (uintptr_t)dst & 15u;
    if (ms == md) {
        u64 head = ms ? 16 - ms : 0;
        if (head > nbytes) head = nbytes;
        // One strip of 256 x 4 vectors per CTA and as many CTAs as that takes, not a persistent grid:
        // 6890 GB/s at 1 GiB (a persistent grid of 8 CTAs per SM: 5850; torch's copy_: 6530).
        const u64 strips = (nbytes / 16 + 1023) / 1024;
        if (strips >= (1ull << 31)) return KF_ERR_INVALID_ARG;
        vcopy_kernel<256, 4><<<(unsigned)(strips < 1 ? 1 : strips), 256, 0, s>>>((const unsigned char *)src, (unsigned char *)dst, nbytes, head);
        note_launch();
    } else {
        bcopy_kernel<<<device_sm_count() * 8, 256, 0, s>>>((const unsigned char *)src, (unsigned char *)dst, nbytes); note_launch();
    }
    KF_CUDA_TRY(cudaGetLastError());
    return KF_OK;
}

extern "C" int32_t kf_setvalue(int32_t dtype, void *dst, uint64_t n, const void *value, kf_stream_t stream) {
    const int eb = dtype_bytes(dtype);
    if (eb == 0) return KF_ERR_INVALID_ARG;
    if (n == 0) return KF_OK;
    if (!dst || !value || ((uintptr_t)dst % eb)) return KF_ERR_INVALID_ARG;
    unsigned char pb[16];
    for (int k = 0; k < 16; k += eb) memcpy(pb + k, value, eb);
    uint4 pattern;
    memcpy(&pattern, pb, 16);
    const u64 nbytes = n * (u64)eb;
    const uintptr_t md = (uintptr_t)dst & 15u;
    u64 head = md ? 16 - md : 0;  // a multiple of the element size, so the pattern stays in phase
    if (head > nbytes) head = nbytes;
    // Four plain 128-bit stores per thread and as many CTAs as that takes: 7340 GB/s at 1 GiB (a
    // persistent grid with evict-first stores: 5930; torch's fill_: 7410).
    const u64 strips = (nbytes / 16 + 1023) / 1024;
    if (strips >= (1ull << 31)) return KF_ERR_INVALID_ARG;
    fill_kernel<256><<<(unsigned)(strips < 1 ? 1 : strips), 256, 0, (cudaStream_t)stream>>>((unsigned char *)dst, nbytes, head, pattern);
    note_launch();
    KF_CUDA_TRY(cudaGetLastError());
    return KF_OK;
}
