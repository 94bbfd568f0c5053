// Shared device/host helpers for the sm_100a kernels: element operators, 128-bit streaming
// loads/stores, relaxed 64-bit descriptor accesses, bounded waits and the workspace header.
#pragma once

#include <cuda_runtime.h>
#include <cstdio>
#include <stdint.h>
#include <stddef.h>

#include "../../include/kf_b200.h"

namespace kf {

typedef unsigned long long u64;
typedef unsigned int u32;

// ---------------------------------------------------------------------------------------------
// Workspace header. Every workspace starts with this 256-byte block; the callee clears it (and
// the descriptors behind it) with one memset at the start of a call.
//   word 0      : device status (0 = OK, else a kf_status a kernel recorded)
//   word 1      : where a wait gave up (tile index), for diagnostics
//   words 8..23 : tile tickets / completion counters (one per kernel launch of the call)
// ---------------------------------------------------------------------------------------------
constexpr size_t kHeaderBytes = 256;
constexpr int kStatusWord = 0;
constexpr int kStatusAux = 1;
constexpr int kTicketBase = 8;

// Polls before a waiting tile gives up. Each poll is an L2 round trip (~1 us with back-off), so
// the limit is on the order of a second; a healthy look-back needs a handful of polls.
constexpr u32 kSpinLimit = 1u << 20;

// kf_launch_cfg.reserved is 0 in production. Tests use it to make a bounded wait run out without
// faulting anything: bits 0..15 = polls before a wait gives up (0 = kSpinLimit), bits 16..31 = 1 + the
// index of one tile that stays silent (publishes no descriptor and writes no output).
inline u32 test_spin_limit(const kf_launch_cfg *cfg) {
    const u32 v = cfg ? ((u32)cfg->reserved & 0xFFFFu) : 0u;
    return v ? v : kSpinLimit;
}
inline u32 test_mute_tile(const kf_launch_cfg *cfg) { return cfg ? ((u32)cfg->reserved >> 16) : 0u; }

__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Programmatic dependent launch (sm_90+): a kernel launched with the programmatic-serialization
// attribute may be scheduled while its predecessor in the stream is still draining. grid_dep_wait()
// returns once the predecessor has completed and its writes are visible; grid_dep_launch() tells the
// scheduler that, as far as this CTA is concerned, the successor's CTAs may be brought onto the SMs.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Host side of the same: launches `kern` so that it may become resident while the kernel before it in
// the stream drains. The kernel must call grid_dep_wait() before it touches anything that kernel wrote.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kern)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t s, Args &&...args) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(grid);
    lc.blockDim = dim3(block);
    lc.dynamicSmemBytes = smem;
    lc.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    return cudaLaunchKernelEx(&lc, kern, static_cast<KArgs>(args)...);
}

// ---------------------------------------------------------------------------------------------
// Raw memory access
// ---------------------------------------------------------------------------------------------

// 128-bit read-only streaming load: bypasses L1 allocation (data is used once).
__device__ __forceinline__ uint4 ld_stream_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// Coherent 128-bit streaming load (used when dst may alias src, where the non-coherent path is
// not allowed); still skips L1 allocation.
__device__ __forceinline__ uint4 ld_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}
// 128-bit streaming store (evict-first: written once, not read again by this kernel).
__device__ __forceinline__ void st_stream_v4(void *p, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// Relaxed, device-scope 64-bit accesses for tile descriptors. A descriptor carries its own
// status in the same word as the value, so no fence is needed to pair them.
__device__ __forceinline__ u64 ld_relaxed_u64(const u64 *p) {
    u64 v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_u64(u64 *p, u64 v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ u32 ld_relaxed_u32(const u32 *p) {
    u32 v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ u32 ld_acquire_u32(const u32 *p) {
    u32 v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ u32 lane_id() {
    u32 l;
    asm("mov.u32 %0, %%laneid;" : "=r"(l));
    return l;
}
__device__ __forceinline__ u32 lanemask_lt() {
    u32 m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// Records a device-side error once (first writer wins) in the workspace header.
__device__ __forceinline__ void record_error(u32 *header, int code, u32 where) {
    if (atomicCAS(&header[kStatusWord], 0u, (u32)code) == 0u) header[kStatusAux] = where;
}

// ---------------------------------------------------------------------------------------------
// Element operators. `apply(l, r)` combines an EARLIER value `l` with a LATER value `r`.
// ---------------------------------------------------------------------------------------------
template <typename T> struct Limits;
template <> struct Limits<uint8_t> { static __host__ __device__ uint8_t lo() { return 0; } static __host__ __device__ uint8_t hi() { return 0xFF; } };
template <> struct Limits<int8_t> { static __host__ __device__ int8_t lo() { return -128; } static __host__ __device__ int8_t hi() { return 127; } };
template <> struct Limits<uint16_t> { static __host__ __device__ uint16_t lo() { return 0; } static __host__ __device__ uint16_t hi() { return 0xFFFF; } };
template <> struct Limits<int16_t> { static __host__ __device__ int16_t lo() { return -32768; } static __host__ __device__ int16_t hi() { return 32767; } };
template <> struct Limits<uint32_t> { static __host__ __device__ uint32_t lo() { return 0; } static __host__ __device__ uint32_t hi() { return 0xFFFFFFFFu; } };
template <> struct Limits<int32_t> { static __host__ __device__ int32_t lo() { return INT32_MIN; } static __host__ __device__ int32_t hi() { return INT32_MAX; } };
template <> struct Limits<u64> { static __host__ __device__ u64 lo() { return 0; } static __host__ __device__ u64 hi() { return ~0ull; } };
template <> struct Limits<long long> { static __host__ __device__ long long lo() { return INT64_MIN; } static __host__ __device__ long long hi() { return INT64_MAX; } };
template <> struct Limits<float> {
    static __host__ __device__ float lo() { return -__builtin_huge_valf(); }
    static __host__ __device__ float hi() { return __builtin_huge_valf(); }
};
template <> struct Limits<double> {
    static __host__ __device__ double lo() { return -__builtin_huge_val(); }
    static __host__ __device__ double hi() { return __builtin_huge_val(); }
};

template <typename T> struct IsFloat { static constexpr bool value = false; };
template <> struct IsFloat<float> { static constexpr bool value = true; };
template <> struct IsFloat<double> { static constexpr bool value = true; };

struct OpAdd {
    static constexpr bool commutative = true;
    template <typename T> static __device__ __forceinline__ T apply(T l, T r) { return (T)(l + r); }
    // -0.0 is the exact additive identity of IEEE floats (+0.0 would turn a leading -0.0 into +0.0).
    template <typename T> static __device__ __forceinline__ T identity() {
        if constexpr (IsFloat<T>::value) return (T)-0.0;
        else return (T)0;
    }
};
struct OpMul {
    static constexpr bool commutative = true;
    template <typename T> static __device__ __forceinline__ T apply(T l, T r) { return (T)(l * r); }
    template <typename T> static __device__ __forceinline__ T identity() { return (T)1; }
};
struct OpMin {
    static constexpr bool commutative = true;
    template <typename T> static __device__ __forceinline__ T apply(T l, T r) { return r < l ? r : l; }
    template <typename T> static __device__ __forceinline__ T identity() { return Limits<T>::hi(); }
};
struct OpMax {
    static constexpr bool commutative = true;
    template <typename T> static __device__ __forceinline__ T apply(T l, T r) { return l < r ? r : l; }
    template <typename T> static __device__ __forceinline__ T identity() { return Limits<T>::lo(); }
};
struct OpAnd {
    static constexpr bool commutative = true;
    template <typename T> static __device__ __forceinline__ T apply(T l, T r) { return (T)(l & r); }
    template <typename T> static __device__ __forceinline__ T identity() { return (T)~(T)0; }
};
struct OpOr {
    static constexpr bool commutative = true;
    template <typename T> static __device__ __forceinline__ T apply(T l, T r) { return (T)(l | r); }
    template <typename T> static __device__ __forceinline__ T identity() { return (T)0; }
};
struct OpXor {
    static constexpr bool commutative = true;
    template <typename T> static __device__ __forceinline__ T apply(T l, T r) { return (T)(l ^ r); }
    template <typename T> static __device__ __forceinline__ T identity() { return (T)0; }
};

// An affine map x -> a*x + b. Composition applies the left map first:
// (a1,b1) o (a2,b2) = (a1*a2, a2*b1 + b2). The b component is one fused multiply-add (a single
// rounding), which is at least as close to the Float64 left fold as separate mul and add.
struct Affine {
    float a, b;
};
struct OpAffine {
    static constexpr bool commutative = false;
    template <typename T> static __device__ __forceinline__ T apply(T l, T r) {
        T o;
        o.a = l.a * r.a;
        o.b = fmaf(r.a, l.b, r.b);
        return o;
    }
    template <typename T> static __device__ __forceinline__ T identity() {
        T o;
        o.a = 1.0f;
        o.b = -0.0f;
        return o;
    }
};

// Quaternion w + xi + yj + zk stored as four consecutive scalars (the layout of Quaternions.jl's
// Quaternion{T}: s, v1, v2, v3) and the Hamilton product, the non-commutative operator that the
// reference's scan test uses (test/tests/scan/scan_test.jl:22-33 of KernelForge.jl).
template <typename F> struct Quat {
    F w, x, y, z;
};
struct OpQuatMul {
    static constexpr bool commutative = false;
    template <typename T> static __device__ __forceinline__ T apply(T l, T r) {
        T o;
        o.w = l.w * r.w - l.x * r.x - l.y * r.y - l.z * r.z;
        o.x = l.w * r.x + l.x * r.w + l.y * r.z - l.z * r.y;
        o.y = l.w * r.y - l.x * r.z + l.y * r.w + l.z * r.x;
        o.z = l.w * r.z + l.x * r.y - l.y * r.x + l.z * r.w;
        return o;
    }
    template <typename T> static __device__ __forceinline__ T identity() {
        T o;
        o.w = 1;
        o.x = 0;
        o.y = 0;
        o.z = 0;
        return o;
    }
};

// Element-wise map f, selected at run time (uniform across the grid; the kernels are
// HBM-bound, the branch is free).
template <typename T> __device__ __forceinline__ T apply_map(int f, T x) {
    if (f == KF_MAP_ABS2) return (T)(x * x);
    if (f == KF_MAP_ABS) return x < (T)0 ? (T)(0 - x) : x;  // integers: wraps at the minimum, like Julia
    return x;
}
template <> __device__ __forceinline__ float apply_map<float>(int f, float x) {
    if (f == KF_MAP_ABS2) return x * x;
    if (f == KF_MAP_ABS) return fabsf(x);
    return x;
}
template <> __device__ __forceinline__ double apply_map<double>(int f, double x) {
    if (f == KF_MAP_ABS2) return x * x;
    if (f == KF_MAP_ABS) return fabs(x);
    return x;
}

// Post-map g (kf_post): applied once to the result of a mapreduce, and to every output element of a
// scan (src/scan/scan_kernel.jl:463,470,474 of the reference).
template <typename T> __device__ __forceinline__ T apply_post(int g, T x) {
    if constexpr (IsFloat<T>::value) {
        if (g == KF_POST_SQRT) return sqrt(x);  // IEEE round-to-nearest in the element type, like Julia's sqrt
    }
    return x;
}

// ---------------------------------------------------------------------------------------------
// Warp shuffles for any trivially copyable type of up to 4 bytes or of a multiple of 4 bytes
// (8-byte scalars, the affine pair, quaternions): one 32-bit shuffle per word.
// ---------------------------------------------------------------------------------------------
template <typename T, typename Shuffle> __device__ __forceinline__ T shfl_words(T v, Shuffle sh) {
    if constexpr (sizeof(T) <= 4) {
        u32 x = 0;
        memcpy(&x, &v, sizeof(T));
        x = sh(x);
        T o;
        memcpy(&o, &x, sizeof(T));
        return o;
    } else {
        static_assert(sizeof(T) % 4 == 0, "unsupported shuffle width");
        constexpr int W = sizeof(T) / 4;
        u32 x[W];
        memcpy(x, &v, sizeof(T));
#pragma unroll
        for (int i = 0; i < W; ++i) x[i] = sh(x[i]);
        T o;
        memcpy(&o, x, sizeof(T));
        return o;
    }
}
template <typename T> __device__ __forceinline__ T shfl_up(T v, int d) {
    return shfl_words(v, [d](u32 x) { return __shfl_up_sync(0xFFFFFFFFu, x, d); });
}
template <typename T> __device__ __forceinline__ T shfl_down(T v, int d) {
    return shfl_words(v, [d](u32 x) { return __shfl_down_sync(0xFFFFFFFFu, x, d); });
}
template <typename T> __device__ __forceinline__ T shfl_xor(T v, int m) {
    return shfl_words(v, [m](u32 x) { return __shfl_xor_sync(0xFFFFFFFFu, x, m); });
}
template <typename T> __device__ __forceinline__ T shfl_idx(T v, int src) {
    return shfl_words(v, [src](u32 x) { return __shfl_sync(0xFFFFFFFFu, x, src); });
}

// Inclusive warp scan that keeps operand order (lane i holds x_0 op ... op x_i).
template <typename Op, typename T> __device__ __forceinline__ T warp_scan_inclusive(T v, u32 lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        T up = shfl_up(v, d);
        up = lane >= (u32)d ? up : Op::template identity<T>();
        v = Op::template apply<T>(up, v);
    }
    return v;
}

// Host-side dtype size.
inline int dtype_bytes(int dtype) {
    switch (dtype) {
    case KF_U8: case KF_I8: return 1;
    case KF_U16: case KF_I16: return 2;
    case KF_U32: case KF_I32: case KF_F32: return 4;
    case KF_U64: case KF_I64: case KF_F64: return 8;
    default: return 0;
    }
}

// Host: remembers the CUDA error behind the last KF_ERR_LAUNCH_FAILED of this thread.
void set_last_cuda_error(cudaError_t e);

#define KF_CUDA_TRY(expr)                                   \
    do {                                                    \
        cudaError_t _e = (expr);                            \
        if (_e != cudaSuccess) {                            \
            ::kf::set_last_cuda_error(_e);                  \
            return KF_ERR_LAUNCH_FAILED;                    \
        }                                                   \
    } while (0)

int device_sm_count();

// Counts one kernel launch of this library (process-wide, read by kf_launch_count).
void note_launch();
// KF_LOG=1 in the environment: one line per library call on stderr with the launch geometry that the
// table (or the caller's kf_launch_cfg) chose. Read once per process.
bool log_enabled();
#define KF_LOGF(...)                          \
    do {                                      \
        if (kf::log_enabled()) {              \
            std::fprintf(stderr, "[kf] ");    \
            std::fprintf(stderr, __VA_ARGS__); \
            std::fprintf(stderr, "\n");       \
        }                                     \
    } while (0)

}  // namespace kf
