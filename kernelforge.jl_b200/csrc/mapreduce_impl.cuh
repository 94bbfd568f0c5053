// Warp- and CTA-level reduction pieces shared by the one-array and the multi-array mapreduce kernels.
#pragma once

#include "common.cuh"

#include <type_traits>

namespace kf {

template <typename Op, typename T> __device__ __forceinline__ T warp_reduce(T v) {
    if constexpr (sizeof(T) == 4 && !IsFloat<T>::value) {
        // redux.sync: single-instruction warp reductions for 32-bit integers.
        if constexpr (std::is_same<Op, OpAdd>::value) return (T)__reduce_add_sync(0xFFFFFFFFu, (unsigned)v);
        else if constexpr (std::is_same<Op, OpAnd>::value) return (T)__reduce_and_sync(0xFFFFFFFFu, (unsigned)v);
        else if constexpr (std::is_same<Op, OpOr>::value) return (T)__reduce_or_sync(0xFFFFFFFFu, (unsigned)v);
        else if constexpr (std::is_same<Op, OpXor>::value) return (T)__reduce_xor_sync(0xFFFFFFFFu, (unsigned)v);
        else if constexpr (std::is_same<Op, OpMin>::value) return (T)__reduce_min_sync(0xFFFFFFFFu, v);
        else if constexpr (std::is_same<Op, OpMax>::value) return (T)__reduce_max_sync(0xFFFFFFFFu, v);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = Op::template apply<T>(v, shfl_down(v, d));
    return v;
}

// CTA-wide reduction; the result is valid in thread 0.
template <typename Op, typename T, int THREADS> __device__ __forceinline__ T block_reduce(T v, T *smem) {
    constexpr int WARPS = THREADS / 32;
    const u32 lane = lane_id(), warp = threadIdx.x >> 5;
    v = warp_reduce<Op, T>(v);
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = lane < WARPS ? smem[lane] : Op::template identity<T>();
        v = warp_reduce<Op, T>(v);
    }
    __syncthreads();
    return v;
}

// Resolves the launch variant and the persistent grid size of a mapreduce call (mapreduce.cu).
int mapreduce_resolve(int dtype, u64 n, const kf_launch_cfg *cfg, int *variant, int *blocks);

}  // namespace kf
