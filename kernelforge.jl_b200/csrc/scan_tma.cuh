// Bulk-copy (TMA, cp.async.bulk) and mbarrier helpers for sm_100a, and the array views that the
// persistent scan kernel (scan_roles.cuh) stages through shared memory with them.
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

}  // namespace kf
