// Host side of the scan kernels: the compiled (threads, vectors) variants, the choice between the
// direct kernel and the persistent ring kernel, and the per-type dispatch that each
// scan_inst_*.cu instantiates.
#pragma once

#include "scan_roles.cuh"

namespace kf {

// `vecs` is 16-byte vectors per thread per tile and per array. The persistent (`ring`) variants
// read tiles ahead through shared memory with the bulk-copy engine and need 16-byte aligned
// arrays; the direct variants work on anything and serve as their fallback (and as the
// small-input path).
struct ScanVariant {
    int threads, vecs;
    bool ring;
};
static const ScanVariant kScanVariants[] = {
    {256, 4, false}, {512, 4, false}, {256, 8, false}, {128, 8, false},  // direct
    {768, 4, true},                                                      // persistent: 2 buffers, reduction 3 tiles ahead
    {384, 8, true},                                                      // persistent: 2 buffers, reduction 3 tiles ahead; fewest warps, holds its rate under the power cap
    {512, 8, true},                                                      // persistent: 2 buffers, reduction 3 tiles ahead (best for 2- and 8-byte elements)
};
constexpr int kNumScanVariants = 7;
constexpr int kScanFallbackVariant = 1;  // direct 512x4: what a ring variant falls back to

struct ScanPlan {
    int variant;
    u64 tile;     // elements per tile
    u64 ntiles;   // upper bound used for sizing (includes a possible head tile)
    int words;    // descriptor words per tile
};

// Elements per tile of a variant. Ring tiles of two-array layouts use half the vectors per thread,
// so that a ring buffer stays the same size.
inline u64 scan_tile_elems(int variant, int epv, int narr) {
    const ScanVariant &v = kScanVariants[variant];
    const int vecs = v.ring ? v.vecs / narr : v.vecs;
    return (u64)v.threads * vecs * epv;
}

int scan_plan(int elem_bytes, int epv, int narr, u64 n, const kf_launch_cfg *cfg, ScanPlan *plan);

template <typename T, typename Op, typename Access, typename Arrays, int THREADS, int VECS, int NBUF, int K, int LAG, bool PACKED = false>
int scan_launch_ring_one(const Access &acc, const Arrays &arr, const ScanArgs &args, cudaStream_t s) {
    constexpr int DEPTH = 8, NRES = 1;  // one resolver warp, 256 descriptors per round trip
    using SM = ScanRolesSmem<Arrays, T, THREADS, VECS, NBUF, K>;
    static_assert(SM::kBytes <= 227 * 1024, "ring does not fit in shared memory");
    constexpr int CTA = THREADS + 32 + 32 * NRES;
    // One-byte `+` with no maps takes the packed instantiation of the kernel.
    if constexpr (!PACKED && sizeof(T) == 1 && std::is_same<Op, OpAdd>::value && Arrays::NARR == 1) {
        if (args.f == KF_MAP_IDENTITY && args.g == KF_POST_IDENTITY)
            return scan_launch_ring_one<T, Op, Access, Arrays, THREADS, VECS, NBUF, K, LAG, true>(acc, arr, args, s);
    }
    auto kern = scan_kernel_roles<T, Op, Access, Arrays, THREADS, VECS, NBUF, K, DEPTH, NRES, LAG, PACKED>;
    KF_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SM::kBytes));
    // One CTA per SM: the look-ahead distance K is tuned for tiles of that size arriving at that rate.
    u64 grid = (u64)device_sm_count();
    if (grid > args.ntiles) grid = args.ntiles;
    kern<<<(unsigned)grid, CTA, SM::kBytes, s>>>(acc, arr, args); note_launch();
    KF_CUDA_TRY(cudaGetLastError());
    return KF_OK;
}

template <typename T, typename Op, typename Access, typename Arrays>
int scan_launch(int variant, const Access &acc, const Arrays &arr, const ScanArgs &args, cudaStream_t s) {
    const unsigned grid = (unsigned)args.ntiles;
    constexpr int RV = 4 / Arrays::NARR;   // ring vectors per thread and array
    constexpr int RV8 = 8 / Arrays::NARR;
    switch (variant) {
    case 0: scan_kernel<T, Op, Access, 256, 4><<<grid, 256, 0, s>>>(acc, args); note_launch(); break;
    case 1: scan_kernel<T, Op, Access, 512, 4><<<grid, 512, 0, s>>>(acc, args); note_launch(); break;
    case 2: scan_kernel<T, Op, Access, 256, 8><<<grid, 256, 0, s>>>(acc, args); note_launch(); break;
    case 3: scan_kernel<T, Op, Access, 128, 8><<<grid, 128, 0, s>>>(acc, args); note_launch(); break;
    case 4: return scan_launch_ring_one<T, Op, Access, Arrays, 768, RV, 2, 3, 2>(acc, arr, args, s);
    case 5: return scan_launch_ring_one<T, Op, Access, Arrays, 384, RV8, 2, 3, 2>(acc, arr, args, s);
    // 8-byte elements and affine pairs (64 KB tiles) read 1.25 x their input from DRAM in this variant:
    // three tiles per SM between reduction and scan, plus the output written in between, overflow what
    // L2 keeps. Both cures were measured and are slower: reducing two tiles ahead (reads back to 1.05 x,
    // but the descriptor latency shows) and 48 KB tiles (512 x 6 vectors).
    case 6: return scan_launch_ring_one<T, Op, Access, Arrays, 512, RV8, 2, 3, 2>(acc, arr, args, s);
    default: return KF_ERR_UNSUPPORTED;
    }
    KF_CUDA_TRY(cudaGetLastError());
    return KF_OK;
}

// One translation unit per element type instantiates this (keeps the build parallel).
template <typename T>
int scan_dispatch_ops(int op, int variant, const T *src, T *dst, const ScanArgs &args, cudaStream_t s) {
    PlainAccess<T> acc{src, dst};
    PlainArrays<T> arr;
    arr.src[0] = reinterpret_cast<const char *>(src);
    arr.dst[0] = reinterpret_cast<char *>(dst);
    switch (op) {
    case KF_OP_ADD: return scan_launch<T, OpAdd>(variant, acc, arr, args, s);
    case KF_OP_MUL: return scan_launch<T, OpMul>(variant, acc, arr, args, s);
    case KF_OP_MIN: return scan_launch<T, OpMin>(variant, acc, arr, args, s);
    case KF_OP_MAX: return scan_launch<T, OpMax>(variant, acc, arr, args, s);
    default: break;
    }
    if constexpr (!IsFloat<T>::value) {
        switch (op) {
        case KF_OP_AND: return scan_launch<T, OpAnd>(variant, acc, arr, args, s);
        case KF_OP_OR: return scan_launch<T, OpOr>(variant, acc, arr, args, s);
        case KF_OP_XOR: return scan_launch<T, OpXor>(variant, acc, arr, args, s);
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
        return scan_dispatch_ops<T>(op, variant, (const T *)src, (T *)dst, args, s);                     \
    }                                                                                                    \
    }

}  // namespace kf
