// Inclusive scan of quaternions under the Hamilton product (C ABI): the non-commutative operator of
// the reference's own scan test (test/tests/scan/scan_test.jl:22-33 of KernelForge.jl, where a
// QuaternionF64 array takes the split kernel, src/scan/scan_kernel.jl:94-299). Elements are 16 bytes
// (Float32 components) or 32 bytes (Float64), so a tile descriptor is four or eight self-validating
// words; the direct decoupled look-back kernel of scan_impl.cuh does the rest.
#include "scan_impl.cuh"

namespace kf {

constexpr int kQuatThreads = 256, kQuatPerThread = 4;  // as kQuatPerThread / EPV slots of EPV quaternions
constexpr u64 kQuatTile = (u64)kQuatThreads * kQuatPerThread;

static size_t quat_ws_bytes(int comp_bytes, u64 n, u64 *ntiles) {
    *ntiles = (n + kQuatTile - 1) / kQuatTile;
    return kHeaderBytes + align_up((size_t)*ntiles * comp_bytes * 8, 256);  // 4 * comp_bytes / 4 words of 8 bytes per tile
}

template <typename F>
static int quat_launch(const void *src, void *dst, const ScanArgs &a, cudaStream_t s) {
    using Q = Quat<F>;
    QuatAccess<F> acc{static_cast<const Q *>(src), static_cast<Q *>(dst)};
    scan_kernel<Q, OpQuatMul, QuatAccess<F>, kQuatThreads, kQuatPerThread / QuatAccess<F>::EPV><<<(unsigned)a.ntiles, kQuatThreads, 0, s>>>(acc, a);
    note_launch();
    KF_CUDA_TRY(cudaGetLastError());
    return KF_OK;
}

}  // namespace kf

using namespace kf;

extern "C" size_t kf_scan_quaternion_workspace_bytes(int32_t dtype, uint64_t n) {
    if (dtype != KF_F32 && dtype != KF_F64) return 0;
    u64 ntiles;
    const size_t b = quat_ws_bytes(dtype == KF_F32 ? 4 : 8, n, &ntiles);
    return ntiles < (1ull << 31) ? b : 0;
}

extern "C" int32_t kf_scan_quaternion(int32_t dtype, const void *src, void *dst, uint64_t n, const void *init,
                                      uint32_t ninit, void *ws, size_t ws_bytes, const kf_launch_cfg *cfg,
                                      kf_stream_t stream) {
    if (dtype != KF_F32 && dtype != KF_F64) return dtype_bytes(dtype) ? KF_ERR_UNSUPPORTED : KF_ERR_INVALID_ARG;
    const int cb = dtype == KF_F32 ? 4 : 8;
    if (n == 0) return KF_OK;
    if (!src || !dst || !ws) return KF_ERR_INVALID_ARG;
    if (((uintptr_t)src % cb) || ((uintptr_t)dst % cb) || ((uintptr_t)ws % 256) || (init && ((uintptr_t)init % cb)))
        return KF_ERR_INVALID_ARG;
    u64 ntiles;
    const size_t need = quat_ws_bytes(cb, n, &ntiles);
    if (ntiles >= (1ull << 31)) return KF_ERR_INVALID_ARG;
    if (ws_bytes < need) return KF_ERR_WORKSPACE_TOO_SMALL;

    ScanArgs a;
    a.n = n;
    a.head = 0;
    a.ntiles = ntiles;
    a.header = (u32 *)ws;
    a.desc = (u64 *)((char *)ws + kHeaderBytes);
    a.init = ninit ? init : nullptr;
    a.ninit = init ? ninit : 0;
    a.vec_ok = ((((uintptr_t)src | (uintptr_t)dst) & 15u) == 0) ? 1 : 0;  // else: component-wise accesses
    a.f = KF_MAP_IDENTITY;
    a.g = KF_POST_IDENTITY;
    a.spin_limit = test_spin_limit(cfg);
    a.mute_tile = test_mute_tile(cfg);
    cudaStream_t s = (cudaStream_t)stream;
    KF_CUDA_TRY(cudaMemsetAsync(ws, 0, need, s));
    return dtype == KF_F32 ? quat_launch<float>(src, dst, a, s) : quat_launch<double>(src, dst, a, s);
}
