// Host entry points of the inclusive scan (C ABI): launch geometry, workspace layout, dtype dispatch.
// The kernels live in scan_impl.cuh and are instantiated per element type in scan_inst_*.cu.
#include "scan_launch.cuh"

#include <mutex>

namespace kf {

int scan_plan(int elem_bytes, int epv, int narr, u64 n, const kf_launch_cfg *cfg, ScanPlan *plan) {
    kf_launch_cfg t;
    kf_launch_table_lookup(KF_PRIM_SCAN, elem_bytes, n, &t);
    if (cfg) {
        if (cfg->threads) t.threads = cfg->threads;
        if (cfg->items) t.items = cfg->items;
    }
    int v = -1;
    for (int i = 0; i < kNumScanVariants; ++i)
        if (kScanVariants[i].threads == t.threads && kScanVariants[i].vecs == t.items) v = i;
    if (v < 0) return KF_ERR_UNSUPPORTED;
    plan->variant = v;
    plan->tile = scan_tile_elems(v, epv, narr);
    // A ring variant may fall back to the direct kernel (smaller tiles) when the arrays turn out to
    // be misaligned: size the descriptors for the smaller of the two tiles. +1: a short head tile.
    u64 sizing_tile = plan->tile;
    if (kScanVariants[v].ring) {
        const u64 fb = scan_tile_elems(kScanFallbackVariant, epv, narr);
        if (fb < sizing_tile) sizing_tile = fb;
    }
    plan->ntiles = 1 + (n + sizing_tile - 1) / sizing_tile;
    plan->words = elem_bytes <= 4 ? 1 : 2;
    if (plan->ntiles >= (1ull << 31)) return KF_ERR_INVALID_ARG;
    return KF_OK;
}

static size_t scan_ws_bytes(const ScanPlan &p) { return kHeaderBytes + align_up(p.ntiles * p.words * 8, 256); }

// Fills the geometry that depends on the actual pointers: the shared 16-byte misalignment (if
// any) becomes a short head tile, otherwise every tile takes the element-wise path.
static void scan_geometry(ScanPlan &p, u64 n, int elem_bytes, int epv, int narr, const uintptr_t *ptrs, int nptrs,
                          ScanArgs *a) {
    const uintptr_t mis = ptrs[0] & 15u;
    bool same = (mis % elem_bytes) == 0;
    for (int i = 1; i < nptrs; ++i) same = same && ((ptrs[i] & 15u) == mis);
    u64 head = 0;
    if (same && mis) head = (16 - mis) / elem_bytes;
    if (head > n) head = n;
    a->n = n;
    a->vec_ok = same ? 1 : 0;
    a->head = same ? head : 0;
    if (!same && kScanVariants[p.variant].ring) {  // the bulk-copy path needs 16-byte aligned arrays
        p.variant = kScanFallbackVariant;
        p.tile = scan_tile_elems(p.variant, epv, narr);
    }
    const u64 first = a->head > 0 ? 1 : 0;
    a->ntiles = first + (n - a->head + p.tile - 1) / p.tile;
}

}  // namespace kf

using namespace kf;

extern "C" size_t kf_scan_workspace_bytes(int32_t dtype, int32_t pair, uint64_t n, const kf_launch_cfg *cfg) {
    const int eb = pair ? 8 : dtype_bytes(dtype);
    if (eb == 0 || (pair && dtype != KF_F32)) return 0;
    ScanPlan p;
    // The interleaved pair layout has the smallest tiles (2 pairs per 16-byte vector), so its size
    // also covers the two-array layout.
    if (scan_plan(eb, 16 / eb, 1, n, cfg, &p) != KF_OK) return 0;
    return scan_ws_bytes(p);
}

// Argument checks shared by kf_scan and kf_scan_static (everything that does not involve a workspace).
static int scan_check_enums(int f, int op, int g, int dtype) {
    if (dtype_bytes(dtype) == 0) return KF_ERR_INVALID_ARG;
    if (f < KF_MAP_IDENTITY || f > KF_MAP_ABS) return KF_ERR_UNSUPPORTED;
    if (op < KF_OP_ADD || op > KF_OP_XOR) return KF_ERR_UNSUPPORTED;
    if (g < KF_POST_IDENTITY || g > KF_POST_SQRT) return KF_ERR_UNSUPPORTED;
    if (g == KF_POST_SQRT && dtype != KF_F32 && dtype != KF_F64) return KF_ERR_UNSUPPORTED;
    return KF_OK;
}

extern "C" int32_t kf_scan(int32_t f, int32_t op, int32_t g, int32_t dtype, const void *src, void *dst, uint64_t n,
                           const void *init, uint32_t ninit, void *ws, size_t ws_bytes, const kf_launch_cfg *cfg,
                           kf_stream_t stream) {
    const int erc = scan_check_enums(f, op, g, dtype);
    if (erc != KF_OK) return erc;
    const int eb = dtype_bytes(dtype);
    if (n == 0) return KF_OK;
    if (!src || !dst || !ws) return KF_ERR_INVALID_ARG;
    if (((uintptr_t)src % eb) || ((uintptr_t)dst % eb) || ((uintptr_t)ws % 256) || (init && ((uintptr_t)init % eb)))
        return KF_ERR_INVALID_ARG;
    ScanPlan p;
    int rc = scan_plan(eb, 16 / eb, 1, n, cfg, &p);
    if (rc != KF_OK) return rc;
    if (ws_bytes < scan_ws_bytes(p)) return KF_ERR_WORKSPACE_TOO_SMALL;

    ScanArgs a;
    const uintptr_t ptrs[2] = {(uintptr_t)src, (uintptr_t)dst};
    scan_geometry(p, n, eb, 16 / eb, 1, ptrs, 2, &a);
    a.header = (u32 *)ws;
    a.desc = (u64 *)((char *)ws + kHeaderBytes);
    a.init = ninit ? init : nullptr;
    a.ninit = init ? ninit : 0;
    a.f = f;
    a.g = g;
    a.spin_limit = test_spin_limit(cfg);
    a.mute_tile = test_mute_tile(cfg);
    cudaStream_t s = (cudaStream_t)stream;
    KF_LOGF("scan f=%d op=%d g=%d dtype=%d n=%llu: %dx%d %s kernel, %llu tiles, head %llu, vectors %d", f, op, g, dtype,
            (unsigned long long)n, kScanVariants[p.variant].threads, kScanVariants[p.variant].vecs,
            kScanVariants[p.variant].ring ? "persistent" : "direct", (unsigned long long)a.ntiles, (unsigned long long)a.head, a.vec_ok);
    KF_CUDA_TRY(cudaMemsetAsync(ws, 0, kHeaderBytes + a.ntiles * p.words * 8, s));
    switch (dtype) {
    case KF_U8: return scan_dispatch_u8(op, p.variant, src, dst, a, s);
    case KF_I8: return scan_dispatch_i8(op, p.variant, src, dst, a, s);
    case KF_U16: return scan_dispatch_u16(op, p.variant, src, dst, a, s);
    case KF_I16: return scan_dispatch_i16(op, p.variant, src, dst, a, s);
    case KF_U32: return scan_dispatch_u32(op, p.variant, src, dst, a, s);
    case KF_I32: return scan_dispatch_i32(op, p.variant, src, dst, a, s);
    case KF_U64: return scan_dispatch_u64(op, p.variant, src, dst, a, s);
    case KF_I64: return scan_dispatch_i64(op, p.variant, src, dst, a, s);
    case KF_F32: return scan_dispatch_f32(op, p.variant, src, dst, a, s);
    case KF_F64: return scan_dispatch_f64(op, p.variant, src, dst, a, s);
    default: return KF_ERR_INVALID_ARG;
    }
}

extern "C" int32_t kf_scan_affine_soa(const float *a_src, const float *b_src, float *a_dst, float *b_dst,
                                      uint64_t n, const float *init_ab, uint32_t ninit, void *ws, size_t ws_bytes,
                                      const kf_launch_cfg *cfg, kf_stream_t stream) {
    if (n == 0) return KF_OK;
    if (!a_src || !b_src || !a_dst || !b_dst || !ws) return KF_ERR_INVALID_ARG;
    const uintptr_t ptrs[4] = {(uintptr_t)a_src, (uintptr_t)b_src, (uintptr_t)a_dst, (uintptr_t)b_dst};
    for (int i = 0; i < 4; ++i)
        if (ptrs[i] % 4) return KF_ERR_INVALID_ARG;
    if (((uintptr_t)ws % 256) || (init_ab && ((uintptr_t)init_ab % 4))) return KF_ERR_INVALID_ARG;
    ScanPlan p;
    int rc = scan_plan(8, 4, 2, n, cfg, &p);
    if (rc != KF_OK) return rc;
    if (ws_bytes < scan_ws_bytes(p)) return KF_ERR_WORKSPACE_TOO_SMALL;

    ScanArgs a;
    scan_geometry(p, n, 4, 4, 2, ptrs, 4, &a);
    a.header = (u32 *)ws;
    a.desc = (u64 *)((char *)ws + kHeaderBytes);
    a.init = ninit ? init_ab : nullptr;
    a.ninit = init_ab ? ninit : 0;
    a.f = KF_MAP_IDENTITY;
    a.g = KF_POST_IDENTITY;
    a.spin_limit = test_spin_limit(cfg);
    a.mute_tile = test_mute_tile(cfg);
    cudaStream_t s = (cudaStream_t)stream;
    KF_CUDA_TRY(cudaMemsetAsync(ws, 0, kHeaderBytes + a.ntiles * p.words * 8, s));
    return scan_dispatch_affine_soa(p.variant, a_src, b_src, a_dst, b_dst, a, s);
}

extern "C" int32_t kf_scan_affine_aos(const float *ab_src, float *ab_dst, uint64_t n, const float *init_ab,
                                      uint32_t ninit, void *ws, size_t ws_bytes, const kf_launch_cfg *cfg, kf_stream_t stream) {
    if (n == 0) return KF_OK;
    if (!ab_src || !ab_dst || !ws) return KF_ERR_INVALID_ARG;
    if (((uintptr_t)ab_src % 4) || ((uintptr_t)ab_dst % 4) || ((uintptr_t)ws % 256) ||
        (init_ab && ((uintptr_t)init_ab % 4)))
        return KF_ERR_INVALID_ARG;
    ScanPlan p;
    int rc = scan_plan(8, 2, 1, n, cfg, &p);
    if (rc != KF_OK) return rc;
    if (ws_bytes < scan_ws_bytes(p)) return KF_ERR_WORKSPACE_TOO_SMALL;

    ScanArgs a;
    const uintptr_t ptrs[2] = {(uintptr_t)ab_src, (uintptr_t)ab_dst};
    scan_geometry(p, n, 8, 2, 1, ptrs, 2, &a);
    a.header = (u32 *)ws;
    a.desc = (u64 *)((char *)ws + kHeaderBytes);
    a.init = ninit ? init_ab : nullptr;
    a.ninit = init_ab ? ninit : 0;
    a.f = KF_MAP_IDENTITY;
    a.g = KF_POST_IDENTITY;
    a.spin_limit = test_spin_limit(cfg);
    a.mute_tile = test_mute_tile(cfg);
    cudaStream_t s = (cudaStream_t)stream;
    KF_CUDA_TRY(cudaMemsetAsync(ws, 0, kHeaderBytes + a.ntiles * p.words * 8, s));
    return scan_dispatch_affine_aos(p.variant, ab_src, ab_dst, a, s);
}

// ---- scan without a caller-supplied workspace ---------------------------------------------------------
// The tile descriptors and the ticket of kf_scan live in this fixed device array instead of a
// workspace the caller allocates. Every GPU that loads the library carries the array until the
// process exits. In host code the array's NAME is only a stand-in; its device address comes from
// cudaGetSymbolAddress, looked up once per device with that device current.
static __device__ __align__(256) unsigned char g_scan_static_scratch[KF_SCAN_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void *g_static_ptr[kMaxDevices] = {};

// Device address of the static scratch on the current device (set-up on first use per device).
int static_scratch(void **out) {
    int dev = 0;
    KF_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return KF_ERR_INVALID_ARG;
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[dev]) {
        void *ptr = nullptr;
        KF_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_scan_static_scratch));
        if (!ptr) return KF_ERR_LAUNCH_FAILED;
        g_static_ptr[dev] = ptr;
    }
    *out = g_static_ptr[dev];
    return KF_OK;
}
}  // namespace

extern "C" uint64_t kf_scan_static_max_n(int32_t dtype) {
    const int eb = dtype_bytes(dtype);
    if (eb == 0) return 0;
    // Largest n whose descriptors (sized like kf_scan_workspace_bytes does) fit the fixed array.
    u64 lo = 0, hi = 1ull << 40;
    while (lo < hi) {
        const u64 mid = lo + (hi - lo + 1) / 2;
        const size_t need = kf_scan_workspace_bytes(dtype, 0, mid, nullptr);
        if (need != 0 && need <= (size_t)KF_SCAN_STATIC_SCRATCH_BYTES) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}

extern "C" int32_t kf_scan_static(int32_t f, int32_t op, int32_t g, int32_t dtype, const void *src, void *dst, uint64_t n,
                                  const void *init, uint32_t ninit, kf_stream_t stream) {
    // Same argument checks, in the same order, as kf_scan; then the size, so that a request beyond the
    // fixed scratch is refused before anything touches the device.
    const int erc = scan_check_enums(f, op, g, dtype);
    if (erc != KF_OK) return erc;
    if (n == 0) return KF_OK;
    const size_t need = kf_scan_workspace_bytes(dtype, 0, n, nullptr);
    if (need == 0 || need > (size_t)KF_SCAN_STATIC_SCRATCH_BYTES) return KF_ERR_EXCEEDS_STATIC_SCRATCH;
    void *ws = nullptr;
    const int rc = static_scratch(&ws);
    if (rc != KF_OK) return rc;
    // kf_scan clears the header and the descriptors it is going to use at the start of the call, so
    // whatever the previous call left in the array does no harm.
    return kf_scan(f, op, g, dtype, src, dst, n, init, ninit, ws, (size_t)KF_SCAN_STATIC_SCRATCH_BYTES, nullptr, stream);
}

extern "C" int32_t kf_scan_static_check(kf_stream_t stream) {
    void *ws = nullptr;
    const int rc = static_scratch(&ws);
    if (rc != KF_OK) return rc;
    return kf_check(ws, stream);
}
