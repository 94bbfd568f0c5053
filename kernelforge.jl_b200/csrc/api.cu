// Library-level entry points: version, error text, device status read-back and the B200 launch
// table that stands in for the reference's generated per-architecture tuning files.
#include "common.cuh"

#include "launch_table.h"

#include <atomic>
#include <cstdlib>
#include <string.h>

namespace kf {

static thread_local int g_last_cuda_error = 0;
static std::atomic<unsigned long long> g_launches{0};
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
bool log_enabled() {
    static const bool on = [] {
        const char *e = std::getenv("KF_LOG");
        return e && e[0] && e[0] != '0';
    }();
    return on;
}
void set_last_cuda_error(cudaError_t e) { g_last_cuda_error = (int)e; }

// SM count of the current device; 148 (B200) when no device can be queried, so that size queries
// still answer on a machine without a GPU.
int device_sm_count() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
        (void)cudaGetLastError();
        return 148;
    }
    return sms;
}

}  // namespace kf

using namespace kf;

extern "C" int32_t kf_abi_version(void) { return KF_B200_ABI_VERSION; }

extern "C" const char *kf_error_string(int32_t status) {
    switch (status) {
    case KF_OK: return "ok";
    case KF_ERR_INVALID_ARG: return "invalid argument (null or misaligned pointer, bad enum, or size out of range)";
    case KF_ERR_UNSUPPORTED: return "unsupported combination of map, operator, element type or launch override";
    case KF_ERR_WORKSPACE_TOO_SMALL: return "workspace smaller than the *_workspace_bytes query for these arguments";
    case KF_ERR_LAUNCH_FAILED: return "a CUDA runtime call failed (see kf_last_cuda_error)";
    case KF_ERR_TIMEOUT: return "a bounded device-side wait on a tile descriptor ran out";
    case KF_ERR_EMPTY_REDUCTION: return "reducing over an empty collection is not allowed (no init value)";
    case KF_ERR_EXCEEDS_STATIC_SCRATCH: return "input too large for kf_scan_static: its tile descriptors exceed KF_SCAN_STATIC_SCRATCH_BYTES; use kf_scan with a workspace";
    default: return "unknown kf_status";
    }
}

extern "C" int32_t kf_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" int32_t kf_check(const void *ws, kf_stream_t stream) {
    if (!ws) return KF_ERR_INVALID_ARG;
    unsigned int status = 0;
    cudaStream_t s = (cudaStream_t)stream;
    KF_CUDA_TRY(cudaMemcpyAsync(&status, ws, sizeof(status), cudaMemcpyDeviceToHost, s));
    KF_CUDA_TRY(cudaStreamSynchronize(s));
    return (int32_t)status;
}

extern "C" uint64_t kf_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

// ---- peer-memory helpers of the sharded layer -------------------------------------------------------
// A rank exports one device buffer (allocated here, so that it is a whole cudaMalloc allocation, which is
// what CUDA IPC can share), the other ranks of the node map it and PULL their runs out of it with plain
// device-to-device copies over NVLink. Nothing here is on the single-GPU path.
extern "C" int32_t kf_xbuf_alloc(size_t nbytes, void **out) {
    if (!out || nbytes == 0) return KF_ERR_INVALID_ARG;
    KF_CUDA_TRY(cudaMalloc(out, nbytes));
    return KF_OK;
}

extern "C" int32_t kf_xbuf_free(void *ptr) {
    if (!ptr) return KF_OK;
    KF_CUDA_TRY(cudaFree(ptr));
    return KF_OK;
}

extern "C" int32_t kf_ipc_export(const void *ptr, void *handle64) {
    if (!ptr || !handle64) return KF_ERR_INVALID_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 opaque bytes");
    cudaIpcMemHandle_t h;
    KF_CUDA_TRY(cudaIpcGetMemHandle(&h, const_cast<void *>(ptr)));
    memcpy(handle64, &h, 64);
    return KF_OK;
}

extern "C" int32_t kf_ipc_open(const void *handle64, void **out) {
    if (!handle64 || !out) return KF_ERR_INVALID_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    KF_CUDA_TRY(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
    return KF_OK;
}

extern "C" int32_t kf_ipc_close(void *ptr) {
    if (!ptr) return KF_OK;
    KF_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
    return KF_OK;
}

extern "C" int32_t kf_copy_d2d(void *dst, const void *src, uint64_t nbytes, kf_stream_t stream) {
    if (nbytes == 0) return KF_OK;
    if (!dst || !src) return KF_ERR_INVALID_ARG;
    KF_CUDA_TRY(cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return KF_OK;
}

// ---- one-element allgather over peer memory ------------------------------------------------------------
// The exchange of the sharded mapreduce and scan: every rank contributes ONE element (a shard total).
// Each rank owns a small region that all ranks of the node have mapped; entry (slot, rank) of a region
// is two 64-bit words {epoch:32 | low half:32}, {epoch:32 | high half:32}, each of which validates itself
// (a 64-bit store is atomic), so no fence or flag separates value and tag. The kernel writes this rank's
// element into entry (slot, rank) of EVERY region with system-scope stores over NVLink, then waits, with a
// limit, until all entries of its own region carry the epoch, and writes the elements out in rank order.
// Remote data is only ever read from local memory. Slots rotate with the epoch; since every rank waits
// for every other rank, no rank can run more than one exchange ahead, so a slot is never overwritten
// before it has been read.
namespace kf {
constexpr int kPeerSlots = 4;
constexpr int kPeerMaxWorld = 64;
constexpr size_t kPeerRegionBytes = (size_t)kPeerSlots * kPeerMaxWorld * 16;

__device__ __forceinline__ void st_relaxed_sys_u64(u64 *p, u64 v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ u64 ld_relaxed_sys_u64(const u64 *p) {
    u64 v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kPeerMaxWorld) peer_allgather_kernel(u64 *const *peers, const u64 *local, int world, int rank,
                                                                       u32 epoch, const void *value, int elem_bytes, void *out,
                                                                       u32 *status, u32 spin_limit) {
    const int q = (int)threadIdx.x;
    if (q >= world) return;
    const int slot = (int)(epoch % (u32)kPeerSlots);
    u64 v = 0;
    memcpy(&v, value, (size_t)elem_bytes);  // elem_bytes <= 8
    const u64 tag = (u64)epoch << 32;
    u64 *theirs = peers[q] + ((size_t)slot * kPeerMaxWorld + rank) * 2;
    st_relaxed_sys_u64(theirs, tag | (v & 0xFFFFFFFFull));
    st_relaxed_sys_u64(theirs + 1, tag | (v >> 32));
    const u64 *mine = local + ((size_t)slot * kPeerMaxWorld + q) * 2;
    u64 w0 = 0, w1 = 0;
    bool ok = false;
    for (u32 spins = 0; spins <= spin_limit; ++spins) {
        w0 = ld_relaxed_sys_u64(mine);
        w1 = ld_relaxed_sys_u64(mine + 1);
        if ((w0 >> 32) == epoch && (w1 >> 32) == epoch) {
            ok = true;
            break;
        }
        if (spins > 16) __nanosleep(spins > 256 ? 512 : 64);
    }
    if (!ok) {
        record_error(status, KF_ERR_TIMEOUT, (u32)q);  // word 1: the rank whose element never arrived
        return;
    }
    const u64 got = (w0 & 0xFFFFFFFFull) | (w1 << 32);
    memcpy(static_cast<char *>(out) + (size_t)q * elem_bytes, &got, (size_t)elem_bytes);
}
}  // namespace kf

extern "C" size_t kf_peer_region_bytes(void) { return kPeerRegionBytes; }

extern "C" int32_t kf_peer_allgather(const void *peers, const void *local_region, int32_t world, int32_t rank, uint32_t epoch,
                                     const void *value, int32_t elem_bytes, void *out, void *status_ws,
                                     const kf_launch_cfg *cfg, kf_stream_t stream) {
    if (!peers || !local_region || !value || !out || !status_ws) return KF_ERR_INVALID_ARG;
    if (world < 1 || world > kPeerMaxWorld || rank < 0 || rank >= world || epoch == 0) return KF_ERR_INVALID_ARG;
    if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8) return KF_ERR_UNSUPPORTED;
    peer_allgather_kernel<<<1, kPeerMaxWorld, 0, (cudaStream_t)stream>>>(
        (u64 *const *)peers, (const u64 *)local_region, world, rank, epoch, value, elem_bytes, out, (u32 *)status_ws,
        test_spin_limit(cfg));
    note_launch();
    KF_CUDA_TRY(cudaGetLastError());
    return KF_OK;
}

extern "C" int32_t kf_num_sms(void) { return device_sm_count(); }

extern "C" int32_t kf_launch_table_lookup(int32_t primitive, int32_t elem_bytes, uint64_t n, kf_launch_cfg *out) {
    if (!out) return KF_ERR_INVALID_ARG;
    const LaunchRow *best = nullptr;
    const uint64_t bytes = n * (uint64_t)(elem_bytes > 0 ? elem_bytes : 1);
    // First row that matches the primitive and element size and whose bound covers the input.
    for (int i = 0; i < kNumLaunchRows && !best; ++i) {
        const LaunchRow &r = kLaunchTable[i];
        if (r.primitive != primitive) continue;
        if (r.elem_bytes != 0 && r.elem_bytes != elem_bytes) continue;
        if (bytes <= r.max_bytes) best = &r;
    }
    if (!best) return KF_ERR_UNSUPPORTED;
    out->threads = best->threads;
    out->items = best->items;
    out->blocks = best->blocks_per_sm > 0 ? best->blocks_per_sm * device_sm_count() : 0;
    out->reserved = 0;
    return KF_OK;
}
