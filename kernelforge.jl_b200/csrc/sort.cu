// Host entry points of the radix onesweep sort (C ABI): workspace layout, ping-pong plan, pass loop.
// The kernels live in sort_impl.cuh and are instantiated per key width in sort_inst_*.cu.
#include "sort_impl.cuh"

namespace kf {

__global__ void sort_scan_histogram_kernel(u64 *ghist) {
    __shared__ u64 s_warp[kRadix / 32];
    grid_dep_wait();  // chained behind the histogram kernel
    u64 *h = ghist + (size_t)blockIdx.x * kRadix;
    const u32 tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const u64 c = h[tid];
    u64 incl = c;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const u64 up = __shfl_up_sync(0xFFFFFFFFu, incl, d);
        if (lane >= (u32)d) incl += up;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    u64 base = 0;
    for (u32 w = 0; w < warp; ++w) base += s_warp[w];
    h[tid] = base + incl - c;
}

// One-byte keys without a payload: equal keys are the same byte, so the sorted array is the histogram
// written out as 256 runs. gexcl[d] is the start of digit d's run (digit = byte ^ top_xor, the sign flip
// of signed keys). Each CTA fills one contiguous piece of dst with 128-bit stores; a thread's positions
// only grow, so it walks the run boundaries forward from one binary search at the start of the piece.
// The 1-byte path of the reference (src/sort/byte_sort_kernel.jl:1-17) still scatters every key.
__global__ void __launch_bounds__(256) byte_runs_fill_kernel(uint8_t *dst, u64 n, const u64 *gexcl, u32 top_xor) {
    __shared__ u64 s_excl[kRadix + 1];
    const u32 tid = threadIdx.x;
    grid_dep_wait();  // chained behind the bin scan
    s_excl[tid] = gexcl[tid];
    if (tid == 0) s_excl[kRadix] = n;
    __syncthreads();
    auto digit_at = [&](u64 j) {  // the digit whose run holds position j < n (the largest d with start <= j)
        int lo = 0, hi = kRadix;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_excl[mid] <= j) lo = mid;
            else hi = mid;
        }
        return lo;
    };
    u64 head = (16 - ((uintptr_t)dst & 15u)) & 15u;  // bytes before the first 16-byte boundary
    if (head > n) head = n;
    const u64 nvec = (n - head) / 16;
    const u64 per_cta = (nvec + gridDim.x - 1) / gridDim.x;
    const u64 v_lo = (u64)blockIdx.x * per_cta;
    const u64 v_hi = v_lo + per_cta < nvec ? v_lo + per_cta : nvec;
    if (v_lo + tid < v_hi) {
        int d = digit_at(head + (v_lo + tid) * 16);
        for (u64 v = v_lo + tid; v < v_hi; v += 256) {
            const u64 j0 = head + v * 16;
            while (s_excl[d + 1] <= j0) ++d;
            uint4 o;
            if (s_excl[d + 1] >= j0 + 16) {  // the whole vector lies in one run
                const u32 w = ((u32)d ^ top_xor) * 0x01010101u;
                o = make_uint4(w, w, w, w);
            } else {
                uint8_t b[16];
                int e_d = d;
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    while (s_excl[e_d + 1] <= j0 + e) ++e_d;
                    b[e] = (uint8_t)((u32)e_d ^ top_xor);
                }
                memcpy(&o, b, 16);
            }
            st_stream_v4(dst + j0, o);
        }
    }
    if (blockIdx.x == 0) {  // the ragged ends
        const u64 tail = head + nvec * 16;
        if (tid < head) dst[tid] = (uint8_t)((u32)digit_at(tid) ^ top_xor);
        if (tid < 16 && tail + tid < n) dst[tail + tid] = (uint8_t)((u32)digit_at(tail + tid) ^ top_xor);
    }
}

// Two-byte keys without a payload, large n: the same idea with 65 536 bins. A CTA cannot hold that
// many 32-bit counters, so the CTAs work in pairs over the same piece of the input: the even CTA counts
// the keys whose mapped value is below 32 768, the odd one the rest (128 KB of counters each; the
// second read of a piece comes from L2). `flip` is 0x8000 for signed keys (the uint_map sign flip).
constexpr int kShortBins = 65536;
constexpr u64 kShortRunsMinN = 1ull << 22;  // below this the two-pass onesweep is used (and the counters would not fit the scratch)
__global__ void __launch_bounds__(1024) short_histogram_kernel(const uint16_t *__restrict__ keys, u64 n, u64 *gcount, u32 flip) {
    extern __shared__ __align__(16) u32 sh_half[];  // [32768]
    const u32 tid = threadIdx.x, role = blockIdx.x & 1u;
    const u64 pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    for (u32 i = tid; i < kShortBins / 2 / 4; i += 1024) reinterpret_cast<uint4 *>(sh_half)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    // raw keys are counted; `flip` (0x8000 for signed keys) only swaps which CTA of the pair owns which
    // half of the raw value range, and is applied to the bin index when the counters are flushed
    const u32 raw_role = role ^ (flip >> 15);
    auto count_key = [&](u32 k) {
        if ((k >> 15) == raw_role) atomicAdd(&sh_half[k & 0x7FFFu], 1u);
    };
    const u64 mis = ((uintptr_t)keys & 15u) / 2;
    u64 head = mis ? 8 - mis : 0;
    if (head > n) head = n;
    const u64 nvec = (n - head) / 8;
    const uint4 *vsrc = reinterpret_cast<const uint4 *>(keys + head);
    constexpr int UNROLL = 4;
    const u64 strip = 1024ull * UNROLL;
    for (u64 base = pair * strip; base < nvec; base += npairs * strip) {
        uint4 v[UNROLL];
        bool ok[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const u64 idx = base + (u64)u * 1024 + tid;
            ok[u] = idx < nvec;
            if (ok[u]) v[u] = ld_stream_v4(vsrc + idx);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (ok[u]) {
                const u32 w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    count_key(w[q] & 0xFFFFu);
                    count_key(w[q] >> 16);
                }
            }
        }
    }
    if (pair == 0) {  // the ragged ends (fewer than 8 keys each)
        const u64 tail = head + nvec * 8;
        if (tid < head) count_key(keys[tid]);
        if (tid < 8 && tail + tid < n) count_key(keys[tail + tid]);
    }
    __syncthreads();
    for (u32 i = tid; i < kShortBins / 2; i += 1024) {
        const u32 c = sh_half[i];
        if (c) atomicAdd(reinterpret_cast<unsigned long long *>(gcount) + role * (kShortBins / 2) + i, (unsigned long long)c);
    }
}

// Exclusive prefix of the 65 536 counts in place, and the total in entry 65 536. One CTA of 32 warps;
// a warp owns 2048 consecutive bins and reads them 32 at a time (coalesced), twice: once for its
// total, once for the running prefix.
__global__ void __launch_bounds__(1024) short_scan_kernel(u64 *gcount) {
    __shared__ u64 s_warp[32];
    const u32 tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    grid_dep_wait();  // chained behind the histogram kernel
    u64 *seg = gcount + (size_t)warp * (kShortBins / 32);
    u64 part = 0;
    for (int it = 0; it < kShortBins / 1024; ++it) part += seg[it * 32 + lane];
#pragma unroll
    for (int d = 16; d; d >>= 1) part += __shfl_xor_sync(0xFFFFFFFFu, part, d);
    if (lane == 0) s_warp[warp] = part;
    __syncthreads();
    u64 run = 0;
    for (u32 w = 0; w < warp; ++w) run += s_warp[w];
    for (int it = 0; it < kShortBins / 1024; ++it) {
        const u64 c = seg[it * 32 + lane];
        u64 incl = c;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const u64 up = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= (u32)d) incl += up;
        }
        seg[it * 32 + lane] = run + incl - c;
        run += __shfl_sync(0xFFFFFFFFu, incl, 31);
    }
    if (tid == 1023) gcount[kShortBins] = run;
}

// dst = the 65 536 runs. excl[d] is the start of the run of mapped value d, excl[65536] = n. A thread's
// positions only grow, so it walks the run boundaries forward; after 24 steps without reaching its
// position (sparse keys: long stretches of empty bins) it falls back to a binary search.
__global__ void __launch_bounds__(256) short_runs_fill_kernel(uint16_t *dst, u64 n, const u64 *__restrict__ excl, u32 flip) {
    const u32 tid = threadIdx.x;
    grid_dep_wait();  // chained behind the bin scan
    auto digit_at = [&](u64 j) {  // the largest d with excl[d] <= j, for j < n
        int lo = 0, hi = kShortBins;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (__ldg(excl + mid) <= j) lo = mid;
            else hi = mid;
        }
        return lo;
    };
    auto advance = [&](int d, u64 j) {  // from a digit at or before j's to j's
        for (int steps = 0; __ldg(excl + d + 1) <= j; ++d)
            if (++steps == 24) return digit_at(j);
        return d;
    };
    u64 head = ((16 - ((uintptr_t)dst & 15u)) & 15u) / 2;  // elements before the first 16-byte boundary
    if (head > n) head = n;
    const u64 nvec = (n - head) / 8;
    const u64 per_cta = (nvec + gridDim.x - 1) / gridDim.x;
    const u64 v_lo = (u64)blockIdx.x * per_cta;
    const u64 v_hi = v_lo + per_cta < nvec ? v_lo + per_cta : nvec;
    if (v_lo + tid < v_hi) {
        int d = digit_at(head + (v_lo + tid) * 8);
        for (u64 v = v_lo + tid; v < v_hi; v += 256) {
            const u64 j0 = head + v * 8;
            d = advance(d, j0);
            uint4 o;
            if (__ldg(excl + d + 1) >= j0 + 8) {  // the whole vector lies in one run
                const u32 w = ((u32)d ^ flip) * 0x00010001u;
                o = make_uint4(w, w, w, w);
            } else {
                uint16_t b[8];
                int e_d = d;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    e_d = advance(e_d, j0 + e);
                    b[e] = (uint16_t)((u32)e_d ^ flip);
                }
                memcpy(&o, b, 16);
            }
            st_stream_v4(dst + j0, o);
        }
    }
    if (blockIdx.x == 0) {  // the ragged ends
        const u64 tail = head + nvec * 8;
        if (tid < head) dst[tid] = (uint16_t)((u32)digit_at(tid) ^ flip);
        if (tid < 8 && tail + tid < n) dst[tail + tid] = (uint16_t)((u32)digit_at(tail + tid) ^ flip);
    }
}

struct KeyInfo {
    int bytes;
    bool is_float;
    bool signed_or_float;
};
static bool key_info(int dtype, KeyInfo *k) {
    switch (dtype) {
    case KF_U8: *k = {1, false, false}; return true;
    case KF_I8: *k = {1, false, true}; return true;
    case KF_U16: *k = {2, false, false}; return true;
    case KF_I16: *k = {2, false, true}; return true;
    case KF_U32: *k = {4, false, false}; return true;
    case KF_I32: *k = {4, false, true}; return true;
    case KF_F32: *k = {4, true, true}; return true;
    case KF_U64: *k = {8, false, false}; return true;
    case KF_I64: *k = {8, false, true}; return true;
    case KF_F64: *k = {8, true, true}; return true;
    default: return false;
    }
}

struct SortPlan {
    int variant;
    u64 tile, ntiles;
    size_t off_hist, off_desc, off_keys, off_vals, clear_bytes, total;
};

static int sort_plan(const KeyInfo &k, int val_bytes, u64 n, const kf_launch_cfg *cfg, SortPlan *p) {
    kf_launch_cfg t;
    kf_launch_table_lookup(val_bytes ? KF_PRIM_SORT_PAIRS : KF_PRIM_SORT_KEYS, k.bytes + val_bytes, n, &t);
    if (cfg) {
        if (cfg->threads) t.threads = cfg->threads;
        if (cfg->items) t.items = cfg->items;
    }
    int v = -1;
    for (int i = 0; i < kNumSortVariants; ++i)
        if (kSortVariants[i].threads == t.threads && kSortVariants[i].items == t.items) v = i;
    if (v < 0) return KF_ERR_UNSUPPORTED;
    if (sort_smem_bytes(t.threads, t.items, k.bytes, val_bytes) > 227 * 1024) return KF_ERR_UNSUPPORTED;
    p->variant = v;
    p->tile = (u64)t.threads * t.items;
    p->ntiles = (n + p->tile - 1) / p->tile;
    if (p->ntiles >= (1ull << 31)) return KF_ERR_INVALID_ARG;
    p->off_hist = kHeaderBytes;
    p->off_desc = p->off_hist + align_up((size_t)k.bytes * kRadix * 8, 256);
    p->clear_bytes = p->off_desc + p->ntiles * kRadix * 8;
    p->off_keys = align_up(p->clear_bytes, 256);
    p->off_vals = p->off_keys + align_up(n * k.bytes, 256);
    p->total = p->off_vals + align_up(n * val_bytes, 256);
    return KF_OK;
}

static int sort_run(int key_dtype, const void *keys_src, void *keys_dst, int val_bytes, const void *vals_src,
                    void *vals_dst, u64 n, void *ws, size_t ws_bytes, const kf_launch_cfg *cfg, cudaStream_t s) {
    KeyInfo k;
    if (!key_info(key_dtype, &k)) return dtype_bytes(key_dtype) ? KF_ERR_UNSUPPORTED : KF_ERR_INVALID_ARG;
    if (val_bytes != 0 && val_bytes != 4 && val_bytes != 8) return KF_ERR_UNSUPPORTED;
    if (n == 0) return KF_OK;
    if (!keys_src || !keys_dst || !ws) return KF_ERR_INVALID_ARG;
    if (val_bytes && (!vals_src || !vals_dst)) return KF_ERR_INVALID_ARG;
    if (((uintptr_t)keys_src % k.bytes) || ((uintptr_t)keys_dst % k.bytes) || ((uintptr_t)ws % 256))
        return KF_ERR_INVALID_ARG;
    if (val_bytes && (((uintptr_t)vals_src % val_bytes) || ((uintptr_t)vals_dst % val_bytes)))
        return KF_ERR_INVALID_ARG;
    SortPlan p;
    int rc = sort_plan(k, val_bytes, n, cfg, &p);
    if (rc != KF_OK) return rc;
    if (ws_bytes < p.total) return KF_ERR_WORKSPACE_TOO_SMALL;

    char *base = (char *)ws;
    u32 *header = (u32 *)base;
    u64 *ghist = (u64 *)(base + p.off_hist);
    u64 *desc = (u64 *)(base + p.off_desc);
    void *kscratch = base + p.off_keys;
    void *vscratch = base + p.off_vals;

    // One-byte keys alone (no payload; not under the bounded-wait test hook, which needs the look-back):
    // histogram, 256-bin scan, runs written out. In place works as it is: the histogram has read src
    // before the fill starts.
    const bool byte_runs = k.bytes == 1 && val_bytes == 0 && test_mute_tile(cfg) == 0;
    KF_LOGF("sort key bytes=%d float=%d payload bytes=%d n=%llu: %s, %dx%d, %llu tiles", k.bytes, (int)k.is_float, val_bytes,
            (unsigned long long)n,
            byte_runs ? "256 runs written out" : (k.bytes == 2 && val_bytes == 0 && n >= kShortRunsMinN && test_mute_tile(cfg) == 0)
                                                     ? "65536 runs written out" : "onesweep passes",
            kSortVariants[p.variant].threads, kSortVariants[p.variant].items, (unsigned long long)p.ntiles);
    // Two-byte keys alone, from kShortRunsMinN keys: 65 536-bin histogram (counters in the key scratch,
    // which this path does not otherwise need), scan, runs written out.
    if (k.bytes == 2 && val_bytes == 0 && n >= kShortRunsMinN && test_mute_tile(cfg) == 0) {
        u64 *gcount = (u64 *)kscratch;
        const u32 flip = k.signed_or_float ? 0x8000u : 0u;
        KF_CUDA_TRY(cudaMemsetAsync(ws, 0, kHeaderBytes, s));
        KF_CUDA_TRY(cudaMemsetAsync(gcount, 0, (size_t)(kShortBins + 1) * 8, s));
        const int pairs = device_sm_count() / 2 > 0 ? device_sm_count() / 2 : 1;
        constexpr size_t kSmem = (size_t)kShortBins / 2 * 4;
        KF_CUDA_TRY(cudaFuncSetAttribute(short_histogram_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem));
        short_histogram_kernel<<<2 * pairs, 1024, kSmem, s>>>((const uint16_t *)keys_src, n, gcount, flip); note_launch();
        KF_CUDA_TRY(launch_chained(short_scan_kernel, 1u, 1024u, 0, s, gcount)); note_launch();
        // a persistent grid here: every CTA starts with a binary search in the 65 537 run starts, which
        // sit in global memory (one strip per CTA, as for one-byte keys, was measured: 1.70 against 1.63 ms at 2^30)
        const u64 nvec = n / 8;
        u64 blocks = (nvec + 255) / 256;
        const u64 cap = (u64)device_sm_count() * 8;
        if (blocks > cap) blocks = cap;
        KF_CUDA_TRY(launch_chained(short_runs_fill_kernel, (unsigned)blocks, 256u, 0, s, (uint16_t *)keys_dst, n, (const u64 *)gcount, flip)); note_launch();
        KF_CUDA_TRY(cudaGetLastError());
        return KF_OK;
    }
    KF_CUDA_TRY(cudaMemsetAsync(ws, 0, byte_runs ? p.off_desc : p.clear_bytes, s));
    switch (k.bytes) {
    case 1: rc = sort_hist_k8(keys_src, n, ghist, k.signed_or_float, s); break;
    case 2: rc = sort_hist_k16(keys_src, n, ghist, k.signed_or_float, s); break;
    case 4: rc = sort_hist_k32(k.is_float, keys_src, n, ghist, k.signed_or_float, s); break;
    default: rc = sort_hist_k64(k.is_float, keys_src, n, ghist, k.signed_or_float, s); break;
    }
    if (rc != KF_OK) return rc;
    KF_CUDA_TRY(launch_chained(sort_scan_histogram_kernel, (unsigned)k.bytes, (unsigned)kRadix, 0, s, ghist)); note_launch();
    KF_CUDA_TRY(cudaGetLastError());
    if (byte_runs) {
        // four 16-byte stores per thread and as many CTAs as that takes (streaming writes run faster from
        // many short CTAs than from a persistent grid)
        u64 blocks = (n / 16 + 1023) / 1024;
        if (blocks < 1) blocks = 1;
        if (blocks >= (1ull << 31)) return KF_ERR_INVALID_ARG;
        KF_CUDA_TRY(launch_chained(byte_runs_fill_kernel, (unsigned)blocks, 256u, 0, s, (uint8_t *)keys_dst, n, (const u64 *)ghist,
                                   k.signed_or_float ? 0x80u : 0u));
        note_launch();
        KF_CUDA_TRY(cudaGetLastError());
        return KF_OK;
    }

    // Ping-pong plan: pass p writes dst when the number of passes still to come is even, else the
    // scratch; pass 0 reads src. With an even pass count this never writes src unless dst == src,
    // and the last pass always lands in dst. One-byte keys take a single pass, which would read and
    // write the same array when sorting in place: that case starts from a copy in the scratch.
    const int P = k.bytes;
    const void *kin = keys_src, *vin = vals_src;
    if (P % 2 == 1) {
        if (keys_dst == keys_src) {
            KF_CUDA_TRY(cudaMemcpyAsync(kscratch, keys_src, n * k.bytes, cudaMemcpyDeviceToDevice, s));
            kin = kscratch;
        }
        if (val_bytes && vals_dst == vals_src) {
            KF_CUDA_TRY(cudaMemcpyAsync(vscratch, vals_src, n * val_bytes, cudaMemcpyDeviceToDevice, s));
            vin = vscratch;
        }
    }
    for (int pass = 0; pass < P; ++pass) {
        const bool to_dst = ((P - 1 - pass) % 2) == 0;
        void *kout = to_dst ? keys_dst : kscratch;
        void *vout = to_dst ? vals_dst : vscratch;
        SortPassArgs a;
        a.keys_in = kin;
        a.keys_out = kout;
        a.vals_in = vin;
        a.vals_out = vout;
        a.n = n;
        a.ntiles = p.ntiles;
        a.gexcl = ghist + (size_t)pass * kRadix;
        a.desc = desc;
        a.header = header;
        a.pass = pass;
        a.shift = 8 * pass;
        a.top_xor = (pass == P - 1 && k.signed_or_float) ? 0x80u : 0u;
        a.signed_or_float = k.signed_or_float;
        a.spin_limit = test_spin_limit(cfg);
        a.mute_tile = test_mute_tile(cfg);
        switch (k.bytes) {
        case 1: rc = sort_pass_k8(val_bytes, p.variant, a, s); break;
        case 2: rc = sort_pass_k16(val_bytes, p.variant, a, s); break;
        case 4: rc = sort_pass_k32(k.is_float, val_bytes, p.variant, a, s); break;
        default: rc = sort_pass_k64(k.is_float, val_bytes, p.variant, a, s); break;
        }
        if (rc != KF_OK) return rc;
        kin = kout;
        vin = vout;
    }
    return KF_OK;
}

// ---- small helpers of the sharded layer ---------------------------------------------------------
template <typename T> __global__ void iota_kernel(T *dst, u64 n, u64 start) {
    const u64 stride = (u64)gridDim.x * blockDim.x;
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = (T)(start + i);
}

// Order-preserving unsigned image of a key (the reference's uint_map).
template <typename KeyT, bool IS_FLOAT> __device__ __forceinline__ KeyT mapped_key(KeyT k, bool sof) {
    const KeyT sign = (KeyT)1 << (8 * sizeof(KeyT) - 1);
    return radix_bits<KeyT, IS_FLOAT>(k) ^ (sof ? sign : (KeyT)0);
}

template <typename KeyT, bool IS_FLOAT>
__global__ void upper_bounds_kernel(const KeyT *keys, u64 n, const KeyT *splitters, int nsplit, u64 *out, bool sof) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= nsplit) return;
    const KeyT s = mapped_key<KeyT, IS_FLOAT>(splitters[j], sof);
    u64 lo = 0, hi = n;  // first index whose mapped key is > s
    while (lo < hi) {
        const u64 mid = lo + (hi - lo) / 2;
        if (mapped_key<KeyT, IS_FLOAT>(keys[mid], sof) <= s) lo = mid + 1;
        else hi = mid;
    }
    out[j] = lo;
}

}  // namespace kf

using namespace kf;

extern "C" size_t kf_sort_workspace_bytes(int32_t key_dtype, int32_t val_bytes, uint64_t n, const kf_launch_cfg *cfg) {
    KeyInfo k;
    if (!key_info(key_dtype, &k)) return 0;
    if (val_bytes != 0 && val_bytes != 4 && val_bytes != 8) return 0;
    SortPlan p;
    if (sort_plan(k, val_bytes, n, cfg, &p) != KF_OK) return 0;
    return p.total;
}

extern "C" int32_t kf_sort_keys(int32_t key_dtype, const void *src, void *dst, uint64_t n, void *ws,
                                size_t ws_bytes, const kf_launch_cfg *cfg, kf_stream_t stream) {
    return sort_run(key_dtype, src, dst, 0, nullptr, nullptr, n, ws, ws_bytes, cfg, (cudaStream_t)stream);
}

extern "C" int32_t kf_sort_pairs(int32_t key_dtype, const void *keys_src, void *keys_dst, int32_t val_bytes,
                                 const void *vals_src, void *vals_dst, uint64_t n, void *ws, size_t ws_bytes,
                                 const kf_launch_cfg *cfg, kf_stream_t stream) {
    if (val_bytes == 0) return KF_ERR_INVALID_ARG;
    return sort_run(key_dtype, keys_src, keys_dst, val_bytes, vals_src, vals_dst, n, ws, ws_bytes, cfg,
                    (cudaStream_t)stream);
}

extern "C" int32_t kf_iota(int32_t dtype, void *dst, uint64_t n, uint64_t start, kf_stream_t stream) {
    if (n == 0) return KF_OK;
    if (!dst) return KF_ERR_INVALID_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    u64 blocks = (n + 1023) / 1024;
    const u64 cap = (u64)device_sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (dtype == KF_U32 || dtype == KF_I32) iota_kernel<uint32_t><<<(unsigned)blocks, 256, 0, s>>>((uint32_t *)dst, n, start);
    else if (dtype == KF_U64 || dtype == KF_I64) iota_kernel<u64><<<(unsigned)blocks, 256, 0, s>>>((u64 *)dst, n, start);
    else return KF_ERR_UNSUPPORTED;
    note_launch();
    KF_CUDA_TRY(cudaGetLastError());
    return KF_OK;
}

template <typename KeyT>
static void launch_upper_bounds(const KeyInfo &k, const void *keys, u64 n, const void *splitters, int nsplit, u64 *out, cudaStream_t s) {
    const int threads = 128, blocks = (nsplit + threads - 1) / threads;
    if (k.is_float)
        upper_bounds_kernel<KeyT, sizeof(KeyT) >= 4><<<blocks, threads, 0, s>>>((const KeyT *)keys, n, (const KeyT *)splitters, nsplit, out, true);
    else
        upper_bounds_kernel<KeyT, false><<<blocks, threads, 0, s>>>((const KeyT *)keys, n, (const KeyT *)splitters, nsplit, out,
                                                                     k.signed_or_float);
    note_launch();
}

extern "C" int32_t kf_upper_bounds(int32_t key_dtype, const void *keys, uint64_t n, const void *splitters,
                                   int32_t nsplit, uint64_t *out, kf_stream_t stream) {
    KeyInfo k;
    if (!key_info(key_dtype, &k)) return KF_ERR_UNSUPPORTED;
    if (nsplit <= 0) return KF_OK;
    if (!splitters || !out || (n && !keys)) return KF_ERR_INVALID_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    switch (k.bytes) {
    case 1: launch_upper_bounds<uint8_t>(k, keys, n, splitters, nsplit, (u64 *)out, s); break;
    case 2: launch_upper_bounds<uint16_t>(k, keys, n, splitters, nsplit, (u64 *)out, s); break;
    case 4: launch_upper_bounds<uint32_t>(k, keys, n, splitters, nsplit, (u64 *)out, s); break;
    default: launch_upper_bounds<u64>(k, keys, n, splitters, nsplit, (u64 *)out, s); break;
    }
    KF_CUDA_TRY(cudaGetLastError());
    return KF_OK;
}

// out[i] = number of splitters whose mapped key is smaller than that of keys[i]: the destination of
// key i in a sample sort whose piece j holds the keys in (splitter[j-1], splitter[j]].
template <typename KeyT, bool IS_FLOAT>
__global__ void __launch_bounds__(256) bucket_ids_kernel(const KeyT *keys, u64 n, const KeyT *splitters, int nsplit, uint8_t *out, bool sof) {
    __shared__ KeyT s_split[256];
    for (int j = threadIdx.x; j < nsplit; j += blockDim.x) s_split[j] = mapped_key<KeyT, IS_FLOAT>(splitters[j], sof);
    __syncthreads();
    const u64 stride = (u64)gridDim.x * blockDim.x;
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const KeyT m = mapped_key<KeyT, IS_FLOAT>(keys[i], sof);
        int lo = 0, hi = nsplit;  // first splitter that is >= m
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (s_split[mid] < m) lo = mid + 1;
            else hi = mid;
        }
        out[i] = (uint8_t)lo;
    }
}

// The same for 16-byte aligned arrays: a thread takes 16 consecutive keys with 128-bit loads and writes
// its 16 ids with one 128-bit store (one-byte stores made the scalar kernel issue-bound at a quarter of
// the HBM rate).
template <typename KeyT, bool IS_FLOAT>
__global__ void __launch_bounds__(256) bucket_ids_vec_kernel(const KeyT *keys, u64 n16, const KeyT *splitters, int nsplit, uint8_t *out,
                                                             bool sof) {
    constexpr int KPV = 16 / sizeof(KeyT);  // keys per 16-byte vector
    constexpr int NV = 16 / KPV;            // vectors per 16 keys
    __shared__ KeyT s_split[256];
    for (int j = threadIdx.x; j < nsplit; j += blockDim.x) s_split[j] = mapped_key<KeyT, IS_FLOAT>(splitters[j], sof);
    __syncthreads();
    const u64 stride = (u64)gridDim.x * blockDim.x;
    for (u64 g = (u64)blockIdx.x * blockDim.x + threadIdx.x; g < n16; g += stride) {
        uint4 v[NV];
#pragma unroll
        for (int q = 0; q < NV; ++q) v[q] = ld_stream_v4(reinterpret_cast<const uint4 *>(keys + g * 16) + q);
        KeyT k[16];
        memcpy(k, v, 16 * sizeof(KeyT));
        uint8_t id[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const KeyT m = mapped_key<KeyT, IS_FLOAT>(k[e], sof);
            int lo = 0, hi = nsplit;  // first splitter that is >= m
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (s_split[mid] < m) lo = mid + 1;
                else hi = mid;
            }
            id[e] = (uint8_t)lo;
        }
        uint4 o;
        memcpy(&o, id, 16);
        st_stream_v4(out + g * 16, o);
    }
}

template <typename KeyT>
static void launch_bucket_ids(const KeyInfo &k, const void *keys, u64 n, const void *splitters, int nsplit, uint8_t *out, cudaStream_t s) {
    const bool fl = k.is_float && sizeof(KeyT) >= 4;
    u64 done = 0;
    if ((((uintptr_t)keys | (uintptr_t)out) & 15u) == 0 && n >= 16) {
        const u64 n16 = n / 16;
        u64 blocks = (n16 + 255) / 256;
        const u64 cap = (u64)device_sm_count() * 8;
        if (blocks > cap) blocks = cap;
        if (fl)
            bucket_ids_vec_kernel<KeyT, sizeof(KeyT) >= 4><<<(unsigned)blocks, 256, 0, s>>>((const KeyT *)keys, n16, (const KeyT *)splitters, nsplit, out, true);
        else
            bucket_ids_vec_kernel<KeyT, false><<<(unsigned)blocks, 256, 0, s>>>((const KeyT *)keys, n16, (const KeyT *)splitters, nsplit, out,
                                                                                 k.signed_or_float);
        note_launch();
        done = n16 * 16;
        if (done == n) return;
    }
    // scalar kernel: misaligned arrays, and the last n mod 16 keys
    const KeyT *kp = (const KeyT *)keys + done;
    const u64 rest = n - done;
    u64 blocks = (rest + 255) / 256;
    const u64 cap = (u64)device_sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (fl)
        bucket_ids_kernel<KeyT, sizeof(KeyT) >= 4><<<(unsigned)blocks, 256, 0, s>>>(kp, rest, (const KeyT *)splitters, nsplit, out + done, true);
    else
        bucket_ids_kernel<KeyT, false><<<(unsigned)blocks, 256, 0, s>>>(kp, rest, (const KeyT *)splitters, nsplit, out + done,
                                                                         k.signed_or_float);
    note_launch();
}

extern "C" int32_t kf_bucket_ids(int32_t key_dtype, const void *keys, uint64_t n, const void *splitters, int32_t nsplit,
                                 uint8_t *out, kf_stream_t stream) {
    KeyInfo k;
    if (!key_info(key_dtype, &k)) return KF_ERR_UNSUPPORTED;
    if (nsplit < 0 || nsplit > 255) return KF_ERR_INVALID_ARG;
    if (n == 0) return KF_OK;
    if (!keys || !out || (nsplit && !splitters)) return KF_ERR_INVALID_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    switch (k.bytes) {
    case 1: launch_bucket_ids<uint8_t>(k, keys, n, splitters, nsplit, out, s); break;
    case 2: launch_bucket_ids<uint16_t>(k, keys, n, splitters, nsplit, out, s); break;
    case 4: launch_bucket_ids<uint32_t>(k, keys, n, splitters, nsplit, out, s); break;
    default: launch_bucket_ids<u64>(k, keys, n, splitters, nsplit, out, s); break;
    }
    KF_CUDA_TRY(cudaGetLastError());
    return KF_OK;
}
