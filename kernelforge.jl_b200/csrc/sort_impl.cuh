// Stable LSD radix sort for sm_100a: one fused multi-digit histogram pass, then one "onesweep"
// pass per key byte (rank inside the tile, decoupled look-back for the per-digit global offsets,
// scatter staged through shared memory so each digit's run leaves the CTA contiguously).
//
// Key order is the reference's uint_map (src/sort/uint_map.jl:11-35 of KernelForge.jl): unsigned
// keys by value, signed keys with the sign bit flipped, floats sign-flipped when non-negative and
// complemented when negative. Only digit extraction uses the mapped key; the original bits are
// what moves. For integer keys the map only changes the top byte, so it costs one XOR folded into
// the digit mask (`top_xor`); float keys add a shift and one logic op per key for the complement.
//
// Ranking is done per half-warp ("unit" of 16 lanes, which owns 16 * ITEMS consecutive elements of
// the tile) on a private table of one 32-bit word per digit: {lanes holding the digit in the
// current item : 16 | keys of the digit seen in earlier items : 16}. Per item every lane announces
// itself with an atomic add of its lane bit, the unit meets at a warp barrier, every lane reads the
// word (its rank = count + number of lower lanes in the mask), the unit meets again, and the highest
// lane of each group folds the group into the count with a second atomic add. Atomic adds commute
// and the two warp barriers order them against the reads, so ranks follow element order for any
// data on any schedule: that is what makes each pass stable (the reference leans on lane-ordered
// resolution of same-address shared atomics, src/sort/onesweep_kernel.jl:19-24, which CUDA does
// not promise).
//
// Tile descriptors are one 64-bit word per (tile, digit): {tag:8 | count:56}. The tag encodes the
// pass and the state (aggregate / inclusive prefix / poison), so one descriptor array, cleared
// once per sort call, serves all passes and counts are not limited to 30 bits. Tiles are handed
// out by an atomic ticket; every wait is bounded.
#pragma once

#include "common.cuh"

#include <type_traits>

namespace kf {

constexpr int kRadix = 256;

enum : u32 { kStAggregate = 0, kStPrefix = 1, kStPoison = 2 };
__host__ __device__ __forceinline__ u64 desc_tag(int pass, u32 state) { return (u64)(1 + pass * 3 + (int)state) << 56; }
constexpr u64 kCountMask = (1ull << 56) - 1;

// Bits of the key that feed digit extraction, before the shift. The sign bit is flipped for every
// signed or float key, and only shows in the top digit, so that flip is applied to the top digit
// by `top_xor`. What is left: integers use the key itself; negative floats are complemented
// below the sign bit: key ^ (sign-extension of the sign bit, with the sign bit cleared).
template <typename KeyT, bool IS_FLOAT> __device__ __forceinline__ KeyT radix_bits(KeyT k) {
    if constexpr (IS_FLOAT) {
        if constexpr (sizeof(KeyT) == 4) return k ^ ((KeyT)((int32_t)k >> 31) & (KeyT)0x7FFFFFFFu);
        else return k ^ ((KeyT)((long long)k >> 63) & (KeyT)0x7FFFFFFFFFFFFFFFull);
    } else {
        return k;
    }
}
// A key whose digit is 255 at every position (pads the last, ragged tile; it ranks after every
// real key of the tile and is never written out).
template <typename KeyT, bool IS_FLOAT> __device__ __forceinline__ KeyT pad_key(bool signed_or_float) {
    // integers: digits are key bytes, top digit ^0x80 when signed -> top byte 0x7F, others 0xFF.
    // floats: a non-negative key keeps its bits -> the same pattern 0x7FFF...FF maps to all ones.
    KeyT all = (KeyT)~(KeyT)0;
    return signed_or_float ? (KeyT)(all >> 1) : all;
}

// ---------------------------------------------------------------------------------------------
// Histogram of every digit position in one read of the keys. ghist[p*256 + d] (64-bit counts).
// ---------------------------------------------------------------------------------------------
template <typename KeyT, bool IS_FLOAT, int THREADS>
__global__ void __launch_bounds__(THREADS)
sort_histogram_kernel(const KeyT *__restrict__ keys, u64 n, u64 *ghist, int signed_or_float) {
    constexpr int P = sizeof(KeyT);
    constexpr int EPV = 16 / sizeof(KeyT);
    __shared__ u32 sh[P * kRadix];
    const u32 tid = threadIdx.x;
    for (u32 i = tid; i < P * kRadix; i += THREADS) sh[i] = 0;
    __syncthreads();

    // Raw bytes are counted; the sign flip of the top digit (signed and float keys) is a permutation of
    // that digit's bins and is applied once, when the bins are added to the global histogram.
    auto count_key = [&](KeyT k) {
        const KeyT b = radix_bits<KeyT, IS_FLOAT>(k);
#pragma unroll
        for (int p = 0; p < P; ++p) atomicAdd(&sh[p * kRadix + ((u32)(b >> (8 * p)) & 0xFFu)], 1u);
    };

    const u64 mis = ((uintptr_t)keys & 15u) / sizeof(KeyT);
    u64 head = mis ? (EPV - mis) : 0;
    if (head > n) head = n;
    const u64 nvec = (n - head) / EPV;
    const u64 tail_start = head + nvec * EPV;
    const uint4 *vsrc = reinterpret_cast<const uint4 *>(keys + head);

    constexpr int UNROLL = 4;
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
                KeyT e[EPV];
                memcpy(e, &v[u], 16);
#pragma unroll
                for (int k = 0; k < EPV; ++k) count_key(e[k]);
            }
        }
    }
    if (blockIdx.x == 0) {
        if (tid < head) count_key(keys[tid]);
        const u64 t = tail_start + tid;
        if (t < n) count_key(keys[t]);
    }
    __syncthreads();
    const u32 top_flip = signed_or_float ? 0x80u : 0u;
    for (u32 i = tid; i < P * kRadix; i += THREADS) {
        const u32 c = sh[i];
        if (c) atomicAdd(&ghist[i ^ (i >= (u32)(P - 1) * kRadix ? top_flip : 0u)], (u64)c);
    }
}

// The same histogram with one copy of every bin per LANE (word bin*32 + lane lives in bank `lane`), so
// the shared-memory atomics of a warp never collide on a bank: one wavefront per instruction
// instead of the ~3 that 32 random bins cost. P * 32 KB of shared memory, used for keys of up to 4
// bytes; one persistent CTA per SM.
template <typename KeyT, int THREADS>
__global__ void __launch_bounds__(THREADS)
sort_histogram_lanes_kernel(const KeyT *__restrict__ keys, u64 n, u64 *ghist, int signed_or_float, int is_float) {
    constexpr int P = sizeof(KeyT);
    constexpr int EPV = 16 / sizeof(KeyT);
    static_assert(P <= 4, "P * 32 KB of counters must fit in shared memory");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    u32 *sh = reinterpret_cast<u32 *>(smem_raw);  // [P][256][32]
    const u32 tid = threadIdx.x, lane = tid & 31u;
    for (u32 i = tid; i < P * kRadix * 32; i += THREADS) sh[i] = 0;
    __syncthreads();

    // Raw bytes are counted (the sign flip of the top digit is applied to the bin index at the end).
    u32 *my = sh + lane;
    auto count_key = [&](KeyT k) {
        const KeyT b = is_float ? radix_bits<KeyT, sizeof(KeyT) >= 4>(k) : k;
#pragma unroll
        for (int p = 0; p < P; ++p) atomicAdd(&my[(p * kRadix + ((u32)(b >> (8 * p)) & 0xFFu)) * 32], 1u);
    };

    const u64 mis = ((uintptr_t)keys & 15u) / sizeof(KeyT);
    u64 head = mis ? (EPV - mis) : 0;
    if (head > n) head = n;
    const u64 nvec = (n - head) / EPV;
    const u64 tail_start = head + nvec * EPV;
    const uint4 *vsrc = reinterpret_cast<const uint4 *>(keys + head);

    constexpr int UNROLL = 4;
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
                KeyT e[EPV];
                memcpy(e, &v[u], 16);
#pragma unroll
                for (int k = 0; k < EPV; ++k) count_key(e[k]);
            }
        }
    }
    if (blockIdx.x == 0) {
        if (tid < head) count_key(keys[tid]);
        const u64 t = tail_start + tid;
        if (t < n) count_key(keys[t]);
    }
    __syncthreads();
    // bin i = sum of its 32 lane copies, read in a rotated order so that the 32 threads of a warp
    // (32 consecutive bins, 32 words apart) touch 32 different banks
    const u32 top_flip = signed_or_float ? 0x80u : 0u;
    for (u32 i = tid; i < P * kRadix; i += THREADS) {
        u32 c = 0;
#pragma unroll 8
        for (u32 j = 0; j < 32; ++j) c += sh[i * 32 + ((j + lane) & 31u)];
        if (c) atomicAdd(&ghist[i ^ (i >= (u32)(P - 1) * kRadix ? top_flip : 0u)], (u64)c);
    }
}

// Exclusive prefix over the 256 bins of each digit position, in place. One CTA of 256 threads per
// digit position.
__global__ void sort_scan_histogram_kernel(u64 *ghist);

// ---------------------------------------------------------------------------------------------
// One onesweep pass
// ---------------------------------------------------------------------------------------------
struct SortPassArgs {
    const void *keys_in;
    void *keys_out;
    const void *vals_in;
    void *vals_out;
    u64 n;
    u64 ntiles;
    const u64 *gexcl;  // [256] exclusive digit offsets of this pass
    u64 *desc;         // [ntiles][256]
    u32 *header;
    int pass;
    int shift;
    u32 top_xor;
    int signed_or_float;
    u32 spin_limit;    // polls before a look-back gives up
    u32 mute_tile;     // test hook: 1 + index of a tile that publishes nothing (0 = none)
};

// Shared memory of one CTA: the per-unit digit tables, per-digit bases, the staged tile.
__host__ __device__ constexpr size_t sort_smem_bytes(int threads, int items, int key_bytes, int val_bytes) {
    return (size_t)(threads / 16) * kRadix * 4 + (size_t)kRadix * 16 + (size_t)threads * items * (key_bytes + val_bytes) + 64;
}

template <typename KeyT, typename ValT, int THREADS, int ITEMS> struct SortSmem {
    static constexpr int UNITS = THREADS / 16;  // half-warps: the ranking units
    static constexpr int TILE = THREADS * ITEMS;
    static constexpr bool HAS_VAL = !std::is_same<ValT, void>::value;
    using ValS = typename std::conditional<HAS_VAL, ValT, char>::type;  // storage type (unused without values)
    static constexpr size_t kTbl = (size_t)UNITS * kRadix * 4;
    static constexpr size_t kGbase = (size_t)kRadix * 16;  // global bases (u64) + digit counts + digit starts (u32)
    static constexpr size_t kKeys = (size_t)TILE * sizeof(KeyT);
    static constexpr size_t kVals = HAS_VAL ? (size_t)TILE * sizeof(ValS) : 0;
    static constexpr size_t kBytes = sort_smem_bytes(THREADS, ITEMS, (int)sizeof(KeyT), HAS_VAL ? (int)sizeof(ValS) : 0);
    static_assert(kBytes == kTbl + kGbase + kKeys + kVals + 64, "layout and size formula disagree");
};

// The byte of the key that this pass sorts by, BEFORE the sign flip of the top digit (`top_xor`):
// per-key code works on this raw byte, and the per-digit code visits the table entries in the order
// of the true digit (entry = digit ^ top_xor), which costs nothing per key.
template <typename KeyT, bool IS_FLOAT> __device__ __forceinline__ u32 raw_digit(KeyT k, int shift) {
    const KeyT b = radix_bits<KeyT, IS_FLOAT>(k);
    if constexpr (sizeof(KeyT) == 8) return (u32)(b >> shift) & 0xFFu;
    else return __byte_perm((u32)b, 0u, 0x4440u + (u32)(shift >> 3));  // one PRMT: byte `shift/8`, zero-extended
}

// Returns its argument through an empty asm statement: the compiler then recomputes what derives
// from it (here: the table address of a key's digit) instead of keeping the first computation
// alive in a register across the whole ranking step.
template <typename KeyT> __device__ __forceinline__ KeyT opaque(KeyT k) {
    if constexpr (sizeof(KeyT) == 8) {
        asm volatile("" : "+l"(k));
        return k;
    } else {
        u32 v = (u32)k;
        asm volatile("" : "+r"(v));
        return (KeyT)v;
    }
}

template <typename KeyT, bool IS_FLOAT, typename ValT, int THREADS, int ITEMS>
__global__ void __launch_bounds__(THREADS, (THREADS <= 256 ? 3 : (THREADS <= 512 ? 2 : 1))) onesweep_kernel(SortPassArgs a) {
    using SM = SortSmem<KeyT, ValT, THREADS, ITEMS>;
    using ValS = typename SM::ValS;
    constexpr int UNITS = SM::UNITS;
    constexpr int TILE = SM::TILE;
    static_assert(THREADS >= kRadix && THREADS % 32 == 0, "one thread per digit is required");
    static_assert(TILE < 65536, "ranks and tile positions are kept in 16 bits");

    extern __shared__ __align__(16) unsigned char smem[];
    u64 *s_gbase = reinterpret_cast<u64 *>(smem);                              // [256] by table entry
    u32 *s_cnt = reinterpret_cast<u32 *>(smem + kRadix * 8);                   // [256] keys per digit (pads excluded)
    u32 *s_dexcl = s_cnt + kRadix;                                             // [256] start of each digit's run
    u32 *s_tbl = reinterpret_cast<u32 *>(smem + SM::kGbase);                   // [UNITS][256]
    KeyT *s_keys = reinterpret_cast<KeyT *>(smem + SM::kGbase + SM::kTbl);     // [TILE]
    ValS *s_vals = reinterpret_cast<ValS *>(smem + SM::kGbase + SM::kTbl + SM::kKeys);
    u32 *s_misc = reinterpret_cast<u32 *>(smem + SM::kGbase + SM::kTbl + SM::kKeys + SM::kVals);
    // s_misc[0..7]: warp sums of the digit scan; [8]: tile ticket; [10]: abort flag

    const u32 tid = threadIdx.x, lane = lane_id(), warp = tid >> 5;
    const u32 hl = lane & 15u, unit = tid >> 4;
    const KeyT *kin = static_cast<const KeyT *>(a.keys_in);
    KeyT *kout = static_cast<KeyT *>(a.keys_out);

    // The passes are launched with programmatic serialization: this grid may be resident before the
    // pass (or the bin scan) before it has finished, so nothing it wrote is touched before this point.
    grid_dep_wait();
    if (tid == 0) {
        const u32 t = atomicAdd(&a.header[kTicketBase + 1 + a.pass], 1u);
        s_misc[8] = t;
        s_misc[10] = ld_relaxed_u32(&a.header[kStatusWord]) != 0u;
    }
    {
        uint4 *z = reinterpret_cast<uint4 *>(s_tbl);
#pragma unroll
        for (int i = 0; i < UNITS * kRadix / 4 / THREADS; ++i) z[i * THREADS + tid] = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    const u64 tile = s_misc[8];
    if (tile >= a.ntiles) return;
    const u64 tag_agg = desc_tag(a.pass, kStAggregate), tag_pfx = desc_tag(a.pass, kStPrefix),
              tag_poison = desc_tag(a.pass, kStPoison);
    u64 *my_desc = a.desc + tile * kRadix;
    if (s_misc[10]) {  // an earlier tile failed: pass the poison on
        if (tid < kRadix) st_relaxed_u64(my_desc + tid, tag_poison);
        return;
    }
    if (a.mute_tile && tile + 1 == (u64)a.mute_tile) return;  // test hook: a tile that never publishes

    const u64 tile_start = tile * (u64)TILE;
    const u32 count = (u32)(a.n - tile_start < (u64)TILE ? a.n - tile_start : (u64)TILE);
    const bool full = count == (u32)TILE;
    const u32 unit_off = unit * 16 * ITEMS + hl;  // + i*16: element offset of item i in the tile

    // ---- 1. load keys (unit-striped: item i of lane hl of a unit is element unit_off + 16*i) -----
    KeyT key[ITEMS];
    if (full) {
        const KeyT *p = kin + tile_start + unit_off;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) key[i] = p[i * 16];
    } else {
        const KeyT pad = pad_key<KeyT, IS_FLOAT>(a.signed_or_float != 0);
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            const u32 off = unit_off + i * 16;
            key[i] = off < count ? kin[tile_start + off] : pad;
        }
    }

    grid_dep_launch();  // the next pass's CTAs may take the SM slots that this grid's last wave frees
    // ---- 2. rank each key within (unit, digit), in element order ---------------------------------
    // Word of the unit's table: {mask of the unit's lanes holding this digit in the current item : 16 |
    // keys of this digit in the unit's earlier items : 16}. Per item: (A) add my lane bit; warp barrier;
    // (B) read the word; warp barrier; (C) the highest lane of each group adds `group size - mask bits`.
    // A, C are atomic adds, which commute, so a fast lane's A of the next item may overtake a slow
    // group's C; every B sits between two warp barriers, after all A of its item and all C of the
    // item before, and before any C of its own item: it reads exactly {group mask | earlier count}.
    u32 *my_tbl = s_tbl + unit * kRadix;
    const u32 bit_hi = 1u << (16 + hl);
    const u32 lt16 = (1u << hl) - 1u;
    u32 rank2[(ITEMS + 1) / 2];  // two 16-bit ranks (later: tile positions) per register
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        u32 *slot = my_tbl + raw_digit<KeyT, IS_FLOAT>(key[i], a.shift);
        atomicAdd(slot, bit_hi);
        __syncwarp();
        const u32 w = *reinterpret_cast<volatile u32 *>(slot);
        __syncwarp();
        const u32 mask = w >> 16;
        if ((mask >> hl) == 1u) atomicAdd(slot, (u32)__popc(mask) - (mask << 16));
        const u32 r = (w & 0xFFFFu) + (u32)__popc(mask & lt16);
        if (i & 1) rank2[i / 2] |= r << 16;
        else rank2[i / 2] = r;
    }
    __syncthreads();

    // The look-back threads: one per digit. With 512 threads or more they are the second group of
    // 256 threads, which has nothing to do in steps 3 and 4, so the first round trip of the look-back
    // overlaps with those steps and with the scatter.
    constexpr bool LB_SPLIT = THREADS >= 2 * kRadix;
    const bool is_lb = LB_SPLIT ? (tid >= (u32)kRadix && tid < 2u * kRadix) : tid < (u32)kRadix;
    const u32 lb_digit = LB_SPLIT ? tid - kRadix : tid;
    constexpr int LB = 2;  // predecessor tiles read per round trip
    u64 lb_w[LB];
    auto lb_read = [&](long long t) {  // descriptors of tiles t, t-1, ... for my digit
#pragma unroll
        for (int k = 0; k < LB; ++k)
            lb_w[k] = t - k >= 0 ? ld_relaxed_u64(a.desc + (u64)(t - k) * kRadix + lb_digit) : tag_pfx;  // before tile 0: prefix 0
    };
    if (LB_SPLIT && is_lb && tile > 0) lb_read((long long)tile - 1);

    // ---- 3. per digit: count over the units, publish the tile aggregate -------------------------
    // Thread `tid` owns the digit `tid` (in sorted order), whose table entry is tid ^ top_xor.
    const u32 entry = (tid ^ a.top_xor) & 0xFFu;
    u32 cnt = 0;  // keys of digit `tid` in the tile, pads included
    if (tid < kRadix) {
#pragma unroll
        for (int u = 0; u < UNITS; ++u) cnt += s_tbl[u * kRadix + entry];
        u32 cnt_real = cnt;  // pads excluded (they all have digit 255)
        if (!full && tid == kRadix - 1) cnt_real = cnt - ((u32)TILE - count);
        st_relaxed_u64(my_desc + tid, (tile == 0 ? tag_pfx : tag_agg) | (u64)cnt_real);
        s_cnt[tid] = cnt_real;
    }
    if (!LB_SPLIT && is_lb && tile > 0) lb_read((long long)tile - 1);
    // ---- 4. exclusive scan of the digit counts: start of each digit's run in the sorted tile ----
    u32 incl = cnt;
    if (tid < kRadix) {
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const u32 up = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            incl += lane >= (u32)d ? up : 0u;
        }
        if (lane == 31) s_misc[warp] = incl;
    }
    __syncthreads();
    if (tid < kRadix) {
        u32 wbase = 0;
#pragma unroll
        for (int w = 0; w < kRadix / 32; ++w) wbase += w < (int)warp ? s_misc[w] : 0u;
        const u32 dexcl = wbase + incl - cnt;  // exclusive prefix of digit `tid` within the tile
        s_dexcl[tid] = dexcl;
        // Turn the per-unit counts into the position of each (unit, digit) group in the sorted tile.
        u32 run = dexcl;
#pragma unroll
        for (int u = 0; u < UNITS; ++u) {
            const u32 c = s_tbl[u * kRadix + entry];
            s_tbl[u * kRadix + entry] = run;
            run += c;
        }
    }
    __syncthreads();

    // ---- 5. scatter keys (and values) to their sorted position in shared memory -----------------
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const u32 pos = my_tbl[raw_digit<KeyT, IS_FLOAT>(opaque(key[i]), a.shift)] + ((i & 1) ? rank2[i / 2] >> 16 : rank2[i / 2] & 0xFFFFu);
        s_keys[pos] = key[i];
        if constexpr (SM::HAS_VAL) rank2[i / 2] = (i & 1) ? (rank2[i / 2] & 0xFFFFu) | (pos << 16) : (rank2[i / 2] & 0xFFFF0000u) | pos;
    }
    if constexpr (SM::HAS_VAL) {
        const ValS *vin = static_cast<const ValS *>(a.vals_in);
        ValS val[ITEMS];
        if (full) {
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) val[i] = (vin + tile_start + unit_off)[i * 16];
        } else {
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) {
                const u32 off = unit_off + i * 16;
                val[i] = off < count ? vin[tile_start + off] : (ValS)0;
            }
        }
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) s_vals[(i & 1) ? rank2[i / 2] >> 16 : rank2[i / 2] & 0xFFFFu] = val[i];
    }

    // ---- 6. look back: keys of my digit in all earlier tiles, LB tiles per round trip; the first
    //         round was read before the scatter ------------------------------------------------------
    if (is_lb) {
        u64 excl = 0;
        bool ok = true;
        if (tile > 0) {
            long long t = (long long)tile - 1;
            u32 spins = 0;
            bool done = false;
            while (!done) {
                int used = 0;
#pragma unroll
                for (int k = 0; k < LB; ++k) {
                    if (!done && used == k) {
                        const u64 w = lb_w[k];
                        const u64 tag = w & ~kCountMask;
                        if (tag == tag_pfx) {
                            excl += w & kCountMask;
                            done = true;
                        } else if (tag == tag_agg) {
                            excl += w & kCountMask;
                            used = k + 1;
                        } else if (tag == tag_poison) {
                            ok = false;
                            done = true;
                        }
                    }
                }
                if (done) break;
                t -= used;  // tile 0 always publishes a prefix, so t never passes below -LB
                if (used == 0) {
                    if (++spins > a.spin_limit) {
                        record_error(a.header, KF_ERR_TIMEOUT, (u32)tile);
                        ok = false;
                        break;
                    }
                    if (spins > 8) __nanosleep(spins > 64 ? 256 : 32);
                } else {
                    spins = 0;
                }
                lb_read(t);
            }
        }
        if (ok) {
            if (tile > 0) st_relaxed_u64(my_desc + lb_digit, tag_pfx | (excl + (u64)s_cnt[lb_digit]));
            // Global index of element idx of the sorted tile with digit d: gbase + idx.
            // keys only: the byte address of that element, so that the stream-out needs one multiply-add
            const u64 g0 = a.gexcl[lb_digit] + excl - (u64)s_dexcl[lb_digit];
            s_gbase[(lb_digit ^ a.top_xor) & 0xFFu] = SM::HAS_VAL ? g0 : (u64)(uintptr_t)kout + g0 * sizeof(KeyT);
        } else {
            st_relaxed_u64(my_desc + lb_digit, tag_poison);
            s_misc[10] = 1;
        }
    }
    __syncthreads();
    if (s_misc[10]) return;

    // ---- 7. stream the sorted tile out: consecutive threads write consecutive addresses within
    //         each digit's run ----------------------------------------------------------------
    // (32-bit element bases instead of 64-bit ones were tried for n < 2^32: slower, the saved shared
    // traffic is less than what the wider address arithmetic costs)
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const u32 idx = i * THREADS + tid;
        if (full || idx < count) {
            const KeyT k = s_keys[idx];
            const u32 d = raw_digit<KeyT, IS_FLOAT>(k, a.shift);
            if constexpr (SM::HAS_VAL) {
                const u64 o = s_gbase[d] + idx;
                kout[o] = k;
                static_cast<ValS *>(a.vals_out)[o] = s_vals[idx];
            } else {
                *reinterpret_cast<KeyT *>(s_gbase[d] + (u64)idx * sizeof(KeyT)) = k;
            }
        }
    }
}

// ---- host side ---------------------------------------------------------------------------------
struct SortVariant {
    int threads, items;
};
static const SortVariant kSortVariants[] = {{256, 16}, {512, 16}, {512, 24}, {384, 24}};
constexpr int kNumSortVariants = 4;

template <typename KeyT, bool IS_FLOAT, typename ValT, int THREADS, int ITEMS>
int onesweep_launch_one(const SortPassArgs &a, cudaStream_t s) {
    using SM = SortSmem<KeyT, ValT, THREADS, ITEMS>;
    auto kern = onesweep_kernel<KeyT, IS_FLOAT, ValT, THREADS, ITEMS>;
    if (SM::kBytes > 227 * 1024) return KF_ERR_UNSUPPORTED;
    KF_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SM::kBytes));
    KF_CUDA_TRY(launch_chained(kern, (unsigned)a.ntiles, THREADS, SM::kBytes, s, a));
    note_launch();
    return KF_OK;
}

template <typename KeyT, bool IS_FLOAT, typename ValT>
int onesweep_launch(int variant, const SortPassArgs &a, cudaStream_t s) {
    switch (variant) {
    case 0: return onesweep_launch_one<KeyT, IS_FLOAT, ValT, 256, 16>(a, s);
    case 1: return onesweep_launch_one<KeyT, IS_FLOAT, ValT, 512, 16>(a, s);
    case 2: return onesweep_launch_one<KeyT, IS_FLOAT, ValT, 512, 24>(a, s);
    case 3: return onesweep_launch_one<KeyT, IS_FLOAT, ValT, 384, 24>(a, s);
    default: return KF_ERR_UNSUPPORTED;
    }
}

template <typename KeyT, bool IS_FLOAT>
int histogram_launch(const void *keys, u64 n, u64 *ghist, int signed_or_float, cudaStream_t s) {
    const int sms = device_sm_count();
    if constexpr (sizeof(KeyT) <= 4) {
        // lane-private bins: one persistent CTA per SM, P * 32 KB of shared memory
        constexpr int THREADS = 1024;
        constexpr size_t kSmem = sizeof(KeyT) * kRadix * 32 * 4;
        if (n * sizeof(KeyT) >= (8u << 20)) {
            auto kern = sort_histogram_lanes_kernel<KeyT, THREADS>;
            KF_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem));
            kern<<<(unsigned)sms, THREADS, kSmem, s>>>(static_cast<const KeyT *>(keys), n, ghist, signed_or_float, IS_FLOAT ? 1 : 0); note_launch();
            KF_CUDA_TRY(cudaGetLastError());
            return KF_OK;
        }
    }
    constexpr int THREADS = 512;
    u64 blocks = (u64)sms * 4;
    const u64 need = (n * sizeof(KeyT) + (u64)THREADS * 64 - 1) / ((u64)THREADS * 64);
    if (blocks > need) blocks = need < 1 ? 1 : need;
    sort_histogram_kernel<KeyT, IS_FLOAT, THREADS><<<(unsigned)blocks, THREADS, 0, s>>>(
        static_cast<const KeyT *>(keys), n, ghist, signed_or_float); note_launch();
    KF_CUDA_TRY(cudaGetLastError());
    return KF_OK;
}

// Per key width, defined in sort_inst_*.cu. val_bytes in {0, 4, 8}.
int sort_pass_k32(bool is_float, int val_bytes, int variant, const SortPassArgs &a, cudaStream_t s);
int sort_pass_k64(bool is_float, int val_bytes, int variant, const SortPassArgs &a, cudaStream_t s);
int sort_hist_k32(bool is_float, const void *keys, u64 n, u64 *ghist, int sof, cudaStream_t s);
int sort_hist_k64(bool is_float, const void *keys, u64 n, u64 *ghist, int sof, cudaStream_t s);
// 8- and 16-bit keys are integers only.
int sort_pass_k8(int val_bytes, int variant, const SortPassArgs &a, cudaStream_t s);
int sort_pass_k16(int val_bytes, int variant, const SortPassArgs &a, cudaStream_t s);
int sort_hist_k8(const void *keys, u64 n, u64 *ghist, int sof, cudaStream_t s);
int sort_hist_k16(const void *keys, u64 n, u64 *ghist, int sof, cudaStream_t s);

#define KF_SORT_INSTANTIATE(NAME, KeyT)                                                               \
    namespace kf {                                                                                    \
    int sort_pass_##NAME(bool is_float, int val_bytes, int variant, const SortPassArgs &a,            \
                         cudaStream_t s) {                                                            \
        if (is_float) {                                                                               \
            if (val_bytes == 0) return onesweep_launch<KeyT, true, void>(variant, a, s);              \
            if (val_bytes == 4) return onesweep_launch<KeyT, true, uint32_t>(variant, a, s);          \
            if (val_bytes == 8) return onesweep_launch<KeyT, true, u64>(variant, a, s);               \
        } else {                                                                                      \
            if (val_bytes == 0) return onesweep_launch<KeyT, false, void>(variant, a, s);             \
            if (val_bytes == 4) return onesweep_launch<KeyT, false, uint32_t>(variant, a, s);         \
            if (val_bytes == 8) return onesweep_launch<KeyT, false, u64>(variant, a, s);              \
        }                                                                                             \
        return KF_ERR_UNSUPPORTED;                                                                    \
    }                                                                                                 \
    int sort_hist_##NAME(bool is_float, const void *keys, u64 n, u64 *ghist, int sof, cudaStream_t s) { \
        return is_float ? histogram_launch<KeyT, true>(keys, n, ghist, sof, s)                        \
                        : histogram_launch<KeyT, false>(keys, n, ghist, sof, s);                      \
    }                                                                                                 \
    }

#define KF_SORT_INSTANTIATE_INT(NAME, KeyT)                                                           \
    namespace kf {                                                                                    \
    int sort_pass_##NAME(int val_bytes, int variant, const SortPassArgs &a, cudaStream_t s) {         \
        if (val_bytes == 0) return onesweep_launch<KeyT, false, void>(variant, a, s);                 \
        if (val_bytes == 4) return onesweep_launch<KeyT, false, uint32_t>(variant, a, s);             \
        if (val_bytes == 8) return onesweep_launch<KeyT, false, u64>(variant, a, s);                  \
        return KF_ERR_UNSUPPORTED;                                                                    \
    }                                                                                                 \
    int sort_hist_##NAME(const void *keys, u64 n, u64 *ghist, int sof, cudaStream_t s) {              \
        return histogram_launch<KeyT, false>(keys, n, ghist, sof, s);                                 \
    }                                                                                                 \
    }

}  // namespace kf
