/*
 * kf_oracle.c — CPU oracle and CPU baseline for the mapreduce / scan / sort path.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the product path (kernelforge.jl_b200/) loads or calls this
 * file; it is used by tests/, by the smoke check and by the CPU-baseline leg of bench.py.
 *
 * The reference (KernelForge.jl) is Julia and cannot run on this machine, and its tests hold no
 * stored golden vectors for this path: every expectation is computed at test time by Julia `Base`
 * on the host (test/tests/mapreduce/mapreduce1d_test.jl:14-29, test/tests/scan/scan_test.jl:35-125,
 * test/tests/sort/sort_test.jl:15-38, test/tests/sort/sort_keyval_test.jl:15-38). This file restates
 * those `Base` semantics in plain C:
 *
 *   kfo_*  — the ORACLE: float reductions and scans as a Float64 sequential left fold (what the
 *            tolerance of the parity tests is measured against); integers in the element type
 *            with wrap-around (Julia `+`/`*` on machine integers); sort = stable sort by the
 *            reference's order-preserving unsigned key map (src/sort/uint_map.jl:11-35), which
 *            equals `Base.sort` / `sortperm` under `isless` for every non-NaN input.
 *   kfb_*  — the timed CPU BASELINE: the same operations computed the way `Base.mapreduce`
 *            (pairwise, 1024-element leaves), `Base.accumulate` (sequential, element type) and
 *            `Base.sort!` (LSD radix for machine keys) do, with optional OpenMP threads.
 *
 * Pins: the closed-form cases of the reference's tests (sum(1:n); adversarial and boundary sort
 * arrays) and an independent numpy restatement; see tests/test_oracle.py. The affine-composition
 * scan has no counterpart in the reference's tests: for it, parity is unpinned on the reference
 * side and defined by the Float64 left fold alone.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* enums shared with include/kf_b200.h */
enum { U8 = 0, I8, U16, I16, U32, I32, U64, I64, F32, F64 };
enum { MAP_IDENTITY = 0, MAP_ABS2, MAP_ABS };
enum { OP_ADD = 0, OP_MUL, OP_MIN, OP_MAX, OP_AND, OP_OR, OP_XOR };

static int dtype_bytes(int d) {
    switch (d) {
    case U8: case I8: return 1;
    case U16: case I16: return 2;
    case U32: case I32: case F32: return 4;
    default: return 8;
    }
}
static int dtype_signed(int d) { return d == I8 || d == I16 || d == I32 || d == I64; }

int kfo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---------------------------------------------------------------------------------------------
 * Float oracle: Float64 left fold. mapreduce1d_kernel.jl:1-3 fixes the type flow T -> f -> op -> g;
 * scan.jl:33-36 fixes "f before, inclusive".
 * ------------------------------------------------------------------------------------------- */
static double fmap(int f, double x) { return f == MAP_ABS2 ? x * x : (f == MAP_ABS ? fabs(x) : x); }
static double fop(int op, double l, double r) {
    switch (op) {
    case OP_ADD: return l + r;
    case OP_MUL: return l * r;
    case OP_MIN: return r < l ? r : l;
    default: return l < r ? r : l;
    }
}

double kfo_mapreduce_f32(int f, int op, const float *x, size_t n) {
    double acc = fmap(f, (double)x[0]);
    for (size_t i = 1; i < n; ++i) acc = fop(op, acc, fmap(f, (double)x[i]));
    return acc;
}
double kfo_mapreduce_f64(int f, int op, const double *x, size_t n) {
    double acc = fmap(f, x[0]);
    for (size_t i = 1; i < n; ++i) acc = fop(op, acc, fmap(f, x[i]));
    return acc;
}
void kfo_scan_f32(int f, int op, const float *x, size_t n, const double *init, double *out) {
    if (n == 0) return;
    double acc = fmap(f, (double)x[0]);
    if (init) acc = fop(op, *init, acc);
    out[0] = acc;
    for (size_t i = 1; i < n; ++i) out[i] = acc = fop(op, acc, fmap(f, (double)x[i]));
}
void kfo_scan_f64(int f, int op, const double *x, size_t n, const double *init, double *out) {
    if (n == 0) return;
    double acc = fmap(f, x[0]);
    if (init) acc = fop(op, *init, acc);
    out[0] = acc;
    for (size_t i = 1; i < n; ++i) out[i] = acc = fop(op, acc, fmap(f, x[i]));
}
/* Affine composition (a1,b1) o (a2,b2) = (a1*a2, a2*b1 + b2), sequential left fold in Float64. */
void kfo_scan_affine(const float *a, const float *b, size_t n, const double *init_ab, double *oa, double *ob) {
    double A = 1.0, B = 0.0;
    if (init_ab) {
        A = init_ab[0];
        B = init_ab[1];
    }
    for (size_t i = 0; i < n; ++i) {
        const double ai = (double)a[i], bi = (double)b[i];
        B = ai * B + bi;
        A = A * ai;
        oa[i] = A;
        ob[i] = B;
    }
}

/* accumulate(*, src) over quaternions (w, x, y, z), the Hamilton product as Quaternions.jl defines
 * `*` (the reference's non-commutative scan test, test/tests/scan/scan_test.jl:22-33, compares with
 * exactly this left fold on the host). Components are read as Float32 or Float64; the fold runs in
 * Float64. init4 (one quaternion) seeds the fold from the left, or is NULL. */
void kfo_scan_quat(const void *src, int is_f64, size_t n, const double *init4, double *out) {
    double w = 1.0, x = 0.0, y = 0.0, z = 0.0;
    if (init4) {
        w = init4[0];
        x = init4[1];
        y = init4[2];
        z = init4[3];
    }
    for (size_t i = 0; i < n; ++i) {
        double r[4];
        for (int k = 0; k < 4; ++k)
            r[k] = is_f64 ? ((const double *)src)[4 * i + k] : (double)((const float *)src)[4 * i + k];
        if (i == 0 && !init4) {
            w = r[0];
            x = r[1];
            y = r[2];
            z = r[3];
        } else {
            const double nw = w * r[0] - x * r[1] - y * r[2] - z * r[3];
            const double nx = w * r[1] + x * r[0] + y * r[3] - z * r[2];
            const double ny = w * r[2] - x * r[3] + y * r[0] + z * r[1];
            const double nz = w * r[3] + x * r[2] - y * r[1] + z * r[0];
            w = nw;
            x = nx;
            y = ny;
            z = nz;
        }
        out[4 * i + 0] = w;
        out[4 * i + 1] = x;
        out[4 * i + 2] = y;
        out[4 * i + 3] = z;
    }
}

/* ---------------------------------------------------------------------------------------------
 * Integer oracle: arithmetic in the element type with wrap-around. Values travel as 64-bit
 * containers and are truncated to the element width after every step.
 * ------------------------------------------------------------------------------------------- */
static int64_t load_int(int dtype, const void *p, size_t i) {
    switch (dtype) {
    case U8: return ((const uint8_t *)p)[i];
    case I8: return ((const int8_t *)p)[i];
    case U16: return ((const uint16_t *)p)[i];
    case I16: return ((const int16_t *)p)[i];
    case U32: return ((const uint32_t *)p)[i];
    case I32: return ((const int32_t *)p)[i];
    case U64: return (int64_t)((const uint64_t *)p)[i];
    default: return ((const int64_t *)p)[i];
    }
}
static void store_int(int dtype, void *p, size_t i, int64_t v) {
    switch (dtype) {
    case U8: case I8: ((uint8_t *)p)[i] = (uint8_t)v; break;
    case U16: case I16: ((uint16_t *)p)[i] = (uint16_t)v; break;
    case U32: case I32: ((uint32_t *)p)[i] = (uint32_t)v; break;
    default: ((uint64_t *)p)[i] = (uint64_t)v; break;
    }
}
/* truncate to the element width, then sign- or zero-extend back to the container */
static int64_t wrap_int(int dtype, int64_t v) {
    switch (dtype) {
    case U8: return (uint8_t)v;
    case I8: return (int8_t)v;
    case U16: return (uint16_t)v;
    case I16: return (int16_t)v;
    case U32: return (uint32_t)v;
    case I32: return (int32_t)v;
    default: return v;
    }
}
static int64_t imap(int dtype, int f, int64_t x) {
    if (f == MAP_ABS2) return wrap_int(dtype, (int64_t)((uint64_t)x * (uint64_t)x));
    if (f == MAP_ABS) return dtype_signed(dtype) && x < 0 ? wrap_int(dtype, (int64_t)(0 - (uint64_t)x)) : x;
    return x;
}
static int64_t iop(int dtype, int op, int64_t l, int64_t r) {
    const int u64cmp = dtype == U64;
    switch (op) {
    case OP_ADD: return wrap_int(dtype, (int64_t)((uint64_t)l + (uint64_t)r));
    case OP_MUL: return wrap_int(dtype, (int64_t)((uint64_t)l * (uint64_t)r));
    case OP_MIN: return u64cmp ? ((uint64_t)r < (uint64_t)l ? r : l) : (r < l ? r : l);
    case OP_MAX: return u64cmp ? ((uint64_t)l < (uint64_t)r ? r : l) : (l < r ? r : l);
    case OP_AND: return l & r;
    case OP_OR: return l | r;
    default: return wrap_int(dtype, l ^ r);
    }
}
int64_t kfo_mapreduce_int(int f, int op, int dtype, const void *x, size_t n) {
    int64_t acc = imap(dtype, f, load_int(dtype, x, 0));
    for (size_t i = 1; i < n; ++i) acc = iop(dtype, op, acc, imap(dtype, f, load_int(dtype, x, i)));
    return acc;
}
void kfo_scan_int(int f, int op, int dtype, const void *x, size_t n, const void *init, void *out) {
    if (n == 0) return;
    int64_t acc = imap(dtype, f, load_int(dtype, x, 0));
    if (init) acc = iop(dtype, op, load_int(dtype, init, 0), acc);
    store_int(dtype, out, 0, acc);
    for (size_t i = 1; i < n; ++i) {
        acc = iop(dtype, op, acc, imap(dtype, f, load_int(dtype, x, i)));
        store_int(dtype, out, i, acc);
    }
}

/* ---------------------------------------------------------------------------------------------
 * Sort oracle: stable ascending sort by the unsigned image of the key (uint_map.jl:11-35):
 *   unsigned -> identity; signed -> bits ^ sign bit; float -> (sign clear ? bits | sign : ~bits).
 * Implemented as an LSD radix sort of (mapped key, original index) pairs, which is stable by
 * construction; `perm[j]` is the index of the element that lands at position j.
 * ------------------------------------------------------------------------------------------- */
uint64_t kfo_uint_map(int dtype, uint64_t bits) {
    switch (dtype) {
    case I8: return (bits ^ 0x80u) & 0xFFu;
    case I16: return (bits ^ 0x8000u) & 0xFFFFu;
    case I32: return (bits ^ 0x80000000u) & 0xFFFFFFFFu;
    case I64: return bits ^ 0x8000000000000000ull;
    case F32: {
        uint32_t u = (uint32_t)bits;
        return (u & 0x80000000u) ? (uint32_t)~u : (u | 0x80000000u);
    }
    case F64: return (bits & 0x8000000000000000ull) ? ~bits : (bits | 0x8000000000000000ull);
    default: return bits;
    }
}
static uint64_t load_bits(int dtype, const void *p, size_t i) {
    switch (dtype_bytes(dtype)) {
    case 1: return ((const uint8_t *)p)[i];
    case 2: return ((const uint16_t *)p)[i];
    case 4: return ((const uint32_t *)p)[i];
    default: return ((const uint64_t *)p)[i];
    }
}
int kfo_sort_perm(int key_dtype, const void *keys, size_t n, uint64_t *perm) {
    const int P = dtype_bytes(key_dtype);
    uint64_t *k0 = (uint64_t *)malloc(n * 8), *k1 = (uint64_t *)malloc(n * 8), *p1 = (uint64_t *)malloc(n * 8);
    if (n && (!k0 || !k1 || !p1)) {
        free(k0); free(k1); free(p1);
        return -1;
    }
    uint64_t *p0 = perm;
    for (size_t i = 0; i < n; ++i) {
        k0[i] = kfo_uint_map(key_dtype, load_bits(key_dtype, keys, i));
        p0[i] = i;
    }
    for (int pass = 0; pass < P; ++pass) {
        size_t count[257] = {0};
        const int sh = 8 * pass;
        for (size_t i = 0; i < n; ++i) count[((k0[i] >> sh) & 0xFF) + 1]++;
        for (int d = 0; d < 256; ++d) count[d + 1] += count[d];
        for (size_t i = 0; i < n; ++i) {
            const size_t o = count[(k0[i] >> sh) & 0xFF]++;
            k1[o] = k0[i];
            p1[o] = p0[i];
        }
        uint64_t *t = k0; k0 = k1; k1 = t;
        t = p0; p0 = p1; p1 = t;
    }
    if (p0 != perm) memcpy(perm, p0, n * 8);
    free(k0); free(k1);
    free(p0 == perm ? p1 : p0);
    return 0;
}
/* out[j] = in[perm[j]] for elements of `bytes` width */
void kfo_gather(const void *in, const uint64_t *perm, size_t n, int bytes, void *out) {
    for (size_t j = 0; j < n; ++j) memcpy((char *)out + j * bytes, (const char *)in + perm[j] * bytes, bytes);
}

/* ---------------------------------------------------------------------------------------------
 * CPU baseline (timed): the way Julia Base computes the same calls.
 * ------------------------------------------------------------------------------------------- */
static float bmap(int f, float x) { return f == MAP_ABS2 ? x * x : (f == MAP_ABS ? fabsf(x) : x); }
/* Base.mapreduce_impl: pairwise reduction with sequential leaves of 1024 elements. */
static float pairwise_sum_f32(int f, const float *x, size_t lo, size_t hi) {
    if (hi - lo <= 1024) {
        float v = bmap(f, x[lo]);
        for (size_t i = lo + 1; i < hi; ++i) v += bmap(f, x[i]);
        return v;
    }
    const size_t mid = lo + (hi - lo) / 2;
    return pairwise_sum_f32(f, x, lo, mid) + pairwise_sum_f32(f, x, mid, hi);
}
float kfb_mapreduce_add_f32(int f, const float *x, size_t n, int threads) {
    if (threads <= 1) return pairwise_sum_f32(f, x, 0, n);
    float total = 0.0f;
#ifdef _OPENMP
    float *part = (float *)calloc((size_t)threads, sizeof(float));
#pragma omp parallel num_threads(threads)
    {
        const int t = omp_get_thread_num(), nt = omp_get_num_threads();
        const size_t lo = n * (size_t)t / nt, hi = n * (size_t)(t + 1) / nt;
        if (hi > lo) part[t] = pairwise_sum_f32(f, x, lo, hi);
    }
    for (int t = 0; t < threads; ++t) total += part[t];
    free(part);
#endif
    return total;
}

/* Base.accumulate(+, x): sequential, element type. Threads > 1: chunked two-sweep scan. */
#define DEF_ACCUMULATE(NAME, T)                                                              \
    void NAME(const T *x, size_t n, T *out, int threads) {                                   \
        if (n == 0) return;                                                                  \
        if (threads <= 1) {                                                                  \
            T acc = x[0];                                                                    \
            out[0] = acc;                                                                    \
            for (size_t i = 1; i < n; ++i) out[i] = acc = (T)(acc + x[i]);                   \
            return;                                                                          \
        }                                                                                    \
        T *tot = (T *)calloc((size_t)threads + 1, sizeof(T));                                \
        _Pragma("omp parallel num_threads(threads)") {                                       \
            int t = 0, nt = 1;                                                               \
            OMP_IDS(t, nt);                                                                  \
            const size_t lo = n * (size_t)t / nt, hi = n * (size_t)(t + 1) / nt;             \
            T acc = 0;                                                                       \
            for (size_t i = lo; i < hi; ++i) out[i] = acc = (T)(acc + x[i]);                 \
            tot[t + 1] = acc;                                                                \
            _Pragma("omp barrier")                                                           \
            _Pragma("omp single") {                                                          \
                for (int k = 1; k <= nt; ++k) tot[k] = (T)(tot[k] + tot[k - 1]);             \
            }                                                                                \
            const T carry = tot[t];                                                          \
            if (t > 0)                                                                       \
                for (size_t i = lo; i < hi; ++i) out[i] = (T)(carry + out[i]);               \
        }                                                                                    \
        free(tot);                                                                           \
    }
#ifdef _OPENMP
#define OMP_IDS(t, nt) do { t = omp_get_thread_num(); nt = omp_get_num_threads(); } while (0)
#else
#define OMP_IDS(t, nt) do { } while (0)
#endif
DEF_ACCUMULATE(kfb_accumulate_f32, float)
DEF_ACCUMULATE(kfb_accumulate_u32, uint32_t)

/* accumulate(op, pairs) for the affine composition, Float32 arithmetic, sequential. */
void kfb_accumulate_affine_f32(const float *a, const float *b, size_t n, float *oa, float *ob) {
    float A = 1.0f, B = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        B = a[i] * B + b[i];
        A = A * a[i];
        oa[i] = A;
        ob[i] = B;
    }
}

/* Base.sort! on machine keys: LSD radix, 8-bit digits. keys are sorted by their mapped image and
 * written back as original bits. vals (4-byte payload) may be NULL. Threads > 1: per-thread
 * histograms, stable. `tmp_k` / `tmp_v` are n-element scratch arrays. */
void kfb_sort_k32(int key_dtype, uint32_t *keys, uint32_t *vals, size_t n, uint32_t *tmp_k, uint32_t *tmp_v,
                  int threads) {
    if (threads < 1) threads = 1;
    const int has_v = vals != NULL;
#pragma omp parallel for num_threads(threads)
    for (size_t i = 0; i < n; ++i) keys[i] = (uint32_t)kfo_uint_map(key_dtype, keys[i]);
    size_t *hist = (size_t *)malloc((size_t)threads * 256 * sizeof(size_t));
    uint32_t *src_k = keys, *dst_k = tmp_k, *src_v = vals, *dst_v = tmp_v;
    for (int pass = 0; pass < 4; ++pass) {
        const int sh = 8 * pass;
        memset(hist, 0, (size_t)threads * 256 * sizeof(size_t));
#pragma omp parallel num_threads(threads)
        {
            int t = 0, nt = 1;
            OMP_IDS(t, nt);
            const size_t lo = n * (size_t)t / nt, hi = n * (size_t)(t + 1) / nt;
            size_t *h = hist + (size_t)t * 256;
            for (size_t i = lo; i < hi; ++i) h[(src_k[i] >> sh) & 0xFF]++;
#pragma omp barrier
#pragma omp single
            {
                size_t run = 0;
                for (int d = 0; d < 256; ++d)
                    for (int k = 0; k < nt; ++k) {
                        const size_t c = hist[(size_t)k * 256 + d];
                        hist[(size_t)k * 256 + d] = run;
                        run += c;
                    }
            }
            if (has_v) {
                for (size_t i = lo; i < hi; ++i) {
                    const size_t o = h[(src_k[i] >> sh) & 0xFF]++;
                    dst_k[o] = src_k[i];
                    dst_v[o] = src_v[i];
                }
            } else {
                for (size_t i = lo; i < hi; ++i) dst_k[h[(src_k[i] >> sh) & 0xFF]++] = src_k[i];
            }
        }
        uint32_t *t = src_k; src_k = dst_k; dst_k = t;
        t = src_v; src_v = dst_v; dst_v = t;
    }
    free(hist);
    /* four passes: the result is back in keys/vals; undo the key map */
#pragma omp parallel for num_threads(threads)
    for (size_t i = 0; i < n; ++i) {
        uint32_t u = keys[i];
        switch (key_dtype) {
        case I32: u ^= 0x80000000u; break;
        case F32: u = (u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u; break;
        default: break;
        }
        keys[i] = u;
    }
}
