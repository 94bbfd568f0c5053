/*
 * kf_b200.h — C ABI of libkf_b200.so: hand-written sm_100a kernels for the memory-bound
 * primitive core of KernelForge.jl (full mapreduce, inclusive scan, radix onesweep sort).
 *
 * Conventions shared by every entry point
 *   - All data pointers are DEVICE pointers, element-aligned only (views are fine).
 *   - The library never allocates or frees device memory: the caller passes a workspace
 *     (`ws`, `ws_bytes`) sized by the matching `*_workspace_bytes` query. A workspace can be
 *     reused across calls on the same stream; the callee re-initialises what it needs.
 *   - Every entry point is asynchronous on `stream` and returns a `kf_status` (0 = OK) for
 *     errors the host can see. Errors the device detects (a bounded wait that ran out) land in
 *     a status word inside the workspace and are read back by `kf_check`.
 *   - `cfg == NULL` selects the launch parameters from the built-in B200 launch table.
 *   - Indices are 0-based. Sizes are element counts (`uint64_t`).
 *
 * Each declaration cites the reference interface (file:line inside KernelForge.jl v0.2.0) that it
 * replaces.
 */
#ifndef KF_B200_H
#define KF_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KF_B200_ABI_VERSION 2

/* CUDA stream handle (a `cudaStream_t` / `CUstream`); NULL = the legacy default stream. */
typedef struct CUstream_st *kf_stream_t;

typedef enum kf_status {
    KF_OK = 0,
    KF_ERR_INVALID_ARG = 1,        /* null pointer, bad enum, length mismatch */
    KF_ERR_UNSUPPORTED = 2,        /* (f, op, dtype) or launch override outside the compiled set */
    KF_ERR_WORKSPACE_TOO_SMALL = 3,
    KF_ERR_LAUNCH_FAILED = 4,      /* a CUDA runtime call failed; see kf_last_cuda_error() */
    KF_ERR_TIMEOUT = 5,            /* a bounded device-side wait ran out (reported by kf_check) */
    KF_ERR_EMPTY_REDUCTION = 6,    /* mapreduce over n == 0 has no value (no init element) */
    KF_ERR_EXCEEDS_STATIC_SCRATCH = 7 /* kf_scan_static: the input needs more than KF_SCAN_STATIC_SCRATCH_BYTES */
} kf_status;

/* Element types: the reference's BitwiseTypes (src/KernelForge.jl:15) without Float16. */
typedef enum kf_dtype {
    KF_U8 = 0, KF_I8 = 1, KF_U16 = 2, KF_I16 = 3, KF_U32 = 4, KF_I32 = 5,
    KF_U64 = 6, KF_I64 = 7, KF_F32 = 8, KF_F64 = 9
} kf_dtype;

/* Element-wise map `f` applied on load (closures the Julia layer recognises by identity). */
typedef enum kf_map {
    KF_MAP_IDENTITY = 0,
    KF_MAP_ABS2 = 1,               /* x*x */
    KF_MAP_ABS = 2
} kf_map;

/* Maps over several arrays at once (the tuple form mapreduce(f, op, (x, y, ...))): what the
 * reference's tests pass as closures (test/tests/mapreduce/mapreduce1d_test.jl:106-194). */
typedef enum kf_mapn {
    KF_MAPN_PROD = 0,              /* x1*x2*...*xk   (k = 2: dot product)        k in 2..4 */
    KF_MAPN_SQDIFF = 1,            /* (x1 - x2)^2    (squared distance)          k = 2 */
    KF_MAPN_WSQ = 2                /* x1 * x2 * x2   (weighted sum of squares)   k = 2 */
} kf_mapn;

/* Binary operator `op`. KF_OP_AFFINE is the non-commutative composition of affine maps
 * (a1,b1) o (a2,b2) = (a1*a2, a2*b1 + b2), i.e. "apply the left map, then the right one". */
typedef enum kf_op {
    KF_OP_ADD = 0, KF_OP_MUL = 1, KF_OP_MIN = 2, KF_OP_MAX = 3,
    KF_OP_AND = 4, KF_OP_OR = 5, KF_OP_XOR = 6,
    KF_OP_AFFINE = 7
} kf_op;

/* Post-map `g`: applied once to the final value (mapreduce) and to every output element (scan). */
typedef enum kf_post {
    KF_POST_IDENTITY = 0,
    KF_POST_SQRT = 1
} kf_post;

/* Primitive ids for the launch table. */
typedef enum kf_primitive {
    KF_PRIM_MAPREDUCE = 0,
    KF_PRIM_SCAN = 1,
    KF_PRIM_SORT_KEYS = 2,
    KF_PRIM_SORT_PAIRS = 3
} kf_primitive;

/*
 * Optional launch override; replaces the reference's per-call kwargs `workgroup`, `Nitem`,
 * `blocks` (src/mapreduce/1D/mapreduce1d.jl:186-196, src/scan/scan.jl:261-271,
 * src/sort/sort1d.jl:337-347). A field left 0 is taken from the launch table. Only the
 * compiled (threads, items) pairs are accepted; anything else returns KF_ERR_UNSUPPORTED.
 *   threads : CTA size.
 *   items   : mapreduce/scan: 16-byte vectors per thread per tile; sort: keys per thread.
 *   blocks  : mapreduce only: number of persistent CTAs.
 */
typedef struct kf_launch_cfg {
    int32_t threads;
    int32_t items;
    int32_t blocks;
    int32_t reserved;  /* 0. Tests set it to make a bounded device-side wait run out on purpose: bits 0..15 =
                        * polls before a look-back gives up (0 = the default, about a second), bits 16..31 =
                        * 1 + index of one tile that stays silent. The call then returns normally and kf_check
                        * reports KF_ERR_TIMEOUT; nothing faults or hangs. */
} kf_launch_cfg;

/* ---- library / errors ---------------------------------------------------------------------- */

/* ABI version of the loaded library (== KF_B200_ABI_VERSION it was built with). */
int32_t kf_abi_version(void);

/* Human-readable text for a kf_status. Replaces the reference's Julia exceptions
 * (e.g. src/sort/sort1d.jl:348-349,367-389). */
const char *kf_error_string(int32_t status);

/* The CUDA runtime error code behind the calling thread's last KF_ERR_LAUNCH_FAILED (0 if none).
 * No counterpart in the reference (CUDA.jl raises its own exceptions). */
int32_t kf_last_cuda_error(void);

/* Reads the device-side status word of a workspace after synchronising `stream`.
 * Returns KF_OK or the error a kernel recorded (KF_ERR_TIMEOUT). The reference has no
 * counterpart: its look-back spins are unbounded (src/scan/scan_kernel.jl:388-415). */
int32_t kf_check(const void *ws, kf_stream_t stream);

/* The launch table entry for (primitive, element size in bytes, n). Replaces the generated
 * `default_*` overrides loaded by src/tuning/loader.jl:93-130 from data/tuning/<Arch>_inline.jl. */
int32_t kf_launch_table_lookup(int32_t primitive, int32_t elem_bytes, uint64_t n, kf_launch_cfg *out);

/* Kernels this library has launched in the calling process so far (all threads, all devices; memsets
 * and copies issued through the CUDA runtime are not kernels of the library and are not counted).
 * A benchmark reads it before and after its timed region. It has no counterpart in the reference. */
uint64_t kf_launch_count(void);

/* Number of SMs of the current device. Replaces `num_sms` (ext/KernelForgeCUDAExt.jl:31-33). */
int32_t kf_num_sms(void);

/* ---- mapreduce ----------------------------------------------------------------------------- */

/* Workspace for kf_mapreduce. Replaces get_allocation(MapReduce1D, ...)
 * (src/mapreduce/1D/mapreduce1d.jl:140-170): per-CTA partials + a completion counter. */
size_t kf_mapreduce_workspace_bytes(int32_t dtype, uint64_t n, const kf_launch_cfg *cfg);

/* dst[0] = g(op-reduce_i f(src[i])), i in [0, n). `op` must be associative and commutative
 * (KF_OP_AFFINE is rejected). Accumulates in the element type, like the reference
 * (H = promote_op(f, T), src/mapreduce/1D/mapreduce1d_kernel.jl:1-3). One kernel launch; the
 * last CTA to finish folds the per-CTA partials in index order, so the result is
 * deterministic for a given launch configuration.
 * Replaces mapreduce1d! / _mapreduce1d_impl! (src/mapreduce/1D/mapreduce1d.jl:259-346) and
 * mapreduce1d_kernel! (src/mapreduce/1D/mapreduce1d_kernel.jl:5-94). n == 0 returns
 * KF_ERR_EMPTY_REDUCTION. */
int32_t kf_mapreduce(int32_t f, int32_t op, int32_t g, int32_t dtype,
                     const void *src, uint64_t n, void *dst,
                     void *ws, size_t ws_bytes, const kf_launch_cfg *cfg, kf_stream_t stream);

/* Tuple form: dst[0] = g(op-reduce_i fn(srcs[0][i], ..., srcs[nsrc-1][i])). `srcs` is a HOST array of
 * `nsrc` device pointers (2..4 arrays of `dtype`, n elements each). Same kernel structure, workspace
 * (kf_mapreduce_workspace_bytes) and determinism as kf_mapreduce; `op` is one of ADD, MUL, MIN, MAX.
 * Algorithmic bytes: nsrc * n * sizeof(T). Arrays that do not share their 16-byte misalignment are
 * read element-wise.
 * Replaces the tuple methods of mapreduce1d / mapreduce1d! (src/mapreduce/1D/mapreduce1d.jl:177-288,
 * exercised by test/tests/mapreduce/mapreduce1d_test.jl:106-194). */
int32_t kf_mapreduce_multi(int32_t fn, int32_t op, int32_t g, int32_t dtype,
                           const void *const *srcs, int32_t nsrc, uint64_t n, void *dst,
                           void *ws, size_t ws_bytes, const kf_launch_cfg *cfg, kf_stream_t stream);

/* ---- scan ---------------------------------------------------------------------------------- */

/* Workspace for kf_scan / kf_scan_affine_*. Replaces get_allocation(Scan1D, ...)
 * (src/scan/scan.jl:156-211): one tile descriptor per tile + a tile ticket. `dtype` is the
 * element type; pass KF_F32 with `pair = 1` for the affine (a, b) pair. */
size_t kf_scan_workspace_bytes(int32_t dtype, int32_t pair, uint64_t n, const kf_launch_cfg *cfg);

/* Inclusive scan: dst[i] = g([seed op] f(src[0]) op ... op f(src[i])). Single pass, decoupled
 * look-back over tile descriptors in the workspace; operand order is preserved. `g` (a kf_post) is
 * applied to every output element, never to the carried prefix (src/scan/scan_kernel.jl:463,470,474).
 * `init` (device pointer to `ninit` elements, or NULL / 0) seeds the scan from the left with
 * init[0] op ... op init[ninit-1]; a sharded scan passes the totals of all shards and ninit = its
 * rank, so the carry of the shards before it needs no kernel of its own.
 * `dst == src` is allowed. n == 0 is a no-op (src/scan/scan.jl:273).
 * Replaces scan! / _scan_impl! (src/scan/scan.jl:261-284,414-479) and scan_kernel_packed! /
 * scan_kernel! (src/scan/scan_kernel.jl:310-478,94-299). */
int32_t kf_scan(int32_t f, int32_t op, int32_t g, int32_t dtype,
                const void *src, void *dst, uint64_t n, const void *init, uint32_t ninit,
                void *ws, size_t ws_bytes, const kf_launch_cfg *cfg, kf_stream_t stream);

/* Inclusive scan of affine maps x -> a*x + b under composition (KF_OP_AFFINE), Float32,
 * structure-of-arrays: (a_dst[i], b_dst[i]) = (a_0,b_0) o ... o (a_i,b_i). `init_ab` points to
 * `ninit` interleaved (a, b) pairs that seed the scan from the left, or is NULL. In reference terms
 * this is scan!(op, dst, src) over NTuple{2,Float32} on the split-descriptor kernel
 * (src/scan/scan_kernel.jl:94-299). */
int32_t kf_scan_affine_soa(const float *a_src, const float *b_src, float *a_dst, float *b_dst,
                           uint64_t n, const float *init_ab, uint32_t ninit,
                           void *ws, size_t ws_bytes, const kf_launch_cfg *cfg, kf_stream_t stream);

/* Same, array-of-structures: src/dst hold n interleaved (a, b) pairs, i.e. the reference's
 * scan!(op, dst, src) over a Vector{NTuple{2,Float32}} (src/scan/scan.jl:261-284). */
int32_t kf_scan_affine_aos(const float *ab_src, float *ab_dst, uint64_t n, const float *init_ab, uint32_t ninit,
                           void *ws, size_t ws_bytes, const kf_launch_cfg *cfg, kf_stream_t stream);

/* Workspace for kf_scan_quaternion (dtype KF_F32 or KF_F64 = the component type; 0 otherwise).
 * In reference terms get_allocation(Scan1D, ...) for a Quaternion element type
 * (src/scan/scan.jl:156-211, split layout). */
size_t kf_scan_quaternion_workspace_bytes(int32_t dtype, uint64_t n);

/* Inclusive scan of quaternions under the Hamilton product, which is not commutative:
 * dst[i] = src[0] * src[1] * ... * src[i]. An element is four consecutive components (w, x, y, z) of
 * type `dtype` (KF_F32: 16 bytes, KF_F64: 32 bytes), the layout of Quaternions.jl's Quaternion{T}.
 * `init` points to `ninit` quaternions that seed the scan from the left, or is NULL. This is the
 * reference's own non-commutative scan case, scan!(*, dst, src) over QuaternionF64 on the split
 * kernel (test/tests/scan/scan_test.jl:22-33, src/scan/scan_kernel.jl:94-299). */
int32_t kf_scan_quaternion(int32_t dtype, const void *src, void *dst, uint64_t n, const void *init, uint32_t ninit,
                           void *ws, size_t ws_bytes, const kf_launch_cfg *cfg, kf_stream_t stream);

/* Size of the fixed device array behind kf_scan_static: 1 MiB, held by every GPU that loads the
 * library until the process exits. It bounds the input: the call is refused when
 * kf_scan_workspace_bytes(dtype, 0, n, NULL) exceeds it. Largest n accepted, by element width
 * (kf_scan_static_max_n computes it): 1 byte 4 293 885 952; 2 bytes 2 146 942 976;
 * 4 bytes 1 073 471 488 (just under 2^30); 8 bytes 268 365 824 (just under 2^28). */
#define KF_SCAN_STATIC_SCRATCH_BYTES (1u << 20)

/* kf_scan for callers that cannot hand over a workspace because they cannot allocate device memory
 * at the point of the call. It has no counterpart in the reference, whose scan! allocates its
 * descriptors itself when `tmp` is not given (src/scan/scan.jl:291-307). Typical callers: code that
 * runs under a host framework's memory pool and must not call cudaMalloc behind its back, a process
 * that sits close to the device's memory limit where an allocation may fail or stall, and
 * latency-sensitive loops where cudaMalloc / cudaFree would synchronise the device.
 *
 * Same arguments, checks (in the same order), semantics and results as kf_scan with cfg == NULL,
 * minus `ws`, `ws_bytes`, `cfg`. The tile descriptors live in a fixed 1 MiB device array inside the
 * library; the call itself calls no cudaMalloc, cudaFree or allocating library routine.
 *   - The FIRST call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current) and caches it; make that first call before any stream capture.
 *   - All calls on one device share the array, and it keeps what the last call left there. Each call
 *     clears the part it uses first, so calls that follow one another on a stream are fine. Calls
 *     that overlap on the GPU (different streams, no ordering between them) race: do not do that.
 *   - Inputs whose descriptors do not fit (n > kf_scan_static_max_n(dtype)) return
 *     KF_ERR_EXCEEDS_STATIC_SCRATCH and touch nothing.
 *   - kf_scan_static_check plays the part of kf_check: it reads the status word of the array. */
int32_t kf_scan_static(int32_t f, int32_t op, int32_t g, int32_t dtype,
                       const void *src, void *dst, uint64_t n, const void *init, uint32_t ninit,
                       kf_stream_t stream);

/* Largest n that kf_scan_static accepts for `dtype` (0 for an unknown dtype). No counterpart in the
 * reference. */
uint64_t kf_scan_static_max_n(int32_t dtype);

/* kf_check for kf_scan_static: synchronises `stream` and returns the status word that the last
 * kf_scan_static call on the current device left in the fixed array (KF_OK or KF_ERR_TIMEOUT).
 * No counterpart in the reference, whose look-back spins are unbounded
 * (src/scan/scan_kernel.jl:388-415). */
int32_t kf_scan_static_check(kf_stream_t stream);

/* ---- sort ---------------------------------------------------------------------------------- */

/* Workspace for kf_sort_keys (val_bytes == 0) / kf_sort_pairs (val_bytes in {4, 8}).
 * Replaces get_allocation(Sort1D, ...) (src/sort/sort1d.jl:237-300): digit histograms, tile
 * descriptors, tile tickets and the n-element ping-pong scratch (keys, and values if any). */
size_t kf_sort_workspace_bytes(int32_t key_dtype, int32_t val_bytes, uint64_t n, const kf_launch_cfg *cfg);

/* Stable ascending LSD radix sort, 8-bit digits, one onesweep pass per key byte (every kf_dtype is
 * a valid key type: 1, 2, 4 or 8 passes). Keys are
 * ordered by the reference's uint_map (src/sort/uint_map.jl:11-35): unsigned = identity,
 * signed = sign bit flipped, floats = sign-flip / complement (-0.0 before +0.0, NaNs by bit
 * pattern); the original key bits are what is moved. `dst == src` sorts in place.
 * Replaces _sort1d_impl! (src/sort/sort1d.jl:780-874), _sort_histograms! (:655-697),
 * bucket_histogram_kernel! (src/sort/bucket_histogram_kernel.jl:77-145),
 * scan_histogram_kernel! (src/sort/scan_histogram_kernel.jl:20-46) and the onesweep pass
 * kernel (src/sort/onesweep_kernel.jl:113-488). One-byte keys replace the reference's
 * byte_sort_kernel (src/sort/byte_sort_kernel.jl:32-167): without a payload equal keys are the
 * same byte, so kf_sort_keys writes the 256 runs of the histogram out instead of scattering keys
 * (two-byte keys the same way with 65 536 bins from 2^22 keys on); with a payload (kf_sort_pairs)
 * they take the stable onesweep kernel with a single pass. n == 0 is a no-op. */
int32_t kf_sort_keys(int32_t key_dtype, const void *src, void *dst, uint64_t n,
                     void *ws, size_t ws_bytes, const kf_launch_cfg *cfg, kf_stream_t stream);

/* Key-value form: sorts (keys, vals) by key, stable; vals are opaque `val_bytes`-wide payloads.
 * Replaces _sort1d_keyval_impl! (src/sort/sort1d.jl:1006-1090) and the key-value pass kernel
 * (src/sort/keyval_onesweep_kernel.jl:45-317). */
int32_t kf_sort_pairs(int32_t key_dtype, const void *keys_src, void *keys_dst,
                      int32_t val_bytes, const void *vals_src, void *vals_dst, uint64_t n,
                      void *ws, size_t ws_bytes, const kf_launch_cfg *cfg, kf_stream_t stream);

/* ---- helpers used by the sharded (multi-GPU) layer and by sortperm --------------------------- */

/* dst[i] = start + i (uint32 or uint64 by `dtype`). The iota fill of sortperm!
 * (src/sort/sortperm.jl:162-214). */
int32_t kf_iota(int32_t dtype, void *dst, uint64_t n, uint64_t start, kf_stream_t stream);

/* For each of `nsplit` splitters (ascending, same dtype as keys), the index of the first element
 * of the SORTED array `keys` whose mapped key is greater than the splitter ("upper bound").
 * out[j] is uint64. Used to cut a sorted shard into per-destination runs for the sample sort;
 * the reference has no multi-GPU layer, the closest code is the splitter search of
 * src/sort/sample_sort.jl:284-312. */
int32_t kf_upper_bounds(int32_t key_dtype, const void *keys, uint64_t n,
                        const void *splitters, int32_t nsplit, uint64_t *out, kf_stream_t stream);

/* out[i] (uint8) = number of splitters (ascending, same dtype as keys, at most 255) whose mapped key
 * is smaller than that of keys[i]: the destination piece of key i when piece j holds the keys in
 * (splitter[j-1], splitter[j]]. With kf_sort_pairs on these one-byte ids (one stable pass, the keys
 * riding as the payload) it cuts an UNSORTED shard into per-destination runs for the sample sort.
 * The reference has no multi-GPU layer; the closest code is the bucket assignment of its
 * single-GPU sample sort (src/sort/sample_sort.jl:284-312). */
int32_t kf_bucket_ids(int32_t key_dtype, const void *keys, uint64_t n,
                      const void *splitters, int32_t nsplit, uint8_t *out, kf_stream_t stream);

/* Peer-memory exchange of the sharded sample sort (one process per GPU on one node); the reference
 * is single-device, so this group of entry points has no counterpart in the reference. A rank allocates ONE exchange buffer with
 * kf_xbuf_alloc (a whole cudaMalloc allocation, which is what CUDA IPC shares; the only place where
 * the library allocates device memory, at the caller's explicit request), exports it as 64 opaque
 * bytes (kf_ipc_export), the other ranks map it (kf_ipc_open: enables peer access) and pull their runs
 * out of it with kf_copy_d2d (one cudaMemcpyAsync per run, device-to-device over NVLink; remote data
 * lands in local HBM before any kernel touches it). kf_ipc_close / kf_xbuf_free undo the two. */
int32_t kf_xbuf_alloc(size_t nbytes, void **out);

/* Frees a buffer of kf_xbuf_alloc (after every peer has closed its mapping). No counterpart in the
 * reference. */
int32_t kf_xbuf_free(void *ptr);

/* The CUDA IPC handle of an exchange buffer as 64 opaque bytes, to be sent to the other ranks of the
 * node by whatever channel the host layer has. No counterpart in the reference. */
int32_t kf_ipc_export(const void *ptr, void *handle64);

/* Maps a peer's exchange buffer into this process (and enables peer access to that GPU); `out` is a
 * device pointer valid in this process. No counterpart in the reference. */
int32_t kf_ipc_open(const void *handle64, void **out);

/* Unmaps a buffer of kf_ipc_open. No counterpart in the reference. */
int32_t kf_ipc_close(void *ptr);

/* One asynchronous device-to-device copy (cudaMemcpyAsync) on `stream`; `src` may be a mapped peer
 * buffer, in which case the bytes cross NVLink once and land in local memory. No counterpart in the
 * reference. */
int32_t kf_copy_d2d(void *dst, const void *src, uint64_t nbytes, kf_stream_t stream);

/* Bytes of the region behind kf_peer_allgather (allocate it with kf_xbuf_alloc, clear it once, export
 * it with kf_ipc_export). No counterpart in the reference. */
size_t kf_peer_region_bytes(void);

/* Allgather of ONE element per rank over peer memory, as a kernel of this library: the exchange of the
 * sharded mapreduce (partials) and scan (shard totals) without a communication library and without the
 * host. `peers` is a DEVICE array of `world` pointers to every rank's region (mapped with kf_ipc_open;
 * entry `rank` is `local_region` itself), `value` one element of `elem_bytes` (1, 2, 4 or 8: the 8-byte
 * case also carries an affine (a, b) pair) in device memory, `out` receives the `world` elements in rank
 * order. `epoch` is a counter that all ranks advance together, starting at 1 (never 0); at most 64
 * ranks. The kernel stores its element into every region over NVLink and then waits, with a limit, for
 * the other ranks' elements in its OWN region; if one does not arrive it records KF_ERR_TIMEOUT in
 * `status_ws` (a 256-byte cleared workspace header, read with kf_check; word 1 = the missing rank) and
 * returns. All ranks must call it once per epoch. No counterpart in the reference, which is
 * single-device. */
int32_t kf_peer_allgather(const void *peers, const void *local_region, int32_t world, int32_t rank, uint32_t epoch,
                          const void *value, int32_t elem_bytes, void *out, void *status_ws,
                          const kf_launch_cfg *cfg, kf_stream_t stream);

/* ---- callers one step out: search, copy, fill ------------------------------------------------ */

/* Comparison of an element with a scalar operand, for kf_find. */
typedef enum kf_pred {
    KF_PRED_GT = 0, KF_PRED_LT = 1, KF_PRED_GE = 2, KF_PRED_LE = 3, KF_PRED_EQ = 4, KF_PRED_NE = 5
} kf_pred;

/* Workspace for kf_argmax: per-CTA (value, index) partials + a completion counter. Replaces
 * get_allocation(ArgMax1D, ...) (src/search/argmax.jl:117-150). */
size_t kf_argmax_workspace_bytes(int32_t dtype, uint64_t n);

/* out_index[0] (uint64, 0-based) = index of the first element whose f(src[i]) is extremal:
 * `greater` != 0 is rel = `>` (argmax), 0 is rel = `<` (argmin); ties go to the smallest index.
 * out_value (may be NULL) receives the extremal f(src[i]). One launch, last-CTA fold.
 * Replaces argmax1d / argmax1d! (src/search/argmax.jl:8-86,153-270) and argmax_kernel!
 * (src/search/argmax_kernel.jl:1-148). n == 0 returns KF_ERR_EMPTY_REDUCTION. */
int32_t kf_argmax(int32_t f, int32_t greater, int32_t dtype, const void *src, uint64_t n,
                  void *out_value, uint64_t *out_index, void *ws, size_t ws_bytes, kf_stream_t stream);

/* out_index[0] (uint64, device) = index (0-based) of the first (`last` == 0) or last (`last` != 0)
 * element with `src[i] pred operand`; `operand` is a HOST pointer to one element of `dtype`.
 * Not found: first -> UINT64_MAX, last -> 0 with found indices stored as index + 1 (so 0 means
 * none). CTAs stop early once a match ahead of them is known.
 * Replaces findfirst / findlast (src/search/findfirst.jl:3-110) and findfirst_kernel!
 * (src/search/findfirst_kernel.jl:1-67) for comparison predicates. */
int32_t kf_find(int32_t pred, int32_t last, int32_t dtype, const void *src, uint64_t n,
                const void *operand, uint64_t *out_index, kf_stream_t stream);

/* dst[0 .. nbytes) = src[0 .. nbytes) with 128-bit streaming accesses (element-wise when the two
 * arrays do not share their 16-byte misalignment). The roofline calibration kernel.
 * Replaces vcopy! (src/copy/copy.jl:1-28, src/copy/copy_kernel.jl:1-18). */
int32_t kf_vcopy(void *dst, const void *src, uint64_t nbytes, kf_stream_t stream);

/* dst[i] = *value for i in [0, n); `value` is a HOST pointer to one element of `dtype`.
 * Replaces setvalue! (src/copy/copy.jl:30-55, src/copy/copy_kernel.jl:20-36). */
int32_t kf_setvalue(int32_t dtype, void *dst, uint64_t n, const void *value, kf_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* KF_B200_H */
