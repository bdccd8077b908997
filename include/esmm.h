/*
 * esmm.h - C ABI of libesmm_b200: joint-sparse FP32 SGEMM ("ESMM") for NVIDIA B200 (sm_100a).
 *
 * The library replaces one path of the ESMM research harness: the A/B pattern
 * preprocessor, the joint-sparse SGEMM kernel (kernel id 29) and the runner /
 * kernel-id dispatch around them.  Every entry point names the reference
 * interface it stands in for (paths relative to the reference project root).
 *
 * Conventions
 *   - Matrices are dense row-major FP32: A is M x K (ld = K), B is K x N
 *     (ld = N), C is M x N (ld = N).  The reference names them rows = M,
 *     cols = N, inners = K.
 *   - Pointers are DEVICE pointers unless the name starts with h_.
 *   - Pattern arrays: one byte per (row block x 8-wide K block) of A and per
 *     (32-column block x 8-deep K block) of B, K-block index fastest; bit k
 *     (LSB = k 0) is set iff the tile holds a nonzero at K offset k.
 *   - Every function returns an esmm_status (0 = ESMM_OK) and never exits the
 *     process.  `stream` is a cudaStream_t passed as void* (NULL = default
 *     stream).  Launches are asynchronous unless stated otherwise.
 *   - There is no CPU fallback: without a usable CUDA device every compute
 *     entry point returns ESMM_ERR_CUDA.
 */
#ifndef ESMM_H_
#define ESMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum esmm_status {
    ESMM_OK = 0,
    ESMM_ERR_NULL = 1,        /* a required pointer is NULL */
    ESMM_ERR_SHAPE = 2,       /* non-positive dimension, or K / N not a multiple of 4 */
    ESMM_ERR_ALIGN = 3,       /* a matrix pointer is not 16-byte aligned */
    ESMM_ERR_CUDA = 4,        /* a CUDA runtime / driver call failed (see esmm_last_cuda_error) */
    ESMM_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up; results are invalid */
    ESMM_ERR_IO = 6,          /* file could not be read / written, or has the wrong size */
    ESMM_ERR_UNSUPPORTED = 7, /* kernel id or granularity this library does not provide */
    ESMM_ERR_VERIFY = 8,      /* verification against the reference result failed */
    ESMM_ERR_TOO_LARGE = 9,   /* K exceeds what the kernel's shared-memory masks can hold */
    ESMM_ERR_MISMATCH = 10,   /* cached pattern file does not match the requested shape */
    ESMM_ERR_BOUNDS = 11      /* checked build only: a kernel computed an index outside its buffer (access skipped) */
} esmm_status;

const char *esmm_strerror(int status);
/* Text of the last CUDA error this library saw on the calling thread ("" if none). */
const char *esmm_last_cuda_error(void);
int esmm_version(void);

/* ---- pattern geometry -------------------------------------------------- */

/* ceil(K / 8).  The reference computes K / BK (src/preprocessors/ab_preprocessor.cu:305). */
int esmm_num_k_blocks(int K);
/* Bytes of an A pattern array: ceil(M / tile_m) * ceil(K / 8)   (ab_preprocessor.cu:309). */
size_t esmm_a_pattern_bytes(int M, int K, int tile_m);
/* Bytes of a B pattern array: ceil(N / 32) * ceil(K / 8)        (ab_preprocessor.cu:310). */
size_t esmm_b_pattern_bytes(int K, int N);
/* "11110000" -> 0x0F: string position i is K offset i is bit i (include/utils.cuh:146-147,
 * ab_preprocessor.cu:70).  Returns -1 unless the string is eight '0'/'1' characters. */
int esmm_pattern_from_string(const char *pattern);
/* PatternLUT semantics (include/pattern_lut.cuh:13-19): *count = popcount(pattern),
 * offsets[0..count) = set bit indices ascending, remaining entries 0. */
void esmm_pattern_lut(uint8_t pattern, uint8_t *count, uint8_t offsets[8]);

/* ---- pattern preprocessor ---------------------------------------------- */

/*
 * A patterns: replaces preprocess_a_patterns_kernel<8, TILE_M, 256>
 * (src/preprocessors/ab_preprocessor.cu:31-84).  d_out[mb * nKB + kb], bit k set
 * iff any row of row block mb has a nonzero at column kb*8+k.  tile_m is the
 * rows per block (32 for kernel id 29; any positive value is accepted).
 * Ragged M or K are covered by a final partial block.  -0.0f is zero, NaN and
 * denormals are nonzero.
 */
int esmm_preprocess_a(const float *d_A, int M, int K, int tile_m, uint8_t *d_out, void *stream);

/*
 * B patterns: replaces preprocess_b_patterns_kernel<8, 32, 256>
 * (src/preprocessors/ab_preprocessor.cu:91-144).  d_out[nb * nKB + kb] (N-block
 * major, :141), bit k set iff any of columns nb*32..nb*32+31 has a nonzero in
 * row kb*8+k.  B is static in the intended use: compute once, keep or save.
 */
int esmm_preprocess_b(const float *d_B, int K, int N, uint8_t *d_out, void *stream);

/*
 * The reference's ABPatternMetadata (ab_preprocessor.cu:7-17), same fields.
 * owns_b_patterns is 0 when d_b_patterns was supplied by the caller (cached).
 */
typedef struct esmm_ab_pattern_metadata {
    uint8_t *d_a_patterns;
    uint8_t *d_b_patterns;
    int owns_b_patterns;
    int numMBlocks;
    int numNBlocks;
    int numKBlocks;
    float a_sparsity;
    float b_sparsity;
    float joint_sparsity;
} esmm_ab_pattern_metadata;

/*
 * Replaces preprocess_ab<8, TILE_M_A, 32> (ab_preprocessor.cu:297-326): allocates
 * the pattern arrays and launches the pattern kernels on the default stream
 * without synchronising.  If d_b_cached is not NULL it is used as the B pattern
 * array (not recomputed, not owned); the reference always recomputes B.
 */
int esmm_preprocess_ab(const float *d_A, const float *d_B, int M, int N, int K, int tile_m,
                       const uint8_t *d_b_cached, esmm_ab_pattern_metadata *meta);
/* Replaces free_ab_pattern_metadata (ab_preprocessor.cu:19-24). */
int esmm_free_ab_pattern_metadata(esmm_ab_pattern_metadata *meta);

/* B pattern cache file: 32-byte header (magic, K, N, nNB, nKB) + raw bytes.
 * Load fails with ESMM_ERR_MISMATCH if the file was written for another K x N.
 * The reference only reserves the hook for this (owns_b_patterns, ab_preprocessor.cu:10,21). */
int esmm_bpat_save(const char *path, const uint8_t *h_b_patterns, int K, int N);
int esmm_bpat_load(const char *path, uint8_t *h_b_patterns, int K, int N);

/* ---- joint-sparse SGEMM ------------------------------------------------- */

/*
 * C = A * B over the k whose joint bit (a_pat[i/32][k/8] & b_pat[j/32][k/8]) >> (k%8) & 1
 * is set; one FFMA chain per output in ascending k; C is overwritten.  Replaces
 * esmm_ab_optimized_v3 + dispatch_v3 (src/kernels/esmm_ab_optimized_v3.cu:18-235,
 * include/runners.cuh:801-825).  a_tile_m is the row granularity of d_a_pat
 * (32 for id 29; 8, 16, 64, 128 are accepted and folded to 32-row warp tiles).
 * Needs K % 4 == 0, N % 4 == 0, 16-byte aligned A, B, C; M is arbitrary.
 * No hidden allocation; a device-side wait that gives up is reported by
 * esmm_device_status.
 */
int esmm_gemm_ab(int M, int N, int K, const float *d_A, const float *d_B, float *d_C,
                 const uint8_t *d_a_pat, const uint8_t *d_b_pat, int a_tile_m, void *stream);

/*
 * Packing variant of the A preprocessor: one pass over A writes the 32-row pattern
 * bytes (same bytes as esmm_preprocess_a with tile_m = 32) and a k-major copy of A,
 *   packed[((row / 128) * nKB * 8 + k) * 128 + row % 128],
 * esmm_a_packed_bytes(M, K) bytes, which esmm_gemm_ab_packed reads instead of A.
 * Entries whose pattern bit is clear are left unwritten (they are never multiplied).
 * Needs K % 4 == 0 and 16-byte aligned pointers.  No counterpart in the reference,
 * whose kernel transposes A tiles in shared memory on every K step
 * (src/kernels/esmm_ab_optimized_v3.cu:126-132).
 */
size_t esmm_a_packed_bytes(int M, int K);
int esmm_preprocess_a_packed(const float *d_A, int M, int K, uint8_t *d_out, float *d_packed,
                             void *stream);
/*
 * Same contract as esmm_gemm_ab (32-row A patterns) with the packed copy in place of A, except that
 * the first call on a device sets aside one 64-byte word of host-mapped memory (kept for the life of
 * the process): every launch of the tiled kernel notes there whether its first tile was one of
 * scattered single rows, and the next launch on that device picks its launch shape (12 or 16 warps
 * per CTA) by it, without waiting for anything.  The shapes differ in speed only, never in a bit of
 * C; esmm_tuning_set("PRODUCER_WARPS", ...) pins one.  No device memory is allocated.  Make the first
 * call on a device outside any stream capture (the set-up is not a stream operation).
 */
int esmm_gemm_ab_packed(int M, int N, int K, const float *d_a_packed, const float *d_B, float *d_C,
                        const uint8_t *d_a_pat, const uint8_t *d_b_pat, void *stream);

/*
 * The per-call path with B patterns cached ("B offline, A per call"): the packing
 * preprocessor and the packed GEMM, both on `stream`.  d_workspace is caller-owned
 * device memory of esmm_sgemm_joint_workspace_bytes(M, K) bytes, 256-byte aligned
 * (A patterns followed by the packed copy); no device memory is allocated here (the first call on
 * a device sets up the host-mapped word described at esmm_gemm_ab_packed).
 */
size_t esmm_sgemm_joint_workspace_bytes(int M, int K);
int esmm_sgemm_joint(int M, int N, int K, const float *d_A, const float *d_B, float *d_C,
                     const uint8_t *d_b_pat, void *d_workspace, void *stream);

/*
 * esmm_sgemm_joint for callers that cannot allocate and cannot pass scratch memory: hosts whose
 * operator contract forbids allocation at call time, processes whose allocator already owns the
 * whole GPU, loops that cannot afford the device-wide synchronisation of a cudaMalloc.  Same
 * inputs, outputs and results as esmm_sgemm_joint, but the scratch (A patterns + packed copy of A)
 * is a fixed array inside the library image: the call performs no cudaMalloc / cudaFree and uses
 * no allocating library routine.  It has no counterpart in the reference, whose runner allocates
 * and frees its pattern buffers on every run.
 *   - Limit: esmm_a_packed_bytes(M, K) <= ESMM_STATIC_MAX_PACKED_FLOATS * 4 (32 MiB, e.g. A of
 *     2048 x 4096) and esmm_a_pattern_bytes(M, K, 32) <= ESMM_STATIC_MAX_PATTERN_BYTES; larger A
 *     returns ESMM_ERR_TOO_LARGE with the sizes in esmm_last_cuda_error().
 *   - Cost: every GPU that loads the library holds the 32 MiB + 64 KiB array until the library
 *     is unloaded.
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call before any stream capture begins.  It is also the call
 *     that may make the CUDA runtime load this library's device code, which is when the driver
 *     sets the array aside: a host whose allocator is about to claim all free memory should make
 *     one (small) call first, at initialisation.
 *   - All calls on a GPU share the array and it keeps the previous call's contents (nothing in it
 *     needs clearing).  Calls whose kernels overlap on one GPU race on it: serialise them.
 */
#define ESMM_STATIC_MAX_PACKED_FLOATS (8u << 20)
#define ESMM_STATIC_MAX_PATTERN_BYTES (64u << 10)
int esmm_sgemm_joint_static(int M, int N, int K, const float *d_A, const float *d_B, float *d_C,
                            const uint8_t *d_b_pat, void *stream);

/* Synchronises `stream`, returns and clears the device status word:
 * ESMM_OK, ESMM_ERR_TIMEOUT (a bounded wait expired) or ESMM_ERR_CUDA. */
int esmm_device_status(void *stream);

/*
 * The checked build (libesmm_b200_checked.so, same ABI, compiled with -DESMM_CHECKED) stands in for a
 * memory sanitizer: its kernels test the shared- and global-memory indices that depend on the problem's shape
 * or data (list and mask positions, ring slots, pattern loads, loads of A and B in the preprocessors, every store
 * to a caller's buffer) and, instead of trapping, record ESMM_ERR_BOUNDS plus the site in the device status word and skip the access;
 * esmm_device_status() then returns ESMM_ERR_BOUNDS and esmm_last_cuda_error() names the site.  The
 * reference has only `#ifdef DEBUG` synchronisations (src/preprocessors/a_preprocessor_hybrid.cu:115-120).
 *   esmm_checked_build            1 in the checked build, 0 in the product build.
 *   esmm_selftest_bounds_report   launches one thread that reports a failed check WITHOUT making any
 *                                 access: the next esmm_device_status() returns ESMM_ERR_BOUNDS in the checked
 *                                 build and ESMM_OK in the product build.
 */
int esmm_checked_build(void);
int esmm_selftest_bounds_report(void *stream);

/*
 * Failure-path self test: launches one CTA that waits (bounded, `budget_us` microseconds, at most
 * one second) on a barrier nothing arrives on.  The wait gives up, the kernel returns normally and
 * the next esmm_device_status() reports ESMM_ERR_TIMEOUT; the context stays usable.  The reference
 * has no device-side waits and no counterpart.
 */
int esmm_selftest_bounded_wait(unsigned budget_us, void *stream);

/*
 * Tuning and test hooks.  The launch heuristics (tile height, ring depth, row-fetch policy, grid size,
 * which kernel variant runs) can be overridden per process by name; tests use this to force every
 * variant through the same parity cases.  Nothing is read from the environment: a caller's
 * environment cannot change what the library does.  No counterpart in the reference, whose tile
 * shapes are compile-time template constants (include/runners.cuh:830-838).
 * Names: TILE_M (64 | 128), STAGES, BROW_BITS, ROW_DENSITY, FORCE_LISTED, NO_RUN_TILES, VEC_PATTERNS
 * (0 | 4 | 16), NO_SKINNY, SKINNY_ROWS (32), PRODUCER_WARPS (3 | 7 | 0: pins the tiled kernel's launch shape), NO_DEPENDENT_LAUNCH, GROUP_M, GRID, PACK (64 | 128), SWIZZLE, TF32_PAIR (0 | 128 | 256), TF32_SPLIT_LAST,
 * TF32_DIRECT_STORES.  esmm_tuning_set returns ESMM_ERR_UNSUPPORTED for any other name;
 * esmm_tuning_reset returns every hook to "unset" (the library's own choice).
 */
int esmm_tuning_set(const char *name, int value);
void esmm_tuning_reset(void);
/*
 * Warps per CTA (12 or 16) of the last launch of the tiled kernel issued by this process on the current
 * device, 0 if there was none: shows which launch shape the note of the launch before it selected
 * (see esmm_gemm_ab_packed).  For tests and logs; no counterpart in the reference.
 */
int esmm_last_tiled_kernel_warps(void);

/* ---- host-buffer (end-to-end) path -------------------------------------- */

/*
 * A plan keeps B and its patterns resident on the device ("B offline") and owns
 * device buffers for A, C and the A patterns.  esmm_plan_run takes HOST A and C
 * (pinned memory gives the best copy rate), copies A in row chunks, computes and
 * copies C back, overlapping the three, and returns when h_C is complete.
 */
typedef struct esmm_plan esmm_plan;
int esmm_plan_create(int M, int N, int K, const float *h_B, int chunks, esmm_plan **plan);
int esmm_plan_run(esmm_plan *plan, const float *h_A, float *h_C);
/*
 * The two halves of esmm_plan_run.  esmm_plan_submit only enqueues (copies, kernels, copies back) and
 * returns; esmm_plan_wait returns when everything submitted to the plan has landed in its h_C, with
 * the device status.  Several submissions to one plan, or to several plans, may be in flight: the copies
 * of one overlap the kernels of another (a plan's device buffers are handed from one submission to the
 * next chunk by chunk).  h_A and h_C must be pinned host memory for the copies to be asynchronous, and
 * must stay valid and untouched until the wait returns.
 */
int esmm_plan_submit(esmm_plan *plan, const float *h_A, float *h_C);
int esmm_plan_wait(esmm_plan *plan);
int esmm_plan_destroy(esmm_plan *plan);

/* ---- comparison baselines, measurement helpers ---------------------------- */

/* cuBLAS SGEMM exactly as run_cuBlas calls it (include/runners.cuh:122-123): row-major
 * trick, alpha 1, beta 0, default math mode.  The handle is created once per device. */
int esmm_cublas_sgemm(int M, int N, int K, const float *d_A, const float *d_B, float *d_C,
                      void *stream);
/* Measured FP32 FFMA throughput of the current device in TFLOP/s (dependent-free FFMA
 * chains on every SM, timed with CUDA events); *sm_count gets the SM count. */
int esmm_ffma_peak_tflops(double *tflops, int *sm_count);

/* Optional tensor-core variant: the joint-sparse product as 3xTF32 on the 5th-generation tensor cores
 * (tcgen05.mma kind::tf32, accumulators in tensor memory).  No counterpart in the reference, whose kernels
 * are FP32 FMA only.  Every operand is split as x = hi + lo (both TF32) and a product is formed as
 * a_hi b_hi + a_hi b_lo + a_lo b_hi; the tensor core accumulates runs of 256 k in FP32, the runs are added in
 * registers.  C agrees with esmm_gemm_ab to a few 1e-6 of max |C| (inside the 1e-4 bound the FP32 path is
 * held to) but is NOT bit-identical to it.  Requires K % 8 == 0, N % 4 == 0, finite inputs.  Tiles of 256 x 256 or
 * 256 x 128 run on pairs of CTAs (cta_group::2), tiles of 128 x 128 on one CTA; the library picks by the number of
 * tiles (esmm_tuning_set("TF32_PAIR", 0 | 128 | 256) forces the single-CTA kernel, 256 x 128 or 256 x 256 per pair).
 * Work is skipped at two levels: k with an all-zero row of B are dropped from both operands when B is prepared
 * (compact != 0), and of what is left a tile multiplies only the 8-wide K blocks in which its A and
 * B patterns share a live k.
 *
 * esmm_tf32x3_b_create: the "B offline" step (beside esmm_preprocess_b): B patterns, the list of kept k, B
 *   transposed and split.  Allocates device memory, synchronises; the handle belongs to the current device.
 * esmm_tf32x3_b_live_k: k kept (K without compaction; else a multiple of 32, padding included).
 * esmm_sgemm_joint_tf32x3: split (and gather) of A with its A patterns + product, two launches on `stream`, no
 *   allocation.  d_A: M x K row-major; d_C: M x N; d_workspace: esmm_tf32x3_workspace_bytes(M, K) bytes,
 *   256-byte aligned. */
typedef struct esmm_tf32x3_b esmm_tf32x3_b;
int esmm_tf32x3_b_create(const float *d_B, int K, int N, int compact, esmm_tf32x3_b **out);
void esmm_tf32x3_b_destroy(esmm_tf32x3_b *b);
int esmm_tf32x3_b_live_k(const esmm_tf32x3_b *b);
size_t esmm_tf32x3_workspace_bytes(int M, int K);
int esmm_sgemm_joint_tf32x3(int M, const float *d_A, const esmm_tf32x3_b *b, float *d_C, void *d_workspace,
                            void *stream);

/* cuSPARSE SpMM baseline (src/benchmarks/cusparse_benchmark.cu:56-247): A (M x K, row-major, dense
 * storage) is converted to CSR and multiplied with dense B into C.  *spmm_ms: average of `runs` SpMM
 * calls with A already in CSR; *total_ms: average of `runs` (conversion + SpMM) calls; *nnz: stored
 * nonzeros of A (the work is 2 * nnz * N flops).  Library calls only, allocates and frees its own
 * buffers, synchronises the device.  Any output pointer may be NULL. */
int esmm_cusparse_spmm(int M, int N, int K, const float *d_A, const float *d_B, float *d_C, int runs,
                       float *spmm_ms, float *total_ms, long long *nnz);

/* Counter-based N(mean, std) generator with block-structured zeros, on the device.
 * Element (r, c) of a rows x cols row-major matrix; k = c when k_axis == 0 (matrix A),
 * k = r when k_axis == 1 (matrix B); the other index is the "outer" index.
 *   mode 0: dense.
 *   mode 1: uniform pattern - element is zero unless bit (k % 8) of `pattern` is set.
 *   mode 2: independent tile patterns - for each (outer / gran, k / 8) tile each of the 8
 *           k offsets is live with probability p_live (decided by hash(seed2, tile, bit)).
 * relu != 0 applies max(x, 0) before the zero pattern.  Not part of the reference, whose
 * generators use rand(); here so that 16384^2 inputs need no host copy. */
int esmm_fill_normal(float *d_out, long rows, long cols, int k_axis, uint64_t seed, float mean,
                     float std, int relu, int mode, uint8_t pattern, float p_live, int gran,
                     uint64_t seed2, void *stream);

/* Interleaves G column shards [g][M][N/G] into row-major M x N (used after an all-gather). */
int esmm_interleave_shards(const float *d_shards, float *d_C, int M, int N, int G, void *stream);

/* ---- harness data generators and usage text (host only) -------------------- */

/*
 * The driver's rand()-based generators, draw for draw: the same calls to the C library's rand() in
 * the same order, rounding where the reference's expressions round, so that a seed gives the matrices
 * the reference driver multiplies.  All take HOST pointers and need no device.
 *   esmm_randomize_matrix_with_pattern   randomize_matrix_with_pattern (include/utils.cuh:142-156): the
 *       default mode; element (i, j) is live when pattern[j % 8] == '1' (for B that is the N index,
 *       driver.cu:404-405); does not seed.
 *   esmm_randomize_matrix_unstructured   randomize_matrix_unstructured (include/utils.cuh:159-194):
 *       --random; seeds when seed != 0; prints the reference's note when the achieved sparsity is more
 *       than 2 points off.
 *   esmm_randomize_matrix_a_blocklevel   randomize_matrix_A_blocklevel<BK, WM> (include/utils.cuh:303-341)
 *       and randomize_matrix_A<BK, TILE_M> (:386-426), which differ only in the default tile height:
 *       one random 8-bit pattern per (tile_m rows x bk columns) tile of A.
 *   esmm_randomize_matrix_b_blocklevel   randomize_matrix_B_blocklevel_fixed<BK, WN> (:343-381): one
 *       pattern per (bk rows x wn columns) tile of B.
 * Values are {0..4} + 0.01 * {0..4} with a random sign.  Rows / columns beyond the last whole tile are
 * left untouched, as in the reference.
 */
int esmm_randomize_matrix_with_pattern(float *h_mat, int M, int N, const char *pattern);
int esmm_randomize_matrix_unstructured(float *h_mat, int M, int N, float sparsity_percent, unsigned seed);
int esmm_randomize_matrix_a_blocklevel(float *h_mat, int M, int K, int bk, int tile_m,
                                       float block_sparsity_percent, unsigned seed);
int esmm_randomize_matrix_b_blocklevel(float *h_mat, int K, int N, int bk, int wn,
                                       float block_sparsity_percent, unsigned seed);
/* print_usage (include/utils.cuh:66-101) on stdout.  additive != 0 also lists the flags and the kernel
 * id this library adds to the reference's command line. */
void esmm_print_usage(const char *program_name, int additive);

/* ---- several GPUs of one machine ------------------------------------------ */

/*
 * N-column sharding from ONE process: C[:, n0:n1] = A * B[:, n0:n1] needs no exchange between the GPUs.
 * Every device holds all of A (and preprocesses its own replica per run), a contiguous K x N/G block of B's
 * columns with that block's cached patterns, and the matching M x N/G block of C; one host thread per device
 * launches its work on a stream of its own.  No counterpart in the reference, which is single-GPU throughout
 * (no cudaSetDevice, stream or communication call anywhere in its tree); this is what `exec_b200 --gpus G`
 * runs.  No kernel reads another GPU's memory.
 *   esmm_multi_shard_columns  columns [n0, n1) of rank `rank`: equal blocks, N % (G * 128) == 0 (whole GEMM
 *                             tiles and pattern blocks per shard), else ESMM_ERR_SHAPE.  Host arithmetic only.
 *   esmm_multi_create         validates, allocates every device's buffers (devices == NULL: 0 .. G-1; a device
 *                             may be named twice, e.g. to exercise the sharding on one GPU - esmm_multi_gather
 *                             then refuses).  ESMM_ERR_UNSUPPORTED if a device does not exist.
 *   esmm_multi_upload         host A (M x K) to every device, host B (K x N) column block by column block, and
 *                             the B patterns of each block ("B offline").  Either pointer may be NULL to keep
 *                             what is there.
 *   esmm_multi_fill           device-side generator instead of an upload (esmm_fill_normal): the same A on every
 *                             device (seed), B's block on rank g from seed + 1 + g.
 *   esmm_multi_run            one untimed call, then `runs` times esmm_sgemm_joint on every device, the devices' loops started together;
 *                             ms_per_gpu[g] = that device's CUDA-event time per run, *ms_max the slowest (the
 *                             whole-box time).  A bounded device wait that gave up returns ESMM_ERR_TIMEOUT.
 *   esmm_multi_download       the blocks of C into a host M x N matrix, device by device, no collective.
 *   esmm_multi_gather         all of C on the first device: NCCL all-gather of the blocks (NCCL is looked up with
 *                             dlopen at the first call) + esmm_interleave_shards there; h_C != NULL also copies it
 *                             to the host; *ms = device time of gather + interleave (slowest device).  Before NCCL
 *                             is entered every device has reported, on the host, that its buffers exist: a device
 *                             that failed never enters a collective the others would wait in.  ESMM_ERR_UNSUPPORTED
 *                             without NCCL or with a device named twice.
 *   esmm_multi_gathered_c     device pointer (first device) of the gathered M x N matrix, NULL before a gather.
 */
typedef struct esmm_multi esmm_multi;
int esmm_multi_shard_columns(int N, int num_gpus, int rank, int *n0, int *n1);
int esmm_multi_create(int M, int N, int K, int num_gpus, const int *devices, esmm_multi **out);
int esmm_multi_num_gpus(const esmm_multi *m);
int esmm_multi_upload(esmm_multi *m, const float *h_A, const float *h_B);
int esmm_multi_fill(esmm_multi *m, uint64_t seed, int mode, uint8_t pattern_a, uint8_t pattern_b, float p_a,
                    float p_b, int gran);
int esmm_multi_run(esmm_multi *m, int runs, float *ms_max, float *ms_per_gpu);
int esmm_multi_download(esmm_multi *m, float *h_C);
int esmm_multi_gather(esmm_multi *m, float *h_C, float *ms);
const float *esmm_multi_gathered_c(const esmm_multi *m);
int esmm_multi_destroy(esmm_multi *m);

/* ---- skip statistics ------------------------------------------------------ */

/* compute_and_print_skip_stats arithmetic (include/runners.cuh:636-706) on HOST pattern
 * arrays for CTA tiles of warps_m x warps_n pattern blocks.
 * out[6] = block_skips, total_k, warp_skips, total_warp_k, dot_skips, total_dot. */
int esmm_skip_stats(const uint8_t *h_a_pat, const uint8_t *h_b_pat, int num_cblocks_m,
                    int num_cblocks_n, int numKBlocks, int warps_m, int warps_n, int bk,
                    long long out[6]);

/* ---- runners: the kernel-id dispatch -------------------------------------- */

/* Valid ids of the reference driver (driver.cu:20): 14-17, 20, 21, 25-30. */
int esmm_kernel_id_valid(int kernel_id);
/* get_kernel_name (include/utils.cuh:48-64). */
const char *esmm_kernel_name(int kernel_id);
/* parse_kernel_selection (include/utils.cuh:18-46): "29", "29,15", "14-17", "all".
 * Writes at most cap ids, returns how many the selection holds (0 = invalid). */
int esmm_parse_kernel_selection(const char *selection, int *ids, int cap);

/*
 * One kernel id through its runner, with the reference's loop: per run a memset of
 * C, pattern allocation + both pattern kernels, the GEMM, a device synchronise and
 * the frees (include/runners.cuh:852-872); prints "Kernel time: ..." and, when
 * verify != 0, copies C to h_C and applies verifyResults' absolute tolerance 1e-2
 * against h_C_ref (include/utils.cuh:222-254).  Stands in for
 * run_esmm_ab_optimized_v3 / _no_check (runners.cuh:827-897), run_cuBlas
 * (:109-144) and the `switch` of run_single_kernel (driver.cu:40-129).
 * Ids served: 15 (cuBLAS), 29, and the joint-sparse ids 20, 21, 25, 26, 27, 28, 30
 * as aliases of the same kernel at their own A granularity; the single-operand ids
 * 16 (A patterns only, B all live), 17 (B patterns only) and 14 (see
 * esmm_run_kernel_pattern) as degenerate cases of it.  *passed gets 1/0; *avg_ms the
 * average time per run.
 */
int esmm_run_kernel(int kernel_id, int rows, int cols, int inners, float *d_A, float *d_B,
                    float *d_C, float *h_C, const float *h_C_ref, int runs, int verify,
                    int print_skip_stats, int *passed, float *avg_ms);

/*
 * Same runner with the B patterns supplied by the caller (device array of esmm_b_pattern_bytes(K, N)
 * bytes, e.g. uploaded from an esmm_bpat_load() file): the timed loop then preprocesses A only.  This
 * is the "B offline, A per call" mode the reference describes (README.md:46,103) but never runs - its
 * runner recomputes B patterns in every iteration (include/runners.cuh:859).  NULL = recompute.
 */
int esmm_run_kernel_cached_b(int kernel_id, int rows, int cols, int inners, float *d_A, float *d_B,
                             float *d_C, float *h_C, const float *h_C_ref, int runs, int verify,
                             int print_skip_stats, const uint8_t *d_b_pat_cached, int *passed,
                             float *avg_ms);

/*
 * The general form: d_b_pat_cached as above, and the driver's 8-character pattern string, which only
 * id 14 reads.  run_esmm_unrolled (include/runners.cuh:30-106) never looks at the data: it multiplies the
 * first popcount(pattern) k of every 8-slice of K - the unrolled kernels exist for 1, 2, 4, 6 and 8 live
 * k; for any other count the reference launches nothing and C stays zero, and so does this.  Here that is
 * the joint kernel with every A pattern byte = (1 << popcount) - 1 and every B byte 0xFF, no
 * preprocessing in the loop.  pattern == NULL means "11111111".  Other ids ignore the string.
 */
int esmm_run_kernel_pattern(int kernel_id, int rows, int cols, int inners, float *d_A, float *d_B,
                            float *d_C, float *h_C, const float *h_C_ref, int runs, int verify,
                            int print_skip_stats, const uint8_t *d_b_pat_cached, const char *pattern,
                            int *passed, float *avg_ms);

#ifdef __cplusplus
}
#endif
#endif /* ESMM_H_ */
