/*
 * CPU oracle for the ESMM joint-sparse SGEMM path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, on the CPU, the algorithm of
 * the reference's A/B pattern preprocessor and of its kernel id 29, so that the
 * CUDA kernels of this repository can be checked against it.  Nothing in the
 * product library links, loads or calls this file; only the tests, the smoke
 * check and the benchmark's CPU-baseline leg do.
 *
 * Parity pin: the reference has no golden vectors for this path.  The oracle is
 * pinned (a) against the reference's own host functions compiled from the
 * reference tree (matrixMultiplyCPU, verifyResults, the rand()-based
 * generators) and (b) against pattern bytes and C produced by the reference's
 * own GPU kernels, captured on a B200 and stored as fixtures under
 * tests/golden/.
 *
 * Every function cites the reference lines it follows (paths are relative to
 * the reference project root).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_BK 8

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

/* `val != 0.0f` exactly as the reference tests it
 * (src/preprocessors/ab_preprocessor.cu:68-71 and :128-131):
 * -0.0f is zero, NaN is nonzero, denormals are nonzero (IEEE compare). */
static inline int is_nonzero(float v) { return v != 0.0f; }

/*
 * A patterns.  Follows preprocess_a_patterns_kernel
 * (src/preprocessors/ab_preprocessor.cu:31-84): one byte per
 * (tile_m-row block, 8-wide K block); bit k (LSB = k 0) is set iff any of the
 * tile's rows has a nonzero in column kb*8+k.  Output index mb*numKBlocks+kb
 * (:81).  Where the reference floors M/tile_m and K/8 and so ignores ragged
 * edges, this restatement covers the ragged tail with a final partial block
 * (elements outside the matrix count as zero); on shapes the reference
 * accepts the bytes are identical.
 */
void oracle_preprocess_a(const float *A, int M, int K, int tile_m, uint8_t *out)
{
    const int nMB = ceil_div(M, tile_m), nKB = ceil_div(K, ORACLE_BK);
    memset(out, 0, (size_t)nMB * nKB);
    for (int i = 0; i < M; ++i) {
        uint8_t *row = out + (size_t)(i / tile_m) * nKB;
        const float *a = A + (size_t)i * K;
        for (int k = 0; k < K; ++k)
            if (is_nonzero(a[k])) row[k >> 3] |= (uint8_t)(1u << (k & 7));
    }
}

/*
 * B patterns.  Follows preprocess_b_patterns_kernel
 * (src/preprocessors/ab_preprocessor.cu:91-144): one byte per
 * (wn-column block, 8-deep K block); bit k set iff any of the block's columns
 * has a nonzero in row kb*8+k.  Output is N-block major: nb*numKBlocks+kb
 * (:141).
 */
void oracle_preprocess_b(const float *B, int K, int N, int wn, uint8_t *out)
{
    const int nNB = ceil_div(N, wn), nKB = ceil_div(K, ORACLE_BK);
    memset(out, 0, (size_t)nNB * nKB);
    for (int k = 0; k < K; ++k) {
        const float *b = B + (size_t)k * N;
        const uint8_t bit = (uint8_t)(1u << (k & 7));
        for (int j = 0; j < N; ++j)
            if (is_nonzero(b[j])) out[(size_t)(j / wn) * nKB + (k >> 3)] |= bit;
    }
}

/*
 * Joint-sparse GEMM.  Follows esmm_ab_optimized_v3
 * (src/kernels/esmm_ab_optimized_v3.cu:18-235):
 *   joint = a_pat[i/tile_m][kb] & b_pat[j/wn][kb]              (:74-77)
 *   for k in 0..7 ascending: if joint bit k, acc = fma(a, b, acc)  (:157, :183-203)
 *   C is overwritten (beta = 0)                                  (:212-234)
 * One fused multiply-add chain per output, in ascending k, over live k only.
 * Loop order here is i -> kb -> k -> j, which leaves every output's chain in
 * ascending k.
 */
void oracle_gemm_joint(int M, int N, int K, const float *A, const float *B, float *C,
                       const uint8_t *a_pat, const uint8_t *b_pat, int tile_m, int wn)
{
    const int nKB = ceil_div(K, ORACLE_BK);
    const int nNB = ceil_div(N, wn);
    for (int i = 0; i < M; ++i) {
        float *c = C + (size_t)i * N;
        const float *a = A + (size_t)i * K;
        const uint8_t *ap = a_pat + (size_t)(i / tile_m) * nKB;
        for (int j = 0; j < N; ++j) c[j] = 0.0f;
        for (int nb = 0; nb < nNB; ++nb) {
            const uint8_t *bp = b_pat + (size_t)nb * nKB;
            const int j0 = nb * wn, j1 = (j0 + wn < N) ? j0 + wn : N;
            for (int kb = 0; kb < nKB; ++kb) {
                const unsigned joint = ap[kb] & bp[kb];
                if (!joint) continue;
                for (int kk = 0; kk < ORACLE_BK; ++kk) {
                    if (!(joint & (1u << kk))) continue;
                    const int k = kb * ORACLE_BK + kk;
                    if (k >= K) break;
                    const float av = a[k];
                    const float *b = B + (size_t)k * N;
                    for (int j = j0; j < j1; ++j) c[j] = fmaf(av, b[j], c[j]);
                }
            }
        }
    }
}

/*
 * The driver's CPU SGEMM.  Follows matrixMultiplyCPU (include/utils.cuh:208-219):
 * i-j-k loops, `sum += A[i*K+k] * B[k*N+j]` with a separate multiply and add
 * (the reference is built for baseline x86-64, which has no FMA instruction to
 * contract into; this file is compiled with -ffp-contract=off).  Computes rows
 * [row0, row1) only, so that callers can split rows across threads or time a
 * bounded sample; every output is still one sequential k loop, so results are
 * identical to the single-thread function.
 */
void oracle_sgemm_naive_rows(const float *A, const float *B, float *C, int M, int N, int K,
                             int row0, int row1)
{
    (void)M;
    for (int i = row0; i < row1; ++i) {
        for (int j = 0; j < N; ++j) {
            float sum = 0.0f;
            for (int k = 0; k < K; ++k) {
                const float p = A[(size_t)i * K + k] * B[(size_t)k * N + j];
                sum = sum + p;
            }
            C[(size_t)i * N + j] = sum;
        }
    }
}

void oracle_sgemm_naive(const float *A, const float *B, float *C, int M, int N, int K)
{
    oracle_sgemm_naive_rows(A, B, C, M, N, K, 0, M);
}

/* float64-accumulated dense product of rows [row0,row1), for tolerance
 * arbitration only (not a restatement of any reference function). */
void oracle_sgemm_f64_rows(const float *A, const float *B, double *C, int M, int N, int K,
                           int row0, int row1)
{
    (void)M;
    for (int i = row0; i < row1; ++i) {
        double *c = C + (size_t)(i - row0) * N;
        for (int j = 0; j < N; ++j) c[j] = 0.0;
        for (int k = 0; k < K; ++k) {
            const double av = A[(size_t)i * K + k];
            if (av == 0.0) continue;
            const float *b = B + (size_t)k * N;
            for (int j = 0; j < N; ++j) c[j] += av * (double)b[j];
        }
    }
}

/*
 * verifyResults (include/utils.cuh:222-254): counts elements whose absolute
 * difference exceeds the tolerance (default 1e-2 there).  Returns the count;
 * max_diff gets the largest offending difference, first_idx the first
 * offender (-1 if none).  NaN differences never compare greater, as in the
 * reference.
 */
long oracle_verify_results(const float *gpu, const float *ref, long size, float tol,
                           float *max_diff, long *first_idx)
{
    long bad = 0, first = -1;
    float md = 0.0f;
    for (long i = 0; i < size; ++i) {
        const float d = fabsf(gpu[i] - ref[i]);
        if (d > tol) {
            ++bad;
            if (first < 0) first = i;
            if (d > md) md = d;
        }
    }
    if (max_diff) *max_diff = md;
    if (first_idx) *first_idx = first;
    return bad;
}

/*
 * Skip statistics.  Follows compute_and_print_skip_stats
 * (include/runners.cuh:636-706): for a CTA tile of warps_m x warps_n pattern
 * blocks, counts K tiles skipped by the whole block (OR over warps of the joint
 * is 0, :661-665), by single warps (:675-678) and single k columns (:680).
 * out[0..5] = block_skips, total_k, warp_skips, total_warp_k, dot_skips, total_dot.
 */
void oracle_skip_stats(const uint8_t *a_pat, const uint8_t *b_pat,
                       int num_cblocks_m, int num_cblocks_n, int nKB,
                       int warps_m, int warps_n, int bk, long long *out)
{
    const int nw = warps_m * warps_n;
    long long block_skips = 0, warp_skips = 0, dot_skips = 0;
    for (int cr = 0; cr < num_cblocks_m; ++cr)
        for (int cc = 0; cc < num_cblocks_n; ++cc)
            for (int k = 0; k < nKB; ++k) {
                uint8_t bj = 0;
                for (int wr = 0; wr < warps_m; ++wr)
                    for (int wc = 0; wc < warps_n; ++wc)
                        bj |= a_pat[(size_t)(cr * warps_m + wr) * nKB + k] &
                              b_pat[(size_t)(cc * warps_n + wc) * nKB + k];
                if (bj == 0) {
                    block_skips++;
                    warp_skips += nw;
                    dot_skips += (long long)nw * bk;
                    continue;
                }
                for (int wr = 0; wr < warps_m; ++wr)
                    for (int wc = 0; wc < warps_n; ++wc) {
                        const uint8_t j = a_pat[(size_t)(cr * warps_m + wr) * nKB + k] &
                                          b_pat[(size_t)(cc * warps_n + wc) * nKB + k];
                        if (j == 0) {
                            warp_skips++;
                            dot_skips += bk;
                        } else {
                            dot_skips += bk - __builtin_popcount(j);
                        }
                    }
            }
    const long long total_k = (long long)num_cblocks_m * num_cblocks_n * nKB;
    out[0] = block_skips;
    out[1] = total_k;
    out[2] = warp_skips;
    out[3] = total_k * nw;
    out[4] = dot_skips;
    out[5] = total_k * nw * bk;
}

/*
 * Pattern string -> byte.  String position i is K column i
 * (include/utils.cuh:146-147) and K column i is bit i
 * (src/preprocessors/ab_preprocessor.cu:70), so "11110000" is 0x0F.
 * Returns -1 for anything but eight '0'/'1' characters (driver.cu:195-205).
 */
int oracle_pattern_from_string(const char *s)
{
    if (!s || strlen(s) != 8) return -1;
    int p = 0;
    for (int i = 0; i < 8; ++i) {
        if (s[i] == '1') p |= 1 << i;
        else if (s[i] != '0') return -1;
    }
    return p;
}

/*
 * PatternLUT entry semantics (include/pattern_lut.cuh:13-19): count is the
 * popcount of the pattern, offsets[0..count) are the set bit indices in
 * ascending order (LSB = 0), the rest are 0.
 */
void oracle_pattern_lut(uint8_t pattern, uint8_t *count, uint8_t offsets[8])
{
    uint8_t c = 0;
    memset(offsets, 0, 8);
    for (uint8_t b = 0; b < 8; ++b)
        if (pattern & (1u << b)) offsets[c++] = b;
    *count = c;
}

/* Executed FFMA count at 32x32x1 granularity: sum over (mb, nb, kb) of
 * popcount(a & b) * tile_m * wn (the dot-level "executed" figure of
 * include/runners.cuh:680 scaled to multiply-adds). */
long long oracle_executed_macs(const uint8_t *a_pat, const uint8_t *b_pat, int nMB, int nNB,
                               int nKB, int tile_m, int wn)
{
    long long bits = 0;
    for (int mb = 0; mb < nMB; ++mb)
        for (int nb = 0; nb < nNB; ++nb) {
            const uint8_t *a = a_pat + (size_t)mb * nKB, *b = b_pat + (size_t)nb * nKB;
            for (int kb = 0; kb < nKB; ++kb) bits += __builtin_popcount(a[kb] & b[kb]);
        }
    return bits * tile_m * wn;
}
