// Host-only entry points of libesmm_b200: the harness's rand()-based matrix generators and its usage
// text.  Nothing here touches a device.
//
// The generators restate include/utils.cuh:142-194 and :303-426 of the reference draw for draw: they
// consume the C library's rand() stream in the same order and round exactly where the reference's
// expressions round, so that for a given seed the driver multiplies the same matrices as the
// reference driver does.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../../include/esmm.h"

namespace {

// Element value of the default and --random modes (include/utils.cuh:148-149, 181-182): the fraction
// is scaled by the DOUBLE constant 0.01 and added in double, the sum is rounded to float once, and
// the sign is kept when rand() is EVEN.  The three rand() calls happen in source order.
inline float draw_value_double_even()
{
    const int whole = rand() % 5;
    const int frac = rand() % 5;
    const float v = (float)((double)(float)whole + 0.01 * (double)frac);
    return (rand() % 2 == 0) ? v : -v;
}

// Element value of the block-level generators (include/utils.cuh:332-333, 372-373, 417-418): float
// constant 0.01f, float arithmetic, sign kept when rand() is ODD.
inline float draw_value_float_odd()
{
    const int whole = rand() % 5;
    const int frac = rand() % 5;
    const float v = (float)whole + 0.01f * (float)frac;
    return (rand() % 2) ? v : -v;
}

// One random 8-bit tile pattern: bit b live when rand() / RAND_MAX >= threshold (utils.cuh:315-320).
inline unsigned draw_tile_pattern(int bk, float threshold)
{
    unsigned pat = 0;
    for (int bit = 0; bit < bk; ++bit)
        if ((float)rand() / RAND_MAX >= threshold) pat |= 1u << bit;
    return pat;
}

bool pattern_string_ok(const char *p)
{
    if (!p || strlen(p) != 8) return false;
    for (int i = 0; i < 8; ++i)
        if (p[i] != '0' && p[i] != '1') return false;
    return true;
}

}  // namespace

extern "C" {

int esmm_randomize_matrix_with_pattern(float *h_mat, int M, int N, const char *pattern)
{
    if (!h_mat || !pattern) return ESMM_ERR_NULL;
    if (M <= 0 || N <= 0 || !pattern_string_ok(pattern)) return ESMM_ERR_SHAPE;
    for (int i = 0; i < M; ++i)
        for (int j = 0; j < N; ++j)
            h_mat[(size_t)i * N + j] = pattern[j % 8] == '1' ? draw_value_double_even() : 0.0f;
    return ESMM_OK;
}

int esmm_randomize_matrix_unstructured(float *h_mat, int M, int N, float sparsity_percent, unsigned seed)
{
    if (!h_mat) return ESMM_ERR_NULL;
    if (M <= 0 || N <= 0) return ESMM_ERR_SHAPE;
    if (seed != 0) srand(seed);
    const float threshold = sparsity_percent / 100.0f;
    int zeros = 0;
    for (int i = 0; i < M; ++i)
        for (int j = 0; j < N; ++j) {
            const float prob = (float)rand() / (float)RAND_MAX;
            if (prob < threshold) {
                h_mat[(size_t)i * N + j] = 0.0f;
                ++zeros;
            } else {
                h_mat[(size_t)i * N + j] = draw_value_double_even();
            }
        }
    const float actual = 100.0f * zeros / (M * N);
    if (fabs(actual - sparsity_percent) > 2.0f)
        printf("  Note: Requested %.1f%% sparsity, achieved %.2f%% (%d/%d zeros)\n", sparsity_percent, actual, zeros,
               M * N);
    return ESMM_OK;
}

int esmm_randomize_matrix_a_blocklevel(float *h_mat, int M, int K, int bk, int tile_m, float block_sparsity_percent,
                                       unsigned seed)
{
    if (!h_mat) return ESMM_ERR_NULL;
    if (M <= 0 || K <= 0 || bk <= 0 || bk > 8 || tile_m <= 0) return ESMM_ERR_SHAPE;
    if (seed != 0) srand(seed);
    const float threshold = block_sparsity_percent / 100.0f;
    for (int mb = 0; mb < M / tile_m; ++mb)
        for (int kb = 0; kb < K / bk; ++kb) {
            const unsigned pat = draw_tile_pattern(bk, threshold);
            for (int row = 0; row < tile_m; ++row)
                for (int k = 0; k < bk; ++k)
                    h_mat[(size_t)(mb * tile_m + row) * K + kb * bk + k] =
                        ((pat >> k) & 1u) ? draw_value_float_odd() : 0.0f;
        }
    return ESMM_OK;
}

int esmm_randomize_matrix_b_blocklevel(float *h_mat, int K, int N, int bk, int wn, float block_sparsity_percent,
                                       unsigned seed)
{
    if (!h_mat) return ESMM_ERR_NULL;
    if (N <= 0 || K <= 0 || bk <= 0 || bk > 8 || wn <= 0) return ESMM_ERR_SHAPE;
    if (seed != 0) srand(seed);
    const float threshold = block_sparsity_percent / 100.0f;
    for (int nb = 0; nb < N / wn; ++nb)
        for (int kb = 0; kb < K / bk; ++kb) {
            const unsigned pat = draw_tile_pattern(bk, threshold);
            for (int col = 0; col < wn; ++col)
                for (int k = 0; k < bk; ++k)
                    h_mat[(size_t)(kb * bk + k) * N + nb * wn + col] =
                        ((pat >> k) & 1u) ? draw_value_float_odd() : 0.0f;
        }
    return ESMM_OK;
}

void esmm_print_usage(const char *program_name, int additive)
{
    static const char *const kernels[][2] = {
        {"14", "A-Only Sparse (Offset List, Templated Dispatch)"},
        {"15", "cuBLAS baseline"},
        {"16", "A-Sparse Block-wise (Warp-Granularity Patterns)"},
        {"17", "B-Sparse Warp-Granularity (32-col, Zero-Divergence)"},
        {"20", "A+B Sparse OPTIMIZED (Zero-Overhead Inner Loop)"},
        {"21", "A+B Sparse - 8x32 Granularity"},
        {"25", "A+B Simple Fused (Main Contribution)"},
        {"26", "A+B Optimized V2 (K20 + 32-row + Block Skip + Float4)"},
        {"27", "A+B Ablation (32-row only, no Block Skip, no Float4)"},
        {"28", "A+B GMem-32 (K25 with 32-row, global mem patterns)"},
        {"29", "A+B Optimized V3 (K26 + templated smem + float2 A-loads)"},
        {"30", "A+B Compressed-K (K29 + compressed K-list + set-bit dotIdx)"},
    };
    const char *prog = program_name ? program_name : "exec";
    printf("Usage: %s [kernel_choice] [runs] [options]\n", prog);
    printf("\nAvailable kernels: 14, 15, 16, 17, 20, 21, 25, 26, 27, 28, 29, 30%s\n", additive ? " (and 129)" : "");
    for (const auto &k : kernels) printf("  %s: %s\n", k[0], k[1]);
    if (additive) printf("  129: A+B 3xTF32 on tensor cores (additive: not in the reference, not part of 'all')\n");
    printf("\nKernel selection formats:\n");
    printf("  Single:   29          (run K29)\n");
    printf("  Multiple: \"29,15\"     (comma-separated)\n");
    printf("  Range:    \"14-17\"    (kernels in range that are valid)\n");
    printf("  All:      all         (all kernels)\n");
    printf("\nOptions:\n");
    printf("  --verbose, -v       Enable verbose output\n");
    printf("  --no-check, -n      Skip result verification (performance-only mode)\n");
    printf("  --random, -r        Use random unstructured sparsity\n");
    printf("  --blockwise, -b     Use block-level sparsity (random per-tile patterns)\n");
    printf("  --size <N>, -s <N>  Set matrix dimensions NxNxN (default: 4096)\n");
    printf("  --pattern <P>       Set 8-bit sparsity pattern for A and B (default: \"11000000\")\n");
    printf("  --pattern-a <P>     Set 8-bit sparsity pattern for A matrix only\n");
    printf("  --pattern-b <P>     Set 8-bit sparsity pattern for B matrix only\n");
    printf("  --load-a/--load-b <file>  Raw float32 row-major matrices (with --dims M K N)\n");
    printf("  --skip-stats        Print block / warp / k skip statistics\n");
    if (additive) {
        printf("  --uniform           N(0,1) values, pattern on A's K columns and B's K rows (device generator)\n");
        printf("  --tile-random pA pB N(0,1) values, independent 64-row / 64-column tile patterns\n");
        printf("  --tile-gran <G>     Rows of A / columns of B per tile of --tile-random (default 64)\n");
        printf("  --tune <NAME=VALUE> Pin one of the library's launch heuristics (names: esmm_tuning_set in esmm.h)\n");
        printf("  --shape M K N       Generated data on a non-cubic problem\n");
        printf("  --seed <S>          Seed for --uniform / --tile-random\n");
        printf("  --cpu-check         Also verify against the CPU SGEMM (rel-inf tolerance 1e-4)\n");
        printf("  --cache-b           Cache B's pattern bytes next to the --load-b file (<file>.bpat)\n");
        printf("  --cache-b-file <f>  Cache B's pattern bytes in <f>\n");
        printf("  --gpus <G>          Shard B and C by columns over G GPUs of this machine (kernel 29)\n");
        printf("  --gather            With --gpus: collect C on GPU 0 (NCCL all-gather) before verification\n");
        printf("  --json              One JSON line per kernel\n");
    }
    printf("  --help, -h          Show this help message\n");
    printf("\nExamples:\n");
    printf("  %s 29,15 10 --blockwise --pattern 11110000 --size 4096 --verbose\n", prog);
    if (additive) printf("  %s 29 10 --uniform --pattern 10000000 --size 4096 --cpu-check\n", prog);
    printf("  %s 29 5 --load-b W.bin --dims 2048 4096 11008 --no-check\n", prog);
    fflush(stdout);
}

}  // extern "C"
