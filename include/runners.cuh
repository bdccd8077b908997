// runners.cuh - the reference's operator surface for the joint-sparse path, as thin inline
// wrappers over the C ABI of libesmm_b200 (include/esmm.h).
//
// A program written against the reference's include/runners.cuh, include/utils.cuh and
// src/preprocessors/ab_preprocessor.cu (as its driver.cu is) compiles against this header with the
// same names and argument lists:
//
//   run_esmm_ab_optimized_v3 (+ 9-argument overload, _no_check)   include/runners.cuh:827-897
//   run_cuBlas, run_cuBlas_no_check                                 include/runners.cuh:109-144
//   the other joint-sparse runners (ids 20, 21, 25, 26, 27, 28, 30) include/runners.cuh:278-995
//   the single-operand runners (ids 14, 16, 17)                     include/runners.cuh:30-106, 150-275
//   preprocess_ab<BK, TILE_M_A, WN>, ABPatternMetadata,
//   free_ab_pattern_metadata                                        src/preprocessors/ab_preprocessor.cu:7-24, 297-326
//
// The helper half of the reference's surface (parse_kernel_selection, get_kernel_name, print_usage,
// the generators, verifyResults, matrixMultiplyCPU, cudaCheckError, CEIL_DIV) is utils.cuh beside this
// file, which this header includes.
//
// Argument naming follows the reference: rows = M, cols = N, inners = K.  Nothing here launches a
// kernel itself; every call goes through the extern "C" entry points.
#pragma once

#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <string>
#include <string_view>
#include <vector>

#include "esmm.h"

#include "utils.cuh"

// ---- src/preprocessors/ab_preprocessor.cu ---------------------------------------------------------
using ABPatternMetadata = esmm_ab_pattern_metadata;

inline void free_ab_pattern_metadata(ABPatternMetadata &meta) { esmm_free_ab_pattern_metadata(&meta); }

template <const int BK = 8, const int TILE_M_A = 64, const int WN = 32>
ABPatternMetadata preprocess_ab(const float *d_A, const float *d_B, int M, int N, int K)
{
    static_assert(BK == 8 && WN == 32, "the pattern format is 8 K offsets per byte, 32 columns per B block");
    ABPatternMetadata meta;
    const int st = esmm_preprocess_ab(d_A, d_B, M, N, K, TILE_M_A, nullptr, &meta);
    if (st != ESMM_OK) fprintf(stderr, "preprocess_ab: %s %s\n", esmm_strerror(st), esmm_last_cuda_error());
    return meta;
}

// ---- include/runners.cuh -------------------------------------------------------------------------
namespace esmm_runner_detail {
inline bool run(int id, int rows, int cols, int inners, float *d_A, float *d_B, float *d_C, float *h_C,
                float *h_C_ref, int runs, bool verify, bool print_skip_stats)
{
    int passed = 0;
    const int st = esmm_run_kernel(id, rows, cols, inners, d_A, d_B, d_C, h_C, h_C_ref, runs, verify ? 1 : 0,
                                   print_skip_stats ? 1 : 0, &passed, nullptr);
    if (st != ESMM_OK && st != ESMM_ERR_VERIFY)
        printf("ESMM runner error (kernel %d): %s %s\n", id, esmm_strerror(st), esmm_last_cuda_error());
    return st == ESMM_OK && passed != 0;
}
}  // namespace esmm_runner_detail

inline void run_cuBlas(int rows, int cols, int inners, float *d_A, float *d_B, float *d_C, float *h_C, int runs)
{
    esmm_run_kernel(15, rows, cols, inners, d_A, d_B, d_C, h_C, nullptr, runs, 0, 0, nullptr, nullptr);
}
inline void run_cuBlas_no_check(int rows, int cols, int inners, float *d_A, float *d_B, float *d_C, int runs)
{
    run_cuBlas(rows, cols, inners, d_A, d_B, d_C, nullptr, runs);
}

#define ESMM_DEFINE_RUNNER(NAME, ID)                                                                             \
    inline bool NAME(int rows, int cols, int inners, float *d_A, float *d_B, float *d_C, float *h_C,            \
                     float *h_C_ref, int runs, bool verify, bool print_skip_stats = false)                      \
    {                                                                                                            \
        return esmm_runner_detail::run(ID, rows, cols, inners, d_A, d_B, d_C, h_C, h_C_ref, runs, verify,       \
                                       print_skip_stats);                                                        \
    }                                                                                                            \
    inline bool NAME(int rows, int cols, int inners, float *d_A, float *d_B, float *d_C, float *h_C,            \
                     float *h_C_ref, int runs)                                                                   \
    {                                                                                                            \
        return NAME(rows, cols, inners, d_A, d_B, d_C, h_C, h_C_ref, runs, true, false);                         \
    }                                                                                                            \
    inline bool NAME##_no_check(int rows, int cols, int inners, float *d_A, float *d_B, float *d_C, int runs,   \
                                bool print_skip_stats = false)                                                   \
    {                                                                                                            \
        return NAME(rows, cols, inners, d_A, d_B, d_C, nullptr, nullptr, runs, false, print_skip_stats);         \
    }

ESMM_DEFINE_RUNNER(run_esmm_ab_optimized_v3, 29)
ESMM_DEFINE_RUNNER(run_esmm_ab_sparse_optimized, 20)
ESMM_DEFINE_RUNNER(run_esmm_ab_8x32, 21)
ESMM_DEFINE_RUNNER(run_esmm_ab_simple_fused, 25)
ESMM_DEFINE_RUNNER(run_esmm_ab_optimized_v2, 26)
ESMM_DEFINE_RUNNER(run_esmm_ab_optimized_v2_baseline, 27)
ESMM_DEFINE_RUNNER(run_esmm_ab_gmem_32, 28)
ESMM_DEFINE_RUNNER(run_esmm_ab_compressed_k, 30)
#undef ESMM_DEFINE_RUNNER

// The single-operand ids (include/runners.cuh:30-106, 150-211, 214-275): the reference's argument lists,
// which have no skip-stats flag; id 14 also takes the driver's pattern string.
inline bool run_esmm_a_sparse_blockwise(int rows, int cols, int inners, float *d_A, float *d_B, float *d_C,
                                        float *h_C, float *h_C_ref, int runs, bool verify = true)
{
    return esmm_runner_detail::run(16, rows, cols, inners, d_A, d_B, d_C, h_C, h_C_ref, runs, verify, false);
}
inline bool run_esmm_a_sparse_blockwise_no_check(int rows, int cols, int inners, float *d_A, float *d_B,
                                                 float *d_C, int runs)
{
    return run_esmm_a_sparse_blockwise(rows, cols, inners, d_A, d_B, d_C, nullptr, nullptr, runs, false);
}
inline bool run_esmm_b_sparse_warp(int rows, int cols, int inners, float *d_A, float *d_B, float *d_C,
                                   float *h_C, float *h_C_ref, int runs, bool verify = true)
{
    return esmm_runner_detail::run(17, rows, cols, inners, d_A, d_B, d_C, h_C, h_C_ref, runs, verify, false);
}
inline bool run_esmm_b_sparse_warp_no_check(int rows, int cols, int inners, float *d_A, float *d_B,
                                            float *d_C, int runs)
{
    return run_esmm_b_sparse_warp(rows, cols, inners, d_A, d_B, d_C, nullptr, nullptr, runs, false);
}
inline bool run_esmm_unrolled(int rows, int cols, int inners, float *d_A, float *d_B, float *d_C, float *h_C,
                              float *h_C_ref, int runs, std::string_view pattern, bool verify = true)
{
    int passed = 0;
    const std::string pat(pattern);
    const int st = esmm_run_kernel_pattern(14, rows, cols, inners, d_A, d_B, d_C, h_C, h_C_ref, runs, verify ? 1 : 0,
                                           0, nullptr, pat.c_str(), &passed, nullptr);
    return st == ESMM_OK && passed != 0;
}
inline bool run_esmm_unrolled_no_check(int rows, int cols, int inners, float *d_A, float *d_B, float *d_C,
                                       int runs, std::string_view pattern)
{
    return run_esmm_unrolled(rows, cols, inners, d_A, d_B, d_C, nullptr, nullptr, runs, pattern, false);
}
