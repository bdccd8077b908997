// utils.cuh - the helper half of the reference's header surface (its include/utils.cuh), as thin
// inline wrappers over the C ABI of libesmm_b200 (esmm.h).  Together with runners.cuh beside it, a
// program written against the reference's two headers - its driver.cu - compiles against these
// with no change beyond the include search path.
//
//   CEIL_DIV, PATTERN_LENGTH                                  include/utils.cuh:10-11
//   parse_kernel_selection, get_kernel_name, print_usage      include/utils.cuh:18-101
//   cudaCheckError / cudaAssert                               include/utils.cuh:104-114
//   randomize_matrix_with_pattern, _unstructured              include/utils.cuh:142-194
//   matrixMultiplyCPU, verifyResults                          include/utils.cuh:208-254
//   randomize_matrix_A_blocklevel<BK, WM>,
//   randomize_matrix_B_blocklevel_fixed<BK, WN>,
//   randomize_matrix_A<BK, TILE_M>                            include/utils.cuh:303-426
//
// The generators and the usage text live in the library (host functions); the two short numeric
// helpers whose loop order IS the contract (CPU SGEMM, verification) are spelled out here.
#pragma once

#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <set>
#include <sstream>
#include <string>
#include <string_view>
#include <vector>

#include "esmm.h"

#ifndef CEIL_DIV
#define CEIL_DIV(M, N) (((M) + (N)-1) / (N))
#endif
#ifndef PATTERN_LENGTH
#define PATTERN_LENGTH 8
#endif

using std::cout;
using std::endl;

// driver.cu:20 / include/utils.cuh:16
static const std::set<int> VALID_KERNEL_SET = {14, 15, 16, 17, 20, 21, 25, 26, 27, 28, 29, 30};

#define cudaCheckError(ans)                      \
    {                                            \
        cudaAssert((ans), __FILE__, __LINE__);   \
    }
inline void cudaAssert(cudaError_t code, const char *file, int line)
{
    if (code != cudaSuccess) {
        fprintf(stderr, "CUDA Error: %s %s %d\n", cudaGetErrorString(code), file, line);
        exit(code);
    }
}

inline std::vector<int> parse_kernel_selection(const std::string &input)
{
    int ids[32];
    const int n = esmm_parse_kernel_selection(input.c_str(), ids, 32);
    return std::vector<int>(ids, ids + (n < 0 ? 0 : (n > 32 ? 32 : n)));
}

inline const char *get_kernel_name(int kernel_choice) { return esmm_kernel_name(kernel_choice); }

inline void print_usage(const char *program_name)
{
    std::cout.flush();
    esmm_print_usage(program_name, 0);
}

// ---- generators: same rand() stream, same values as the reference's ---------------------------------
inline void randomize_matrix_with_pattern(float *mat, int M, int N, std::string_view pattern)
{
    const std::string p(pattern);
    esmm_randomize_matrix_with_pattern(mat, M, N, p.c_str());
}

inline void randomize_matrix_unstructured(float *mat, int M, int N, float sparsity_percent, unsigned int seed = 0)
{
    esmm_randomize_matrix_unstructured(mat, M, N, sparsity_percent, seed);
}

template <int BK = 8, int WM = 64>
void randomize_matrix_A_blocklevel(float *mat, int M, int K, float block_sparsity_percent, unsigned int seed = 0)
{
    esmm_randomize_matrix_a_blocklevel(mat, M, K, BK, WM, block_sparsity_percent, seed);
}

template <int BK = 8, int WN = 32>
void randomize_matrix_B_blocklevel_fixed(float *mat, int K, int N, float block_sparsity_percent, unsigned int seed = 0)
{
    esmm_randomize_matrix_b_blocklevel(mat, K, N, BK, WN, block_sparsity_percent, seed);
}

template <int BK = 8, int TILE_M = 8>
void randomize_matrix_A(float *mat, int M, int K, float block_sparsity_percent, unsigned int seed = 0)
{
    esmm_randomize_matrix_a_blocklevel(mat, M, K, BK, TILE_M, block_sparsity_percent, seed);
}

// ---- the driver's CPU SGEMM: i-j-k loops, one sequential k loop per output ------------------------------
inline void matrixMultiplyCPU(const float *A, const float *B, float *C, int M, int N, int K)
{
    for (int i = 0; i < M; i++)
        for (int j = 0; j < N; j++) {
            float sum = 0.0f;
            for (int k = 0; k < K; k++) sum += A[i * K + k] * B[k * N + j];
            C[i * N + j] = sum;
        }
}

// ---- absolute-tolerance check (default 1e-2), the reference's messages ------------------------------------
inline bool verifyResults(const float *gpuResults, const float *cpuResults, int size, float tolerance = 1e-2)
{
    int mismatchCount = 0, firstMismatchIdx = -1;
    float maxDiff = 0.0f;
    for (int i = 0; i < size; i++) {
        const float diff = std::abs(gpuResults[i] - cpuResults[i]);
        if (diff > tolerance) {
            mismatchCount++;
            if (firstMismatchIdx == -1) firstMismatchIdx = i;
            maxDiff = std::max(maxDiff, diff);
        }
    }
    if (mismatchCount == 0) return true;
    std::cout << "Verification failed: " << mismatchCount << " mismatches out of " << size << " elements."
              << std::endl;
    std::cout << "Max difference: " << maxDiff << std::endl;
    // the reference reports the position as if the result were square: side = size / sqrt(size), the row
    // by a floating-point division, the column by the truncated side
    const double side = size / sqrt((double)size);
    const int row = (int)(firstMismatchIdx / side);
    const int col = firstMismatchIdx % (int)side;
    std::cout << "First mismatch at index " << firstMismatchIdx << " (row=" << row << ", col=" << col << "): "
              << "GPU=" << gpuResults[firstMismatchIdx] << ", CPU=" << cpuResults[firstMismatchIdx] << std::endl;
    return false;
}
