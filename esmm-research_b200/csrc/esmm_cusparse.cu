// cuSPARSE SpMM as a second comparison baseline: A (row-major, dense storage, block-sparse content)
// converted to CSR and multiplied with dense B.  Covers what the reference measures with its
// standalone binary src/benchmarks/cusparse_benchmark.cu (:56-247): two timing bands, "SpMM only"
// (A already in CSR) and "total" (dense -> CSR conversion + SpMM per call, the fair counterpart of
// "A preprocessed per call"), and the effective flop count 2 * nnz * N.  Library calls only; nothing
// here is on the product path.
#include <cusparse.h>

#include "esmm_common.cuh"

namespace esmm {

struct SpmmState {
    cusparseHandle_t handle = nullptr;
    cusparseDnMatDescr_t dnA = nullptr, dnB = nullptr, dnC = nullptr;
    cusparseSpMatDescr_t spA = nullptr;
    int32_t *offsets = nullptr, *cols = nullptr;
    float *vals = nullptr;
    void *conv_buf = nullptr, *spmm_buf = nullptr;
    cudaEvent_t t0 = nullptr, t1 = nullptr;
    ~SpmmState()
    {
        if (dnA) cusparseDestroyDnMat(dnA);
        if (dnB) cusparseDestroyDnMat(dnB);
        if (dnC) cusparseDestroyDnMat(dnC);
        if (spA) cusparseDestroySpMat(spA);
        if (handle) cusparseDestroy(handle);
        cudaFree(offsets);
        cudaFree(cols);
        cudaFree(vals);
        cudaFree(conv_buf);
        cudaFree(spmm_buf);
        if (t0) cudaEventDestroy(t0);
        if (t1) cudaEventDestroy(t1);
    }
};

#define ESMM_SPARSE_TRY(expr)                                                         \
    do {                                                                              \
        cusparseStatus_t _s = (expr);                                                 \
        if (_s != CUSPARSE_STATUS_SUCCESS) {                                          \
            char _msg[400];                                                           \
            snprintf(_msg, sizeof _msg, "%s: %s", #expr, cusparseGetErrorString(_s)); \
            return record_cuda_error_text(_msg);                                      \
        }                                                                             \
    } while (0)

}  // namespace esmm

extern "C" int esmm_cusparse_spmm(int M, int N, int K, const float *d_A, const float *d_B, float *d_C, int runs,
                                  float *spmm_ms, float *total_ms, long long *nnz_out)
{
    using namespace esmm;
    if (!d_A || !d_B || !d_C) return ESMM_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || runs <= 0) return ESMM_ERR_SHAPE;
    SpmmState s;
    const float alpha = 1.0f, beta = 0.0f;
    ESMM_SPARSE_TRY(cusparseCreate(&s.handle));
    ESMM_SPARSE_TRY(cusparseCreateDnMat(&s.dnA, M, K, K, const_cast<float *>(d_A), CUDA_R_32F, CUSPARSE_ORDER_ROW));
    ESMM_SPARSE_TRY(cusparseCreateDnMat(&s.dnB, K, N, N, const_cast<float *>(d_B), CUDA_R_32F, CUSPARSE_ORDER_ROW));
    ESMM_SPARSE_TRY(cusparseCreateDnMat(&s.dnC, M, N, N, d_C, CUDA_R_32F, CUSPARSE_ORDER_ROW));
    ESMM_CUDA_TRY(cudaMalloc(&s.offsets, (size_t)(M + 1) * sizeof(int32_t)));
    ESMM_SPARSE_TRY(cusparseCreateCsr(&s.spA, M, K, 0, s.offsets, nullptr, nullptr, CUSPARSE_INDEX_32I,
                                      CUSPARSE_INDEX_32I, CUSPARSE_INDEX_BASE_ZERO, CUDA_R_32F));
    size_t conv_bytes = 0, spmm_bytes = 0;
    ESMM_SPARSE_TRY(cusparseDenseToSparse_bufferSize(s.handle, s.dnA, s.spA, CUSPARSE_DENSETOSPARSE_ALG_DEFAULT,
                                                     &conv_bytes));
    ESMM_CUDA_TRY(cudaMalloc(&s.conv_buf, conv_bytes ? conv_bytes : 1));
    ESMM_SPARSE_TRY(cusparseDenseToSparse_analysis(s.handle, s.dnA, s.spA, CUSPARSE_DENSETOSPARSE_ALG_DEFAULT,
                                                   s.conv_buf));
    int64_t r64 = 0, c64 = 0, nnz = 0;
    ESMM_SPARSE_TRY(cusparseSpMatGetSize(s.spA, &r64, &c64, &nnz));
    if (nnz_out) *nnz_out = (long long)nnz;
    ESMM_CUDA_TRY(cudaMalloc(&s.cols, (size_t)(nnz ? nnz : 1) * sizeof(int32_t)));
    ESMM_CUDA_TRY(cudaMalloc(&s.vals, (size_t)(nnz ? nnz : 1) * sizeof(float)));
    ESMM_SPARSE_TRY(cusparseCsrSetPointers(s.spA, s.offsets, s.cols, s.vals));
    auto convert = [&]() {
        return cusparseDenseToSparse_convert(s.handle, s.dnA, s.spA, CUSPARSE_DENSETOSPARSE_ALG_DEFAULT, s.conv_buf);
    };
    ESMM_SPARSE_TRY(convert());
    ESMM_SPARSE_TRY(cusparseSpMM_bufferSize(s.handle, CUSPARSE_OPERATION_NON_TRANSPOSE,
                                            CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, s.spA, s.dnB, &beta, s.dnC,
                                            CUDA_R_32F, CUSPARSE_SPMM_ALG_DEFAULT, &spmm_bytes));
    ESMM_CUDA_TRY(cudaMalloc(&s.spmm_buf, spmm_bytes ? spmm_bytes : 1));
    auto spmm = [&]() {
        return cusparseSpMM(s.handle, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha,
                            s.spA, s.dnB, &beta, s.dnC, CUDA_R_32F, CUSPARSE_SPMM_ALG_DEFAULT, s.spmm_buf);
    };
    ESMM_CUDA_TRY(cudaEventCreate(&s.t0));
    ESMM_CUDA_TRY(cudaEventCreate(&s.t1));
    float ms = 0.f;
    // band 1: SpMM alone, 3 warm-up calls
    for (int i = 0; i < 3; ++i) ESMM_SPARSE_TRY(spmm());
    ESMM_CUDA_TRY(cudaDeviceSynchronize());
    ESMM_CUDA_TRY(cudaEventRecord(s.t0));
    for (int i = 0; i < runs; ++i) ESMM_SPARSE_TRY(spmm());
    ESMM_CUDA_TRY(cudaEventRecord(s.t1));
    ESMM_CUDA_TRY(cudaEventSynchronize(s.t1));
    ESMM_CUDA_TRY(cudaEventElapsedTime(&ms, s.t0, s.t1));
    if (spmm_ms) *spmm_ms = ms / runs;
    // band 2: conversion + SpMM per call
    for (int i = 0; i < 3; ++i) {
        ESMM_SPARSE_TRY(convert());
        ESMM_SPARSE_TRY(spmm());
    }
    ESMM_CUDA_TRY(cudaDeviceSynchronize());
    ESMM_CUDA_TRY(cudaEventRecord(s.t0));
    for (int i = 0; i < runs; ++i) {
        ESMM_SPARSE_TRY(convert());
        ESMM_SPARSE_TRY(spmm());
    }
    ESMM_CUDA_TRY(cudaEventRecord(s.t1));
    ESMM_CUDA_TRY(cudaEventSynchronize(s.t1));
    ESMM_CUDA_TRY(cudaEventElapsedTime(&ms, s.t0, s.t1));
    if (total_ms) *total_ms = ms / runs;
    return ESMM_OK;
}
