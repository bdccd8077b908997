// cusparse_bench - cuSPARSE SpMM next to the joint-sparse kernel and cuBLAS on one square problem.
//
// Command line and first six CSV columns of the reference's standalone benchmark
// (src/benchmarks/cusparse_benchmark.cu:56-68, 232):
//
//   cusparse_bench [--size N] [--density D] [--runs R] [--header] [--compare]
//   size,density,spmm_us,total_us,spmm_gflops,total_gflops
//
// A is N x N with independent 64-row x 8-column tiles, each live with probability D (the reference's
// fill_blockwise_sparse, :30-47), B is dense.  --compare appends the joint-sparse path (A packing +
// GEMM per call, B patterns computed once) and cuBLAS SGEMM on the same matrices, and the largest
// relative difference between the cuSPARSE and the joint-sparse result:
//
//   ...,esmm_us,cublas_us,rel_diff
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "include/esmm.h"

#define CK(x)                                                                              \
    do {                                                                                   \
        int _st = (x);                                                                     \
        if (_st != ESMM_OK) {                                                              \
            fprintf(stderr, "%s: %s %s\n", #x, esmm_strerror(_st), esmm_last_cuda_error()); \
            return 1;                                                                      \
        }                                                                                  \
    } while (0)

int main(int argc, char **argv)
{
    int n = 4096, runs = 10;
    float density = 0.5f;
    bool header = false, compare = false;
    for (int i = 1; i < argc; ++i) {
        if (!strcmp(argv[i], "--size") && i + 1 < argc) n = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--density") && i + 1 < argc) density = (float)atof(argv[++i]);
        else if (!strcmp(argv[i], "--runs") && i + 1 < argc) runs = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--header")) header = true;
        else if (!strcmp(argv[i], "--compare")) compare = true;
    }
    if (header) {
        printf("size,density,spmm_us,total_us,spmm_gflops,total_gflops%s\n", compare ? ",esmm_us,cublas_us,rel_diff" : "");
        return 0;
    }
    if (n <= 0 || n % 8 || runs <= 0 || density < 0.f || density > 1.f) {
        fprintf(stderr, "Error: --size must be a positive multiple of 8, --runs positive, --density in [0, 1]\n");
        return 1;
    }
    const size_t elems = (size_t)n * n;
    float *dA, *dB, *dC, *dC2;
    if (cudaMalloc(&dA, elems * 4) || cudaMalloc(&dB, elems * 4) || cudaMalloc(&dC, elems * 4) || cudaMalloc(&dC2, elems * 4)) {
        fprintf(stderr, "cudaMalloc failed\n");
        return 1;
    }
    // whole 64 x 8 tiles live with probability `density`: tile mode with all 8 offsets of a tile sharing
    // one draw is not what esmm_fill_normal offers, so the tiles are drawn on the host and applied there
    std::vector<float> hA(elems);
    CK(esmm_fill_normal(dA, n, n, 0, 42, 0.f, 1.f, 0, 0, 0xFF, 1.f, 64, 0, nullptr));
    cudaMemcpy(hA.data(), dA, elems * 4, cudaMemcpyDeviceToHost);
    srand(42);
    for (int bm = 0; bm < (n + 63) / 64; ++bm)
        for (int bk = 0; bk < n / 8; ++bk)
            if (!((float)rand() / (float)RAND_MAX < density))
                for (int r = bm * 64; r < n && r < bm * 64 + 64; ++r) memset(&hA[(size_t)r * n + bk * 8], 0, 32);
    cudaMemcpy(dA, hA.data(), elems * 4, cudaMemcpyHostToDevice);
    CK(esmm_fill_normal(dB, n, n, 1, 43, 0.f, 1.f, 0, 0, 0xFF, 1.f, 64, 0, nullptr));

    float spmm_ms = 0.f, total_ms = 0.f;
    long long nnz = 0;
    CK(esmm_cusparse_spmm(n, n, n, dA, dB, dC, runs, &spmm_ms, &total_ms, &nnz));
    const double flops = 2.0 * (double)nnz * n;   // the work SpMM does, not 2 N^3
    printf("%d,%.4f,%.3f,%.3f,%.2f,%.2f", n, density, spmm_ms * 1e3, total_ms * 1e3, flops / (spmm_ms * 1e-3) / 1e9,
           flops / (total_ms * 1e-3) / 1e9);
    if (compare) {
        uint8_t *bpat;
        void *ws;
        cudaMalloc(&bpat, esmm_b_pattern_bytes(n, n));
        cudaMalloc(&ws, esmm_sgemm_joint_workspace_bytes(n, n));
        CK(esmm_preprocess_b(dB, n, n, bpat, nullptr));
        cudaEvent_t t0, t1;
        cudaEventCreate(&t0);
        cudaEventCreate(&t1);
        float ms_esmm = 0.f, ms_blas = 0.f;
        for (int pass = 0; pass < 2; ++pass) {
            for (int i = 0; i < 3; ++i)
                CK(pass == 0 ? esmm_sgemm_joint(n, n, n, dA, dB, dC2, bpat, ws, nullptr) : esmm_cublas_sgemm(n, n, n, dA, dB, dC, nullptr));
            cudaEventRecord(t0);
            for (int i = 0; i < runs; ++i)
                CK(pass == 0 ? esmm_sgemm_joint(n, n, n, dA, dB, dC2, bpat, ws, nullptr) : esmm_cublas_sgemm(n, n, n, dA, dB, dC, nullptr));
            cudaEventRecord(t1);
            cudaEventSynchronize(t1);
            cudaEventElapsedTime(pass == 0 ? &ms_esmm : &ms_blas, t0, t1);
        }
        CK(esmm_device_status(nullptr));
        // cuSPARSE result once more into dC (cuBLAS overwrote it), then compare with the joint-sparse C
        CK(esmm_cusparse_spmm(n, n, n, dA, dB, dC, 1, nullptr, nullptr, nullptr));
        std::vector<float> h1(elems), h2(elems);
        cudaMemcpy(h1.data(), dC, elems * 4, cudaMemcpyDeviceToHost);
        cudaMemcpy(h2.data(), dC2, elems * 4, cudaMemcpyDeviceToHost);
        double num = 0, den = 0;
        for (size_t i = 0; i < elems; ++i) {
            const double d = fabs((double)h1[i] - h2[i]);
            if (d > num) num = d;
            if (fabs((double)h2[i]) > den) den = fabs((double)h2[i]);
        }
        printf(",%.3f,%.3f,%.3g", ms_esmm / runs * 1e3, ms_blas / runs * 1e3, den > 0 ? num / den : num);
    }
    printf("\n");
    return 0;
}
