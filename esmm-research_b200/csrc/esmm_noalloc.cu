// esmm_sgemm_joint_static: the per-call joint-sparse SGEMM for callers that must not allocate.
//
// Some hosts of this library cannot hand it device memory at call time and cannot let it call
// cudaMalloc either: an inference runtime whose operator contract forbids allocation once the
// engine is built, a process whose framework allocator has already claimed the whole GPU, a
// real-time loop that cannot afford the device-wide synchronisation an allocation implies.  The
// per-call path needs scratch memory (the A pattern bytes and the k-major packed copy of A).
// Here that scratch is a fixed array inside the library image, so the call needs nothing from any
// allocator: no cudaMalloc, no cudaFree, no library routine that allocates.
//
// The price is a fixed ceiling and a fixed cost: the array below is reserved on every GPU that
// loads the library, for as long as the library stays loaded, and A may not need more than it
// holds (ESMM_STATIC_MAX_PACKED_FLOATS packed floats, ESMM_STATIC_MAX_PATTERN_BYTES pattern bytes).
//
// All calls on one GPU share the one array.  It keeps whatever the previous call left there;
// nothing in it has to start at zero, because every call rewrites the pattern bytes it reads and
// never multiplies a packed entry it did not write.  Two calls whose kernels overlap on the same
// GPU (different streams, different host threads) race on the array and corrupt each other.
#include <cstdio>

#include "esmm_common.cuh"

namespace esmm {

int gemm_ab_packed_launch_form(int M, int N, int K, const float *d_a_packed, const float *d_B, float *d_C,
                               const uint8_t *d_a_pat, const uint8_t *d_b_pat, cudaStream_t stream, bool follow_hint);
int preprocess_a_pack_launch(const float *d_A, int M, int K, uint8_t *d_out, float *d_packed,
                             cudaStream_t stream);

constexpr size_t STATIC_PATTERN_BYTES = ESMM_STATIC_MAX_PATTERN_BYTES;                      // 64 KiB
constexpr size_t STATIC_PACKED_BYTES = (size_t)ESMM_STATIC_MAX_PACKED_FLOATS * sizeof(float);  // 32 MiB

// Pattern bytes first, packed copy after them (both regions 256-byte aligned).
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_PATTERN_BYTES + STATIC_PACKED_BYTES];

// In host code `g_static_scratch` is only a handle for the runtime, not an address a kernel can
// use; the device address is looked up once per device, with that device current.
static unsigned char *static_scratch_for_current_device(int *status)
{
    static unsigned char *ptrs[64] = {nullptr};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        *status = record_cuda_error(e == cudaSuccess ? cudaErrorInvalidDevice : e, "cudaGetDevice");
        return nullptr;
    }
    if (!ptrs[dev]) {
        unsigned char *p = nullptr;
        e = cudaGetSymbolAddress((void **)&p, g_static_scratch);
        if (e != cudaSuccess || !p) {
            *status = record_cuda_error(e == cudaSuccess ? cudaErrorInvalidSymbol : e,
                                        "cudaGetSymbolAddress(static scratch)");
            return nullptr;
        }
        ptrs[dev] = p;
    }
    *status = ESMM_OK;
    return ptrs[dev];
}

}  // namespace esmm

extern "C" int esmm_sgemm_joint_static(int M, int N, int K, const float *d_A, const float *d_B, float *d_C,
                                       const uint8_t *d_b_pat, void *stream)
{
    if (!d_A || !d_B || !d_C || !d_b_pat) return ESMM_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || (K & 3) || (N & 3)) return ESMM_ERR_SHAPE;
    const size_t pattern_bytes = esmm_a_pattern_bytes(M, K, 32);
    const size_t packed_bytes = esmm_a_packed_bytes(M, K);
    if (pattern_bytes > esmm::STATIC_PATTERN_BYTES || packed_bytes > esmm::STATIC_PACKED_BYTES) {
        char msg[200];
        snprintf(msg, sizeof msg,
                 "esmm_sgemm_joint_static: A of %d x %d needs %zu pattern bytes and %zu packed bytes; the static "
                 "scratch holds %zu and %zu",
                 M, K, pattern_bytes, packed_bytes, esmm::STATIC_PATTERN_BYTES, esmm::STATIC_PACKED_BYTES);
        esmm::record_cuda_error_text(msg);
        return ESMM_ERR_TOO_LARGE;
    }
    int st = ESMM_OK;
    unsigned char *scratch = esmm::static_scratch_for_current_device(&st);
    if (!scratch) return st;
    uint8_t *a_pat = scratch;
    float *a_packed = reinterpret_cast<float *>(scratch + esmm::STATIC_PATTERN_BYTES);
    st = esmm::preprocess_a_pack_launch(d_A, M, K, a_pat, a_packed, (cudaStream_t)stream);
    if (st != ESMM_OK) return st;
    return esmm::gemm_ab_packed_launch_form(M, N, K, a_packed, d_B, d_C, a_pat, d_b_pat, (cudaStream_t)stream, false);
}
