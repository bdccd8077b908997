// A/B pattern preprocessor for sm_100a: one coalesced pass over the matrix, 16-byte loads,
// row reduction in registers, packed stores.  Pattern bytes are bit-exact with
// preprocess_a_patterns_kernel / preprocess_b_patterns_kernel of the reference
// (src/preprocessors/ab_preprocessor.cu:31-84, :91-144).
//
// Kernel names keep "preprocess" in them: the reference's sweep scripts split timings by
// that substring (scripts/benchmark.py:456-458).
#include <cstdio>
#include <cstring>

#include "esmm_common.cuh"

namespace esmm {

constexpr int PRE_THREADS = 128;

// `v != 0.0f` as an integer test: -0.0f is zero, NaN and denormals are nonzero.
__device__ __forceinline__ unsigned nz(float v) { return (__float_as_uint(v) << 1) != 0u; }

__device__ __forceinline__ unsigned nz4(const float4 &v)
{
    return nz(v.x) | (nz(v.y) << 1) | (nz(v.z) << 2) | (nz(v.w) << 3);
}

// One warp owns tile_m rows x 128 columns (16 K blocks).  Lane l reads columns 4l..4l+3 of
// every row (one 512-byte request per row per warp), ORs the nonzero bits of its 4 columns
// over the rows in registers, then pairs of lanes join their nibbles into a pattern byte.
// Needs K % 4 == 0 and a 16-byte aligned A.
__global__ void __launch_bounds__(PRE_THREADS)
esmm_preprocess_a_patterns_kernel(const float *__restrict__ A, int M, int K, int tile_m, int nMB,
                                  int nKB, int k_chunks, uint8_t *__restrict__ out, int *status)
{
    // checked build, sites 10 (loads of A) and 11 (pattern stores)
    const size_t a_floats = (size_t)M * K, out_bytes = (size_t)nMB * nKB;
    const int lane = threadIdx.x & 31;
    const long warps_total = (long)gridDim.x * (PRE_THREADS / 32);
    const long tasks = (long)nMB * k_chunks;
    for (long task = (long)blockIdx.x * (PRE_THREADS / 32) + (threadIdx.x >> 5); task < tasks;
         task += warps_total) {
        const int mb = (int)(task / k_chunks);
        const int kc = (int)(task - (long)mb * k_chunks);
        const int col = kc * 128 + lane * 4;
        unsigned nib = 0;
        if (col < K) {
            const int row0 = mb * tile_m;
            const int rows = min(tile_m, M - row0);
            const float *src = A + (size_t)row0 * K + col;
            int r = 0;
            for (; r + 8 <= rows; r += 8) {
                float4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (bounds_ok((size_t)(row0 + r + u) * K + col + 4 <= a_floats, status, 10))
                        v[u] = __ldg(reinterpret_cast<const float4 *>(src + (size_t)(r + u) * K));
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) nib |= nz4(v[u]);
            }
            for (; r < rows; ++r)
                if (bounds_ok((size_t)(row0 + r) * K + col + 4 <= a_floats, status, 10))
                    nib |= nz4(__ldg(reinterpret_cast<const float4 *>(src + (size_t)r * K)));
        }
        const unsigned other = __shfl_xor_sync(0xFFFFFFFFu, nib, 1);
        const int kb = kc * 16 + (lane >> 1);
        if (!(lane & 1) && kb < nKB && bounds_ok((size_t)mb * nKB + kb < out_bytes, status, 11))
            out[(size_t)mb * nKB + kb] = (uint8_t)(nib | (other << 4));
    }
}

// Pattern scan fused with the re-layout the packed GEMM variant reads: besides the pattern
// bytes the warp writes its 32 rows x 128 columns transposed into
//   packed[((tile * nKB + kb) * 8 + k) * 128 + row_in_tile],   tile = row / 128,
// i.e. k-major rows of 128 floats per 128-row tile, so that one K block of a tile is 4 KB of
// contiguous memory.  The transpose goes through a skewed shared-memory tile (conflict-free
// both ways).  A k whose pattern bit is clear for the warp's 32-row block is not written: the
// GEMM never multiplies it, so whatever the buffer holds there is harmless.
constexpr int PACK_WARPS = 4;
constexpr int PACK_SMEM_PER_WARP = 128 * 32 * 4;  // 16 KB

__global__ void __launch_bounds__(PACK_WARPS * 32)
esmm_preprocess_a_pack_kernel(const float *__restrict__ A, int M, int K, int nMB, int nKB, int k_chunks,
                              uint8_t *__restrict__ out, float *__restrict__ packed, int *status)
{
    // checked build, sites 10 (loads of A), 11 (pattern stores), 12 (stores into the packed copy), 13 (the warp's tile)
    const size_t a_floats = (size_t)M * K, out_bytes = (size_t)nMB * nKB;
    const size_t packed_floats = (size_t)((M + 127) / 128) * nKB * BK * 128;
    extern __shared__ __align__(16) float pack_smem[];
    float *tile = pack_smem + (threadIdx.x >> 5) * (PACK_SMEM_PER_WARP / 4);
    const int lane = threadIdx.x & 31;
    const long warps_total = (long)gridDim.x * PACK_WARPS;
    const long tasks = (long)nMB * k_chunks;
    for (long task = (long)blockIdx.x * PACK_WARPS + (threadIdx.x >> 5); task < tasks; task += warps_total) {
        const int mb = (int)(task / k_chunks);
        const int kc = (int)(task - (long)mb * k_chunks);
        const int col = kc * 128 + lane * 4;
        const bool col_ok = col < K;
        const int row0 = mb * 32;
        const float *src = A + (size_t)row0 * K + col;
        unsigned nib = 0;
        // all 32 rows of the lane's 4 columns are requested before anything is consumed: 16 KB in
        // flight per warp, which is what keeps HBM busy at the occupancy the 16 KB tile allows
        float4 v[32];
#pragma unroll
        for (int r = 0; r < 32; ++r) {
            v[r] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (col_ok && row0 + r < M && bounds_ok((size_t)(row0 + r) * K + col + 4 <= a_floats, status, 10))
                v[r] = __ldg(reinterpret_cast<const float4 *>(src + (size_t)r * K));
        }
#pragma unroll
        for (int r = 0; r < 32; ++r) nib |= nz4(v[r]);
        // live columns of the chunk: bit l of liveq[q] says column 4 l + q has a nonzero
        unsigned liveq[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) liveq[q] = __ballot_sync(0xFFFFFFFFu, (nib >> q) & 1u);
        // Only live columns go through the tile.  (This also makes every store depend on all 32
        // loads, so the loads are all in flight together.)
#pragma unroll
        for (int r = 0; r < 32; ++r) {
            // element (r, c) lives at c * 32 + ((r + (c >> 2)) & 31); here c >> 2 == lane
            const int pos = (r + lane) & 31;
            if (!bounds_ok((lane * 4 + 3) * 32 + pos < PACK_SMEM_PER_WARP / 4, status, 13)) continue;
            if (nib & 1u) tile[(lane * 4 + 0) * 32 + pos] = v[r].x;
            if (nib & 2u) tile[(lane * 4 + 1) * 32 + pos] = v[r].y;
            if (nib & 4u) tile[(lane * 4 + 2) * 32 + pos] = v[r].z;
            if (nib & 8u) tile[(lane * 4 + 3) * 32 + pos] = v[r].w;
        }
        const unsigned other = __shfl_xor_sync(0xFFFFFFFFu, nib, 1);
        const int kb_lane = kc * 16 + (lane >> 1);
        if (!(lane & 1) && kb_lane < nKB && bounds_ok((size_t)mb * nKB + kb_lane < out_bytes, status, 11))
            out[(size_t)mb * nKB + kb_lane] = (uint8_t)(nib | (other << 4));
        __syncwarp();
        const size_t dst0 = (size_t)(mb >> 2) * nKB * BK * 128 + (mb & 3) * 32 + lane;
        float *dst = packed + dst0;
#pragma unroll 8
        for (int c = 0; c < 128; ++c) {
            const int k = kc * 128 + c;  // global k = kb * 8 + kk
            if (((liveq[c & 3] >> (c >> 2)) & 1u) && k < nKB * BK &&
                bounds_ok(dst0 + (size_t)k * 128 < packed_floats, status, 12))
                dst[(size_t)k * 128] = tile[c * 32 + ((lane + (c >> 2)) & 31)];
        }
        __syncwarp();
    }
}

// The same with half the task (the default; ESMM_PACK=128 selects the kernel above): 32 rows x 64 columns per warp (8 KB in flight and 8 KB of shared
// memory per warp instead of 16, half the registers), so that more warps are resident and the tail of
// the grid is shorter.  Lane = (row parity h, column group cl): lane loads rows 2 i + h, columns
// 4 cl .. 4 cl + 3.  Element (r, c) of the tile lives at c * 32 + ((r + 2 (c >> 2)) & 31): both the
// stores (lanes differ in 2 cl + h) and the k-major loads (lanes differ in r) are conflict-free.
constexpr int PACK64_SMEM_PER_WARP = 64 * 32 * 4;  // 8 KB

__global__ void __launch_bounds__(PACK_WARPS * 32)
esmm_preprocess_a_pack64_kernel(const float *__restrict__ A, int M, int K, int nMB, int nKB, int k_chunks,
                                uint8_t *__restrict__ out, float *__restrict__ packed, int *status)
{
    // The product kernel, launched as a dependent of this one, may be placed where SMs become free once every CTA of this
    // grid has got here; it waits for this grid's end itself.  (This kernel is launched the ordinary way: launched as a
    // dependent of the product kernel before it, it made a loop of calls 0.2 % slower - its early CTAs and those of the
    // next product kernel then wait on SMs the running grid could use.)
    grid_launch_dependents();
    // checked build, sites 10 (loads of A), 11 (pattern stores), 12 (stores into the packed copy), 13 (the warp's tile)
    const size_t a_floats = (size_t)M * K, out_bytes = (size_t)nMB * nKB;
    const size_t packed_floats = (size_t)((M + 127) / 128) * nKB * BK * 128;
    extern __shared__ __align__(16) float pack_smem[];
    float *tile = pack_smem + (threadIdx.x >> 5) * (PACK64_SMEM_PER_WARP / 4);
    const int lane = threadIdx.x & 31;
    const int h = lane >> 4, cl = lane & 15;
    const long warps_total = (long)gridDim.x * PACK_WARPS;
    const long tasks = (long)nMB * k_chunks;
    for (long task = (long)blockIdx.x * PACK_WARPS + (threadIdx.x >> 5); task < tasks; task += warps_total) {
        const int mb = (int)(task / k_chunks);
        const int kc = (int)(task - (long)mb * k_chunks);
        const int col = kc * 64 + cl * 4;
        const bool col_ok = col < K;
        const int row0 = mb * 32;
        const float *src = A + (size_t)row0 * K + col;
        float4 v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int r = 2 * i + h;
            v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (col_ok && row0 + r < M && bounds_ok((size_t)(row0 + r) * K + col + 4 <= a_floats, status, 10))
                v[i] = __ldg(reinterpret_cast<const float4 *>(src + (size_t)r * K));
        }
        unsigned nib = 0;
#pragma unroll
        for (int i = 0; i < 16; ++i) nib |= nz4(v[i]);
        nib |= __shfl_xor_sync(0xFFFFFFFFu, nib, 16);           // both row parities
        // live columns of the chunk: bit cl of liveq[q] says column 4 cl + q has a nonzero
        unsigned liveq[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) liveq[q] = __ballot_sync(0xFFFFFFFFu, (nib >> q) & 1u);
        // only live columns go through the tile (and every store depends on all the loads, which keeps
        // them in flight together)
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int pos = (2 * i + h + 2 * cl) & 31;
            if (!bounds_ok((cl * 4 + 3) * 32 + pos < PACK64_SMEM_PER_WARP / 4, status, 13)) continue;
            if (nib & 1u) tile[(cl * 4 + 0) * 32 + pos] = v[i].x;
            if (nib & 2u) tile[(cl * 4 + 1) * 32 + pos] = v[i].y;
            if (nib & 4u) tile[(cl * 4 + 2) * 32 + pos] = v[i].z;
            if (nib & 8u) tile[(cl * 4 + 3) * 32 + pos] = v[i].w;
        }
        const unsigned other = __shfl_xor_sync(0xFFFFFFFFu, nib, 1);
        const int kb_lane = kc * 8 + (cl >> 1);
        if (h == 0 && !(cl & 1) && kb_lane < nKB && bounds_ok((size_t)mb * nKB + kb_lane < out_bytes, status, 11))
            out[(size_t)mb * nKB + kb_lane] = (uint8_t)(nib | (other << 4));
        __syncwarp();
        const size_t dst0 = (size_t)(mb >> 2) * nKB * BK * 128 + (mb & 3) * 32 + lane;
        float *dst = packed + dst0;
#pragma unroll 8
        for (int c = 0; c < 64; ++c) {
            const int k = kc * 64 + c;  // global k = kb * 8 + kk
            if (((liveq[c & 3] >> (c >> 2)) & 1u) && k < nKB * BK &&
                bounds_ok(dst0 + (size_t)k * 128 < packed_floats, status, 12))
                dst[(size_t)k * 128] = tile[c * 32 + ((lane + 2 * (c >> 2)) & 31)];
        }
        __syncwarp();
    }
}

// Any K, any alignment: one thread per pattern byte.  Only used when the fast kernel's
// alignment conditions do not hold.
__global__ void esmm_preprocess_a_patterns_generic_kernel(const float *__restrict__ A, int M, int K,
                                                          int tile_m, int nMB, int nKB,
                                                          uint8_t *__restrict__ out, int *status)
{
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)nMB * nKB) return;
    const int mb = (int)(idx / nKB), kb = (int)(idx % nKB);
    unsigned pat = 0;
    for (int r = mb * tile_m; r < min(M, (mb + 1) * tile_m); ++r)
        for (int k = 0; k < BK; ++k) {
            const int c = kb * BK + k;
            if (c < K && bounds_ok((size_t)r * K + c < (size_t)M * K, status, 10)) pat |= nz(A[(size_t)r * K + c]) << k;
        }
    out[idx] = (uint8_t)pat;
}

// One warp owns 128 columns (4 pattern column blocks) x 32 k rows (4 K blocks).  Per k row
// every lane tests its 4 columns; a ballot gives 8 bits per column block, nonzero means the
// row is live for that block.  Lanes 0..3 each collect one column block and store the 4
// bytes of the 4 K blocks.  Needs N % 4 == 0 and a 16-byte aligned B.
__global__ void __launch_bounds__(PRE_THREADS)
esmm_preprocess_b_patterns_kernel(const float *__restrict__ B, int K, int N, int nNB, int nKB,
                                  int n_strips, int k_groups, uint8_t *__restrict__ out, int *status)
{
    // checked build, sites 14 (loads of B) and 15 (pattern stores)
    const size_t b_floats = (size_t)K * N, out_bytes = (size_t)nNB * nKB;
    const int lane = threadIdx.x & 31;
    const long warps_total = (long)gridDim.x * (PRE_THREADS / 32);
    const long tasks = (long)n_strips * k_groups;
    for (long task = (long)blockIdx.x * (PRE_THREADS / 32) + (threadIdx.x >> 5); task < tasks;
         task += warps_total) {
        const int kg = (int)(task / n_strips);
        const int strip = (int)(task - (long)kg * n_strips);
        const int col = strip * 128 + lane * 4;
        const bool col_ok = col < N;
        const float *src = B + col;
        unsigned word = 0;  // lane j < 4: byte g = pattern of (column block strip*4+j, K block kg*4+g)
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const int k0 = (kg * 4 + g) * BK;
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (col_ok && k0 + u < K && bounds_ok((size_t)(k0 + u) * N + col + 4 <= b_floats, status, 14))
                    v[u] = __ldg(reinterpret_cast<const float4 *>(src + (size_t)(k0 + u) * N));
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const unsigned bal = __ballot_sync(0xFFFFFFFFu, nz4(v[u]) != 0u);
                const unsigned mine = (bal >> (8 * (lane & 3))) & 0xFFu;
                word |= (mine ? 1u : 0u) << (8 * g + u);
            }
        }
        if (lane < 4) {
            const int nb = strip * 4 + lane;
            if (nb < nNB) {
                uint8_t *dst = out + (size_t)nb * nKB + kg * 4;
                if (kg * 4 + 4 <= nKB && (nKB & 3) == 0) {
                    if (bounds_ok((size_t)nb * nKB + kg * 4 + 4 <= out_bytes, status, 15)) *reinterpret_cast<uint32_t *>(dst) = word;
                } else {
                    for (int g = 0; g < 4; ++g)
                        if (kg * 4 + g < nKB && bounds_ok((size_t)nb * nKB + kg * 4 + g < out_bytes, status, 15))
                            dst[g] = (uint8_t)(word >> (8 * g));
                }
            }
        }
    }
}

__global__ void esmm_preprocess_b_patterns_generic_kernel(const float *__restrict__ B, int K, int N,
                                                          int nNB, int nKB, uint8_t *__restrict__ out, int *status)
{
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)nNB * nKB) return;
    const int nb = (int)(idx / nKB), kb = (int)(idx % nKB);
    unsigned pat = 0;
    for (int k = 0; k < BK; ++k) {
        const int r = kb * BK + k;
        if (r >= K) break;
        for (int c = nb * PAT_N; c < min(N, (nb + 1) * PAT_N); ++c)
            if (bounds_ok((size_t)r * N + c < (size_t)K * N, status, 14)) pat |= nz(B[(size_t)r * N + c]) << k;
    }
    out[idx] = (uint8_t)pat;
}

static int sm_count()
{
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return sms;
}

int preprocess_a_launch(const float *d_A, int M, int K, int tile_m, uint8_t *d_out, cudaStream_t stream)
{
    if (!d_A || !d_out) return ESMM_ERR_NULL;
    if (M <= 0 || K <= 0 || tile_m <= 0) return ESMM_ERR_SHAPE;
    const int nMB = ceil_div(M, tile_m), nKB = ceil_div(K, BK);
    int *status = kCheckedBuild ? device_status_ptr() : nullptr;   // only the checked build's kernels write it
    if ((K & 3) == 0 && ((uintptr_t)d_A & 15) == 0) {
        const int k_chunks = ceil_div(K, 128);
        const long tasks = (long)nMB * k_chunks;
        const int sms = sm_count();
        if (sms <= 0) return record_cuda_error_text("no CUDA device");
        long blocks = (tasks + PRE_THREADS / 32 - 1) / (PRE_THREADS / 32);
        const long cap = (long)sms * 16 * 4;
        if (blocks > cap) blocks = cap;
        esmm_preprocess_a_patterns_kernel<<<(unsigned)blocks, PRE_THREADS, 0, stream>>>(
            d_A, M, K, tile_m, nMB, nKB, k_chunks, d_out, status);
    } else {
        const long total = (long)nMB * nKB;
        esmm_preprocess_a_patterns_generic_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
            d_A, M, K, tile_m, nMB, nKB, d_out, status);
    }
    ESMM_CUDA_TRY(cudaGetLastError());
    return ESMM_OK;
}

int preprocess_a_pack_launch(const float *d_A, int M, int K, uint8_t *d_out, float *d_packed,
                             cudaStream_t stream)
{
    if (!d_A || !d_out || !d_packed) return ESMM_ERR_NULL;
    if (M <= 0 || K <= 0 || (K & 3)) return ESMM_ERR_SHAPE;
    if (((uintptr_t)d_A | (uintptr_t)d_packed) & 15) return ESMM_ERR_ALIGN;
    const int nMB = ceil_div(M, 32), nKB = ceil_div(K, BK);
    const int sms = sm_count();
    if (sms <= 0) return record_cuda_error_text("no CUDA device");
    int *status = kCheckedBuild ? device_status_ptr() : nullptr;
    if (tuning_get("PACK", 64) == 64) {
        const int k_chunks = ceil_div(K, 64);
        const long tasks = (long)nMB * k_chunks;
        static bool attr64_set[64] = {false};
        int dev = 0;
        ESMM_CUDA_TRY(cudaGetDevice(&dev));
        const int smem = PACK_WARPS * PACK64_SMEM_PER_WARP;
        if (dev >= 0 && dev < 64 && !attr64_set[dev]) {
            ESMM_CUDA_TRY(cudaFuncSetAttribute(esmm_preprocess_a_pack64_kernel,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            attr64_set[dev] = true;
        }
        long blocks = (tasks + PACK_WARPS - 1) / PACK_WARPS;
        const long cap = (long)sms * 6 * 8;
        if (blocks > cap) blocks = cap;
        esmm_preprocess_a_pack64_kernel<<<(unsigned)blocks, PACK_WARPS * 32, smem, stream>>>(
            d_A, M, K, nMB, nKB, k_chunks, d_out, d_packed, status);
        ESMM_CUDA_TRY(cudaGetLastError());
        return ESMM_OK;
    }
    const int k_chunks = ceil_div(K, 128);
    const long tasks = (long)nMB * k_chunks;
    static bool attr_set[64] = {false};
    int dev = 0;
    ESMM_CUDA_TRY(cudaGetDevice(&dev));
    const int smem = PACK_WARPS * PACK_SMEM_PER_WARP;
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        ESMM_CUDA_TRY(cudaFuncSetAttribute(esmm_preprocess_a_pack_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_set[dev] = true;
    }
    long blocks = (tasks + PACK_WARPS - 1) / PACK_WARPS;
    const long cap = (long)sms * 3 * 8;
    if (blocks > cap) blocks = cap;
    esmm_preprocess_a_pack_kernel<<<(unsigned)blocks, PACK_WARPS * 32, smem, stream>>>(
        d_A, M, K, nMB, nKB, k_chunks, d_out, d_packed, status);
    ESMM_CUDA_TRY(cudaGetLastError());
    return ESMM_OK;
}

int preprocess_b_launch(const float *d_B, int K, int N, uint8_t *d_out, cudaStream_t stream)
{
    if (!d_B || !d_out) return ESMM_ERR_NULL;
    if (K <= 0 || N <= 0) return ESMM_ERR_SHAPE;
    const int nNB = ceil_div(N, PAT_N), nKB = ceil_div(K, BK);
    int *status = kCheckedBuild ? device_status_ptr() : nullptr;
    if ((N & 3) == 0 && ((uintptr_t)d_B & 15) == 0 && ((uintptr_t)d_out & 3) == 0) {
        const int n_strips = ceil_div(N, 128), k_groups = ceil_div(nKB, 4);
        const long tasks = (long)n_strips * k_groups;
        const int sms = sm_count();
        if (sms <= 0) return record_cuda_error_text("no CUDA device");
        long blocks = (tasks + PRE_THREADS / 32 - 1) / (PRE_THREADS / 32);
        const long cap = (long)sms * 16 * 4;
        if (blocks > cap) blocks = cap;
        esmm_preprocess_b_patterns_kernel<<<(unsigned)blocks, PRE_THREADS, 0, stream>>>(
            d_B, K, N, nNB, nKB, n_strips, k_groups, d_out, status);
    } else {
        const long total = (long)nNB * nKB;
        esmm_preprocess_b_patterns_generic_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
            d_B, K, N, nNB, nKB, d_out, status);
    }
    ESMM_CUDA_TRY(cudaGetLastError());
    return ESMM_OK;
}

}  // namespace esmm

extern "C" {

int esmm_num_k_blocks(int K) { return K > 0 ? esmm::ceil_div(K, esmm::BK) : 0; }

size_t esmm_a_pattern_bytes(int M, int K, int tile_m)
{
    if (M <= 0 || K <= 0 || tile_m <= 0) return 0;
    return (size_t)esmm::ceil_div(M, tile_m) * esmm::ceil_div(K, esmm::BK);
}

size_t esmm_b_pattern_bytes(int K, int N)
{
    if (N <= 0 || K <= 0) return 0;
    return (size_t)esmm::ceil_div(N, esmm::PAT_N) * esmm::ceil_div(K, esmm::BK);
}

int esmm_preprocess_a(const float *d_A, int M, int K, int tile_m, uint8_t *d_out, void *stream)
{
    return esmm::preprocess_a_launch(d_A, M, K, tile_m, d_out, (cudaStream_t)stream);
}

size_t esmm_a_packed_bytes(int M, int K)
{
    if (M <= 0 || K <= 0) return 0;
    return (size_t)esmm::ceil_div(M, 128) * 128 * (size_t)esmm::ceil_div(K, esmm::BK) * esmm::BK * sizeof(float);
}

int esmm_preprocess_a_packed(const float *d_A, int M, int K, uint8_t *d_out, float *d_packed, void *stream)
{
    return esmm::preprocess_a_pack_launch(d_A, M, K, d_out, d_packed, (cudaStream_t)stream);
}

int esmm_preprocess_b(const float *d_B, int K, int N, uint8_t *d_out, void *stream)
{
    return esmm::preprocess_b_launch(d_B, K, N, d_out, (cudaStream_t)stream);
}

int esmm_preprocess_ab(const float *d_A, const float *d_B, int M, int N, int K, int tile_m,
                       const uint8_t *d_b_cached, esmm_ab_pattern_metadata *meta)
{
    if (!meta) return ESMM_ERR_NULL;
    memset(meta, 0, sizeof *meta);
    if (!d_A || (!d_B && !d_b_cached)) return ESMM_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || tile_m <= 0) return ESMM_ERR_SHAPE;
    meta->numMBlocks = esmm::ceil_div(M, tile_m);
    meta->numNBlocks = esmm::ceil_div(N, esmm::PAT_N);
    meta->numKBlocks = esmm::ceil_div(K, esmm::BK);
    ESMM_CUDA_TRY(cudaMalloc(&meta->d_a_patterns, (size_t)meta->numMBlocks * meta->numKBlocks));
    if (d_b_cached) {
        meta->d_b_patterns = const_cast<uint8_t *>(d_b_cached);
        meta->owns_b_patterns = 0;
    } else {
        cudaError_t e = cudaMalloc(&meta->d_b_patterns, (size_t)meta->numNBlocks * meta->numKBlocks);
        if (e != cudaSuccess) {
            cudaFree(meta->d_a_patterns);
            meta->d_a_patterns = nullptr;
            return esmm::record_cuda_error(e, "cudaMalloc(b patterns)");
        }
        meta->owns_b_patterns = 1;
    }
    int st = esmm::preprocess_a_launch(d_A, M, K, tile_m, meta->d_a_patterns, 0);
    if (st == ESMM_OK && meta->owns_b_patterns) st = esmm::preprocess_b_launch(d_B, K, N, meta->d_b_patterns, 0);
    if (st != ESMM_OK) esmm_free_ab_pattern_metadata(meta);
    return st;
}

int esmm_free_ab_pattern_metadata(esmm_ab_pattern_metadata *meta)
{
    if (!meta) return ESMM_ERR_NULL;
    if (meta->d_a_patterns) cudaFree(meta->d_a_patterns);
    if (meta->owns_b_patterns && meta->d_b_patterns) cudaFree(meta->d_b_patterns);
    meta->d_a_patterns = nullptr;
    meta->d_b_patterns = nullptr;
    return ESMM_OK;
}

}  // extern "C"
