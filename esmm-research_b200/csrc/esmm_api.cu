// C ABI plumbing of libesmm_b200: status / error text, the fused per-call path, the
// host-buffer plan, baselines (cuBLAS, FFMA peak), generators, skip statistics, the B
// pattern cache file and the kernel-id runners.
#include <cublas_v2.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "esmm_common.cuh"

namespace esmm {

int gemm_ab_launch(int M, int N, int K, const float *d_A, const float *d_B, float *d_C,
                   const uint8_t *d_a_pat, const uint8_t *d_b_pat, int a_tile_m, cudaStream_t stream);
int gemm_ab_packed_launch(int M, int N, int K, const float *d_a_packed, const float *d_B, float *d_C,
                          const uint8_t *d_a_pat, const uint8_t *d_b_pat, cudaStream_t stream);
int gemm_ab_packed_prepare();
int preprocess_a_launch(const float *d_A, int M, int K, int tile_m, uint8_t *d_out, cudaStream_t stream);
int preprocess_a_pack_launch(const float *d_A, int M, int K, uint8_t *d_out, float *d_packed,
                             cudaStream_t stream);
int preprocess_b_launch(const float *d_B, int K, int N, uint8_t *d_out, cudaStream_t stream);

// ---------------------------------------------------------------------------
// error text + device status word
// ---------------------------------------------------------------------------
static thread_local char g_cuda_error[256] = "";

int record_cuda_error_text(const char *text)
{
    snprintf(g_cuda_error, sizeof g_cuda_error, "%s", text);
    return ESMM_ERR_CUDA;
}

int record_cuda_error(cudaError_t e, const char *what)
{
    snprintf(g_cuda_error, sizeof g_cuda_error, "%s: %s", what, cudaGetErrorString(e));
    cudaGetLastError();  // clear the sticky-free error state
    return ESMM_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// tuning / test hooks: a fixed table of named integers, unset by default
// ---------------------------------------------------------------------------
static const char *const kTuningNames[] = {"TILE_M", "STAGES", "BROW_BITS", "ROW_DENSITY", "FORCE_LISTED", "NO_RUN_TILES",
                                           "VEC_PATTERNS", "NO_SKINNY", "SKINNY_ROWS", "PRODUCER_WARPS", "NO_DEPENDENT_LAUNCH", "GROUP_M", "GRID", "PACK", "SWIZZLE", "TF32_PAIR",
                                           "TF32_SPLIT_LAST", "TF32_DIRECT_STORES"};
constexpr int kTuningCount = (int)(sizeof kTuningNames / sizeof kTuningNames[0]);
static std::atomic<int> g_tuning_value[kTuningCount];
static std::atomic<bool> g_tuning_set[kTuningCount];

static int tuning_index(const char *name)
{
    if (!name) return -1;
    for (int i = 0; i < kTuningCount; ++i)
        if (strcmp(name, kTuningNames[i]) == 0) return i;
    return -1;
}

int tuning_get(const char *name, int dflt)
{
    const int i = tuning_index(name);
    return (i >= 0 && g_tuning_set[i].load(std::memory_order_acquire)) ? g_tuning_value[i].load() : dflt;
}

__device__ int g_esmm_device_status;

int *device_status_ptr()
{
    // One address per device; looked up with that device current.
    static int *ptrs[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        record_cuda_error_text("cudaGetDevice failed");
        return nullptr;
    }
    if (!ptrs[dev]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_esmm_device_status);
        if (e != cudaSuccess) {
            record_cuda_error(e, "cudaGetSymbolAddress(status)");
            return nullptr;
        }
        e = cudaMemset(p, 0, sizeof(int));
        if (e != cudaSuccess) {
            record_cuda_error(e, "cudaMemset(status)");
            return nullptr;
        }
        ptrs[dev] = static_cast<int *>(p);
    }
    return ptrs[dev];
}

// ---------------------------------------------------------------------------
// small kernels: generator, shard interleave, FFMA peak
// ---------------------------------------------------------------------------
__host__ __device__ inline uint64_t mix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__global__ void esmm_fill_normal_kernel(float *out, long rows, long cols, int k_axis, uint64_t seed,
                                        float mean, float std, int relu, int mode, unsigned pattern,
                                        float p_live, int gran, uint64_t seed2)
{
    const long total = rows * cols;
    const uint32_t thresh = p_live >= 1.0f ? 0xFFFFFFFFu : (uint32_t)(p_live * 4294967296.0f);
    for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long)gridDim.x * blockDim.x) {
        const long r = idx / cols, c = idx - r * cols;
        const long k = k_axis == 0 ? c : r;
        const long outer = k_axis == 0 ? r : c;
        bool live = true;
        if (mode == 1) {
            live = (pattern >> (k & 7)) & 1u;
        } else if (mode == 2) {
            const uint64_t tile = (uint64_t)(outer / gran) * 0x100000000ull + (uint64_t)(k >> 3);
            const uint64_t h = mix64(mix64(seed2 ^ tile) + (uint64_t)(k & 7));
            live = p_live >= 1.0f || (uint32_t)(h >> 32) < thresh;
        }
        float v = 0.0f;
        if (live) {
            const uint64_t h = mix64(seed * 0xD1342543DE82EF95ull + (uint64_t)idx);
            const float u1 = ((float)(uint32_t)(h >> 40) + 1.0f) * (1.0f / 16777216.0f);  // (0, 1]
            const float u2 = (float)(uint32_t)(h & 0xFFFFFFu) * (1.0f / 16777216.0f);      // [0, 1)
            v = mean + std * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
            if (relu) v = fmaxf(v, 0.0f);
        }
        out[idx] = v;
    }
}

__global__ void esmm_interleave_shards_kernel(const float4 *__restrict__ shards, float4 *__restrict__ C,
                                              long M, long n4, int G)
{
    // shards: [G][M][n4] float4; C: [M][G * n4] float4
    const long total = M * n4 * G;
    for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long)gridDim.x * blockDim.x) {
        const long row = idx / (n4 * G);
        const long rem = idx - row * n4 * G;
        const long g = rem / n4, c = rem - g * n4;
        C[idx] = shards[(g * M + row) * n4 + c];
    }
}

__global__ void esmm_ffma_peak_kernel(float *out, int iters, float a, float b)
{
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = (float)(threadIdx.x + i);
#pragma unroll 1
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int rep = 0; rep < 8; ++rep)
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = fmaf(x[i], a, b);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) s += x[i];
    if (s == 123.456f) out[0] = s;  // keeps the chain alive; practically never true
}

// One CTA waits, with the library's bounded wait and a caller-chosen budget, on an mbarrier that
// nothing ever arrives on; the wait runs out, the kernel records ESMM_ERR_TIMEOUT in the status
// word and returns normally.  Exercises the failure path of the GEMM kernels without a fault.
__global__ void esmm_selftest_bounded_wait_kernel(int *status, unsigned long long budget_ns)
{
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    const bool ok = mbar_wait_budget(smem_u32(&bar), 0, &abort_flag, budget_ns);
    if (!ok && (threadIdx.x & 31) == 0) atomicExch(status, (int)ESMM_ERR_TIMEOUT);
}

// Reports a failed bounds check (site 99) without making any access: exercises the checked build's
// reporting path; in the product build bounds_ok() is the constant true and nothing is recorded.
__global__ void esmm_selftest_bounds_kernel(int *status) { (void)bounds_ok(false, status, 99); }

static cublasHandle_t cublas_handle_for_device()
{
    static cublasHandle_t handles[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!handles[dev] && cublasCreate(&handles[dev]) != CUBLAS_STATUS_SUCCESS) handles[dev] = nullptr;
    return handles[dev];
}

static void skip_stats_host(const uint8_t *a, const uint8_t *b, int cbm, int cbn, int nKB, int wm, int wn,
                            int bk, long long out[6])
{
    const int nw = wm * wn;
    long long block_skips = 0, warp_skips = 0, dot_skips = 0;
    std::vector<uint8_t> aor((size_t)nKB), bor((size_t)nKB);
    for (int cr = 0; cr < cbm; ++cr)
        for (int cc = 0; cc < cbn; ++cc)
            for (int k = 0; k < nKB; ++k) {
                uint8_t ao = 0, bo = 0;
                for (int w = 0; w < wm; ++w) ao |= a[(size_t)(cr * wm + w) * nKB + k];
                for (int w = 0; w < wn; ++w) bo |= b[(size_t)(cc * wn + w) * nKB + k];
                if (!(ao & bo)) {  // OR over warps of (a & b) == (OR a) & (OR b)
                    ++block_skips;
                    warp_skips += nw;
                    dot_skips += (long long)nw * bk;
                    continue;
                }
                for (int r = 0; r < wm; ++r)
                    for (int c = 0; c < wn; ++c) {
                        const uint8_t j = a[(size_t)(cr * wm + r) * nKB + k] & b[(size_t)(cc * wn + c) * nKB + k];
                        if (!j) {
                            ++warp_skips;
                            dot_skips += bk;
                        } else {
                            dot_skips += bk - __builtin_popcount(j);
                        }
                    }
            }
    const long long total_k = (long long)cbm * cbn * nKB;
    out[0] = block_skips;
    out[1] = total_k;
    out[2] = warp_skips;
    out[3] = total_k * nw;
    out[4] = dot_skips;
    out[5] = total_k * nw * bk;
}

// Prints the block the reference prints (include/runners.cuh:692-705).
static void print_skip_stats(const long long s[6], int cbm, int cbn, int nKB, int nw, int bk, const char *label)
{
    const long long warp_beyond_block = s[2] - s[0] * nw;
    const long long block_k_hit = s[1] - s[0];
    printf("\n=== Skip Stats: %s ===\n", label);
    printf("Grid: %d x %d CUDA blocks, %d K-tiles, %d warps/block, BK=%d\n", cbm, cbn, nKB, nw, bk);
    printf("Block-level  (all warps skip K-tile):  %lld / %lld  (%.1f%%)\n", s[0], s[1], 100.0 * s[0] / s[1]);
    printf("Warp-level   (one warp  skips K-tile):  %lld / %lld  (%.1f%%)  "
           "[%lld beyond block skips, %.1f%% of non-block-skipped warp-K pairs]\n",
           s[2], s[3], 100.0 * s[2] / s[3], warp_beyond_block,
           block_k_hit > 0 ? 100.0 * warp_beyond_block / (block_k_hit * nw) : 0.0);
    printf("dotIdx-level (one col   skipped):        %lld / %lld  (%.1f%%)  [%lld executed, %.1f%%]\n\n",
           s[4], s[5], 100.0 * s[4] / s[5], s[5] - s[4], 100.0 * (s[5] - s[4]) / s[5]);
}

// A granularity each joint-sparse kernel id preprocesses A at (include/runners.cuh: 20 and 25
// use preprocess_ab<8,64,32>, 21 uses <8,8,32>, 26-30 use <8,32,32>); 0 = not a joint id.
static int a_tile_for_kernel(int id)
{
    switch (id) {
    case 20: case 25: return 64;
    case 21: return 8;
    case 26: case 27: case 28: case 29: case 30: return 32;
    case 129: return 32;                                   // the optional tensor-core variant of id 29
    default: return 0;
    }
}

static const int kValidIds[] = {14, 15, 16, 17, 20, 21, 25, 26, 27, 28, 29, 30};

}  // namespace esmm

// ===========================================================================
extern "C" {

const char *esmm_strerror(int status)
{
    switch (status) {
    case ESMM_OK: return "ok";
    case ESMM_ERR_NULL: return "required pointer is NULL";
    case ESMM_ERR_SHAPE: return "bad shape: dimensions must be positive, K and N multiples of 4";
    case ESMM_ERR_ALIGN: return "matrix pointer is not 16-byte aligned";
    case ESMM_ERR_CUDA: return "CUDA call failed";
    case ESMM_ERR_TIMEOUT: return "device-side wait gave up; results are invalid";
    case ESMM_ERR_IO: return "file I/O failed";
    case ESMM_ERR_UNSUPPORTED: return "kernel id or granularity not provided by this library";
    case ESMM_ERR_VERIFY: return "verification failed";
    case ESMM_ERR_TOO_LARGE: return "K too large for the kernel's shared-memory masks";
    case ESMM_ERR_MISMATCH: return "cached patterns do not match the requested shape";
    case ESMM_ERR_BOUNDS: return "checked build: a kernel computed an index outside its buffer (access skipped)";
    default: return "unknown status";
    }
}

const char *esmm_last_cuda_error(void) { return esmm::g_cuda_error; }
int esmm_version(void) { return 110; }

int esmm_tuning_set(const char *name, int value)
{
    const int i = esmm::tuning_index(name);
    if (i < 0) return ESMM_ERR_UNSUPPORTED;
    esmm::g_tuning_value[i].store(value);
    esmm::g_tuning_set[i].store(true, std::memory_order_release);
    return ESMM_OK;
}

void esmm_tuning_reset(void)
{
    for (int i = 0; i < esmm::kTuningCount; ++i) esmm::g_tuning_set[i].store(false, std::memory_order_release);
}

int esmm_pattern_from_string(const char *s)
{
    if (!s || strlen(s) != 8) return -1;
    int p = 0;
    for (int i = 0; i < 8; ++i) {
        if (s[i] == '1') p |= 1 << i;
        else if (s[i] != '0') return -1;
    }
    return p;
}

void esmm_pattern_lut(uint8_t pattern, uint8_t *count, uint8_t offsets[8])
{
    uint8_t c = 0;
    for (int i = 0; i < 8; ++i) offsets[i] = 0;
    for (unsigned m = pattern; m; m &= m - 1) offsets[c++] = (uint8_t)__builtin_ctz(m);
    if (count) *count = c;
}

static size_t pattern_region_bytes(int M, int K)
{
    return (esmm_a_pattern_bytes(M, K, 32) + 255) & ~(size_t)255;
}

size_t esmm_sgemm_joint_workspace_bytes(int M, int K)
{
    if (M <= 0 || K <= 0) return 0;
    return pattern_region_bytes(M, K) + esmm_a_packed_bytes(M, K);
}

int esmm_sgemm_joint(int M, int N, int K, const float *d_A, const float *d_B, float *d_C,
                     const uint8_t *d_b_pat, void *d_workspace, void *stream)
{
    if (!d_workspace) return ESMM_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || (K & 3) || (N & 3)) return ESMM_ERR_SHAPE;
    if ((uintptr_t)d_workspace & 255) return ESMM_ERR_ALIGN;
    uint8_t *a_pat = static_cast<uint8_t *>(d_workspace);
    float *a_packed = reinterpret_cast<float *>(a_pat + pattern_region_bytes(M, K));
    int st = esmm::preprocess_a_pack_launch(d_A, M, K, a_pat, a_packed, (cudaStream_t)stream);
    if (st != ESMM_OK) return st;
    return esmm::gemm_ab_packed_launch(M, N, K, a_packed, d_B, d_C, a_pat, d_b_pat, (cudaStream_t)stream);
}

int esmm_device_status(void *stream)
{
    int *p = esmm::device_status_ptr();
    if (!p) return ESMM_ERR_CUDA;
    ESMM_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    int v = 0;
    ESMM_CUDA_TRY(cudaMemcpy(&v, p, sizeof v, cudaMemcpyDeviceToHost));
    if (v != 0) ESMM_CUDA_TRY(cudaMemset(p, 0, sizeof v));
    if ((v & 0xFF) == ESMM_ERR_BOUNDS) {
        char buf[96];
        snprintf(buf, sizeof buf, "bounds check failed at site %d (see the site numbers beside bounds_ok() in csrc/)", v >> 8);
        esmm::record_cuda_error_text(buf);
    }
    return v & 0xFF;
}

int esmm_checked_build(void) { return esmm::kCheckedBuild ? 1 : 0; }

int esmm_selftest_bounds_report(void *stream)
{
    int *status = esmm::device_status_ptr();
    if (!status) return ESMM_ERR_CUDA;
    esmm::esmm_selftest_bounds_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(status);
    ESMM_CUDA_TRY(cudaGetLastError());
    return ESMM_OK;
}

int esmm_selftest_bounded_wait(unsigned budget_us, void *stream)
{
    if (budget_us == 0 || budget_us > 1000000u) return ESMM_ERR_SHAPE;  // at most one second
    int *status = esmm::device_status_ptr();
    if (!status) return ESMM_ERR_CUDA;
    esmm::esmm_selftest_bounded_wait_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(status, (unsigned long long)budget_us * 1000ull);
    ESMM_CUDA_TRY(cudaGetLastError());
    return ESMM_OK;
}

// ---- host-buffer plan -------------------------------------------------------
struct esmm_plan {
    int M, N, K, chunks;
    float *d_A, *d_B, *d_C, *d_a_packed;
    uint8_t *d_a_pat, *d_b_pat;
    cudaStream_t streams[4];   // copies in, kernels of even chunks, kernels of odd chunks, copies out
    cudaEvent_t up[64], done[64], down[64];
};

int esmm_plan_destroy(esmm_plan *pl)
{
    if (!pl) return ESMM_ERR_NULL;
    cudaFree(pl->d_A);
    cudaFree(pl->d_B);
    cudaFree(pl->d_C);
    cudaFree(pl->d_a_pat);
    cudaFree(pl->d_a_packed);
    cudaFree(pl->d_b_pat);
    for (int i = 0; i < 4; ++i)
        if (pl->streams[i]) cudaStreamDestroy(pl->streams[i]);
    for (int i = 0; i < pl->chunks; ++i) {
        if (pl->up[i]) cudaEventDestroy(pl->up[i]);
        if (pl->done[i]) cudaEventDestroy(pl->done[i]);
        if (pl->down[i]) cudaEventDestroy(pl->down[i]);
    }
    delete pl;
    return ESMM_OK;
}

int esmm_plan_create(int M, int N, int K, const float *h_B, int chunks, esmm_plan **out)
{
    if (!h_B || !out) return ESMM_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || (K & 3) || (N & 3)) return ESMM_ERR_SHAPE;
    if (chunks < 1) chunks = 1;
    if (chunks > 64) chunks = 64;
    // chunks are whole 128-row tiles
    const int tiles = esmm::ceil_div(M, 128);
    if (chunks > tiles) chunks = tiles;
    esmm_plan *pl = new esmm_plan();
    memset(pl, 0, sizeof *pl);
    pl->M = M;
    pl->N = N;
    pl->K = K;
    pl->chunks = chunks;
    *out = nullptr;
#define PLAN_TRY(expr)                                        \
    do {                                                      \
        cudaError_t _e = (expr);                              \
        if (_e != cudaSuccess) {                              \
            int _st = esmm::record_cuda_error(_e, #expr);     \
            esmm_plan_destroy(pl);                            \
            return _st;                                       \
        }                                                     \
    } while (0)
    PLAN_TRY(cudaMalloc(&pl->d_A, (size_t)M * K * 4));
    PLAN_TRY(cudaMalloc(&pl->d_B, (size_t)K * N * 4));
    PLAN_TRY(cudaMalloc(&pl->d_C, (size_t)M * N * 4));
    PLAN_TRY(cudaMalloc(&pl->d_a_pat, esmm_a_pattern_bytes(M, K, 32)));
    PLAN_TRY(cudaMalloc(&pl->d_a_packed, esmm_a_packed_bytes(M, K)));
    PLAN_TRY(cudaMalloc(&pl->d_b_pat, esmm_b_pattern_bytes(K, N)));
    for (int i = 0; i < 4; ++i) PLAN_TRY(cudaStreamCreateWithFlags(&pl->streams[i], cudaStreamNonBlocking));
    for (int i = 0; i < chunks; ++i) {
        PLAN_TRY(cudaEventCreateWithFlags(&pl->up[i], cudaEventDisableTiming));
        PLAN_TRY(cudaEventCreateWithFlags(&pl->done[i], cudaEventDisableTiming));
        PLAN_TRY(cudaEventCreateWithFlags(&pl->down[i], cudaEventDisableTiming));
    }
    PLAN_TRY(cudaMemcpy(pl->d_B, h_B, (size_t)K * N * 4, cudaMemcpyHostToDevice));
#undef PLAN_TRY
    int st = esmm::preprocess_b_launch(pl->d_B, K, N, pl->d_b_pat, 0);
    if (st == ESMM_OK && cudaDeviceSynchronize() != cudaSuccess) st = ESMM_ERR_CUDA;
    if (st != ESMM_OK) {
        esmm_plan_destroy(pl);
        return st;
    }
    *out = pl;
    return ESMM_OK;
}

int esmm_plan_run(esmm_plan *pl, const float *h_A, float *h_C)
{
    const int st = esmm_plan_submit(pl, h_A, h_C);
    return st != ESMM_OK ? st : esmm_plan_wait(pl);
}

int esmm_plan_wait(esmm_plan *pl)
{
    if (!pl) return ESMM_ERR_NULL;
    ESMM_CUDA_TRY(cudaStreamSynchronize(pl->streams[3]));   // every copy out follows its chunk's kernels
    return esmm_device_status(pl->streams[3]);
}

int esmm_plan_submit(esmm_plan *pl, const float *h_A, float *h_C)
{
    if (!pl || !h_A || !h_C) return ESMM_ERR_NULL;
    const int M = pl->M, N = pl->N, K = pl->K;
    const int tiles = esmm::ceil_div(M, 128);
    const int nKB = esmm::ceil_div(K, esmm::BK);
    cudaStream_t s_up = pl->streams[0], s_down = pl->streams[3];
    int tile0 = 0;
    for (int c = 0; c < pl->chunks; ++c) {
        const int tile1 = (int)((long)tiles * (c + 1) / pl->chunks);
        const int r0 = tile0 * 128, r1 = std::min(M, tile1 * 128);
        tile0 = tile1;
        if (r1 <= r0) continue;
        const size_t a_off = (size_t)r0 * K, c_off = (size_t)r0 * N;
        // Chunks alternate between two kernel streams, so that the first CTAs of a chunk's GEMM fill the
        // SMs that the last, partial wave of the chunk before leaves idle.
        cudaStream_t s_run = pl->streams[1 + (c & 1)];
        // The device buffers are reused by the next submission: its copy of A's chunk waits for this
        // one's kernels, its kernels wait for this one's copy of C's chunk (events never recorded yet
        // count as complete).
        ESMM_CUDA_TRY(cudaStreamWaitEvent(s_up, pl->done[c], 0));
        ESMM_CUDA_TRY(cudaMemcpyAsync(pl->d_A + a_off, h_A + a_off, (size_t)(r1 - r0) * K * 4,
                                      cudaMemcpyHostToDevice, s_up));
        ESMM_CUDA_TRY(cudaEventRecord(pl->up[c], s_up));
        ESMM_CUDA_TRY(cudaStreamWaitEvent(s_run, pl->up[c], 0));
        ESMM_CUDA_TRY(cudaStreamWaitEvent(s_run, pl->down[c], 0));
        uint8_t *apat = pl->d_a_pat + (size_t)(r0 / 32) * nKB;
        float *apacked = pl->d_a_packed + (size_t)r0 * nKB * esmm::BK;  // r0 is a multiple of 128
        int st = esmm::preprocess_a_pack_launch(pl->d_A + a_off, r1 - r0, K, apat, apacked, s_run);
        if (st != ESMM_OK) return st;
        st = esmm::gemm_ab_packed_launch(r1 - r0, N, K, apacked, pl->d_B, pl->d_C + c_off, apat, pl->d_b_pat,
                                         s_run);
        if (st != ESMM_OK) return st;
        ESMM_CUDA_TRY(cudaEventRecord(pl->done[c], s_run));
        ESMM_CUDA_TRY(cudaStreamWaitEvent(s_down, pl->done[c], 0));
        ESMM_CUDA_TRY(cudaMemcpyAsync(h_C + c_off, pl->d_C + c_off, (size_t)(r1 - r0) * N * 4,
                                      cudaMemcpyDeviceToHost, s_down));
        ESMM_CUDA_TRY(cudaEventRecord(pl->down[c], s_down));
    }
    return ESMM_OK;
}

// ---- baselines / helpers -----------------------------------------------------
int esmm_cublas_sgemm(int M, int N, int K, const float *d_A, const float *d_B, float *d_C, void *stream)
{
    if (!d_A || !d_B || !d_C) return ESMM_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0) return ESMM_ERR_SHAPE;
    cublasHandle_t h = esmm::cublas_handle_for_device();
    if (!h) return esmm::record_cuda_error_text("cublasCreate failed");
    if (cublasSetStream(h, (cudaStream_t)stream) != CUBLAS_STATUS_SUCCESS)
        return esmm::record_cuda_error_text("cublasSetStream failed");
    const float alpha = 1.0f, beta = 0.0f;
    cublasStatus_t s = cublasSgemm(h, CUBLAS_OP_N, CUBLAS_OP_N, N, M, K, &alpha, d_B, N, d_A, K, &beta, d_C, N);
    if (s != CUBLAS_STATUS_SUCCESS) return esmm::record_cuda_error_text("cublasSgemm failed");
    return ESMM_OK;
}

int esmm_ffma_peak_tflops(double *tflops, int *sm_count)
{
    if (!tflops) return ESMM_ERR_NULL;
    int dev = 0, sms = 0;
    ESMM_CUDA_TRY(cudaGetDevice(&dev));
    ESMM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (sm_count) *sm_count = sms;
    float *d = nullptr;
    ESMM_CUDA_TRY(cudaMalloc(&d, 4));
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    const int threads = 1024, blocks = sms * 2, iters = 4096;
    esmm::esmm_ffma_peak_kernel<<<blocks, threads>>>(d, 64, 1.0001f, 0.5f);  // warm-up
    double best = 0.0;
    for (int rep = 0; rep < 3; ++rep) {
        cudaEventRecord(e0);
        esmm::esmm_ffma_peak_kernel<<<blocks, threads>>>(d, iters, 1.0001f, 0.5f);
        cudaEventRecord(e1);
        cudaEventSynchronize(e1);
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        const double flops = 2.0 * 16 * 8 * (double)iters * threads * blocks;
        if (ms > 0.f) best = std::max(best, flops / (ms * 1e-3) / 1e12);
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(d);
    ESMM_CUDA_TRY(cudaGetLastError());
    *tflops = best;
    return ESMM_OK;
}

int esmm_fill_normal(float *d_out, long rows, long cols, int k_axis, uint64_t seed, float mean, float std,
                     int relu, int mode, uint8_t pattern, float p_live, int gran, uint64_t seed2, void *stream)
{
    if (!d_out) return ESMM_ERR_NULL;
    if (rows <= 0 || cols <= 0 || mode < 0 || mode > 2 || (mode == 2 && gran <= 0)) return ESMM_ERR_SHAPE;
    const long total = rows * cols;
    long blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    esmm::esmm_fill_normal_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
        d_out, rows, cols, k_axis, seed, mean, std, relu, mode, pattern, p_live, gran > 0 ? gran : 1, seed2);
    ESMM_CUDA_TRY(cudaGetLastError());
    return ESMM_OK;
}

int esmm_interleave_shards(const float *d_shards, float *d_C, int M, int N, int G, void *stream)
{
    if (!d_shards || !d_C) return ESMM_ERR_NULL;
    if (M <= 0 || N <= 0 || G <= 0 || N % G || (N / G) % 4) return ESMM_ERR_SHAPE;
    const long n4 = N / G / 4, total = (long)M * n4 * G;
    long blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    esmm::esmm_interleave_shards_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const float4 *>(d_shards), reinterpret_cast<float4 *>(d_C), M, n4, G);
    ESMM_CUDA_TRY(cudaGetLastError());
    return ESMM_OK;
}

int esmm_skip_stats(const uint8_t *h_a, const uint8_t *h_b, int cbm, int cbn, int nKB, int wm, int wn, int bk,
                    long long out[6])
{
    if (!h_a || !h_b || !out) return ESMM_ERR_NULL;
    if (cbm <= 0 || cbn <= 0 || nKB <= 0 || wm <= 0 || wn <= 0 || bk <= 0) return ESMM_ERR_SHAPE;
    esmm::skip_stats_host(h_a, h_b, cbm, cbn, nKB, wm, wn, bk, out);
    return ESMM_OK;
}

// ---- B pattern cache file ------------------------------------------------------
struct BpatHeader {
    char magic[8];
    int32_t K, N, nNB, nKB;
    int32_t reserved[2];
};

int esmm_bpat_save(const char *path, const uint8_t *h_b, int K, int N)
{
    if (!path || !h_b) return ESMM_ERR_NULL;
    if (K <= 0 || N <= 0) return ESMM_ERR_SHAPE;
    BpatHeader h;
    memset(&h, 0, sizeof h);
    memcpy(h.magic, "ESMMBPT1", 8);
    h.K = K;
    h.N = N;
    h.nNB = esmm::ceil_div(N, esmm::PAT_N);
    h.nKB = esmm::ceil_div(K, esmm::BK);
    FILE *f = fopen(path, "wb");
    if (!f) return ESMM_ERR_IO;
    const size_t n = (size_t)h.nNB * h.nKB;
    const bool ok = fwrite(&h, sizeof h, 1, f) == 1 && fwrite(h_b, 1, n, f) == n;
    return (fclose(f) == 0 && ok) ? ESMM_OK : ESMM_ERR_IO;
}

int esmm_bpat_load(const char *path, uint8_t *h_b, int K, int N)
{
    if (!path || !h_b) return ESMM_ERR_NULL;
    if (K <= 0 || N <= 0) return ESMM_ERR_SHAPE;
    FILE *f = fopen(path, "rb");
    if (!f) return ESMM_ERR_IO;
    BpatHeader h;
    int st = ESMM_OK;
    if (fread(&h, sizeof h, 1, f) != 1 || memcmp(h.magic, "ESMMBPT1", 8) != 0) st = ESMM_ERR_IO;
    else if (h.K != K || h.N != N || h.nNB != esmm::ceil_div(N, esmm::PAT_N) || h.nKB != esmm::ceil_div(K, esmm::BK))
        st = ESMM_ERR_MISMATCH;
    else {
        const size_t n = (size_t)h.nNB * h.nKB;
        if (fread(h_b, 1, n, f) != n) st = ESMM_ERR_IO;
        else if (fgetc(f) != EOF) st = ESMM_ERR_IO;  // trailing bytes: not a file this library wrote
    }
    fclose(f);
    return st;
}

// ---- kernel ids ------------------------------------------------------------------
int esmm_kernel_id_valid(int id)
{
    for (int v : esmm::kValidIds)
        if (v == id) return 1;
    return id == 129;   // additive: 3xTF32 tensor-core variant; outside the reference's 1-100 range, not part of "all"
}

const char *esmm_kernel_name(int id)
{
    switch (id) {
    case 14: return "ESMM A-Only Sparse (Offset List, Templated Dispatch)";
    case 15: return "cuBLAS";
    case 16: return "ESMM A-Sparse Block-wise (Warp-Granularity Patterns)";
    case 17: return "ESMM B-Sparse Warp-Granularity (32-col, Zero-Divergence)";
    case 20: return "ESMM A+B Sparse OPTIMIZED (Zero-Overhead Inner Loop)";
    case 21: return "ESMM A+B Sparse - 8x32 Granularity";
    case 25: return "ESMM A+B Simple Fused (Main Contribution)";
    case 26: return "ESMM A+B Optimized V2 (K20 + 32-row + Block Skip + Float4)";
    case 27: return "ESMM A+B Ablation (32-row only, no Block Skip, no Float4)";
    case 28: return "ESMM A+B GMem-32 (K25 with 32-row, global mem patterns)";
    case 29: return "ESMM A+B Optimized V3 (K26 + templated smem + float2 A-loads)";
    case 30: return "ESMM A+B Compressed-K (K29 + compressed K-list + set-bit dotIdx)";
    case 129: return "ESMM A+B 3xTF32 on tensor cores (tcgen05; optional variant, not in the reference)";
    default: return "Unknown Kernel";
    }
}

// Grammar of the reference parser: "all"; "a-b" (valid ids inside the range); "a,b,c" (invalid
// ids dropped).  Where the reference would throw on non-numeric text, this returns 0.
int esmm_parse_kernel_selection(const char *selection, int *ids, int cap)
{
    if (!selection) return 0;
    std::vector<int> out;
    const std::string in(selection);
    auto to_int = [](const std::string &s, int *v) {
        if (s.empty()) return false;
        char *end = nullptr;
        const long x = strtol(s.c_str(), &end, 10);
        if (end == s.c_str()) return false;
        *v = (int)x;
        return true;
    };
    if (in == "all") {
        for (int v : esmm::kValidIds) out.push_back(v);
    } else if (in.find('-') != std::string::npos) {
        const size_t d = in.find('-');
        int a, b;
        if (!to_int(in.substr(0, d), &a) || !to_int(in.substr(d + 1), &b)) return 0;
        for (int i = a; i <= b; ++i)
            if (esmm_kernel_id_valid(i)) out.push_back(i);
    } else {
        size_t pos = 0;
        while (pos <= in.size()) {
            const size_t c = in.find(',', pos);
            const std::string tok = in.substr(pos, c == std::string::npos ? std::string::npos : c - pos);
            int v;
            if (!to_int(tok, &v)) return 0;
            if (esmm_kernel_id_valid(v)) out.push_back(v);
            if (c == std::string::npos) break;
            pos = c + 1;
        }
    }
    for (size_t i = 0; i < out.size() && (int)i < cap; ++i) ids[i] = out[i];
    return (int)out.size();
}

// verifyResults (include/utils.cuh:222-254): absolute tolerance, prints like the reference.
static bool verify_results_host(const float *gpu, const float *ref, long size, float tol, long cols)
{
    long bad = 0, first = -1;
    float maxd = 0.f;
    for (long i = 0; i < size; ++i) {
        const float d = fabsf(gpu[i] - ref[i]);
        if (d > tol) {
            ++bad;
            if (first < 0) first = i;
            maxd = std::max(maxd, d);
        }
    }
    if (bad > 0) {
        printf("Verification failed: %ld mismatches out of %ld elements.\n", bad, size);
        printf("Max difference: %g\n", maxd);
        printf("First mismatch at index %ld (row=%ld, col=%ld): GPU=%g, CPU=%g\n", first, first / cols,
               first % cols, gpu[first], ref[first]);
        return false;
    }
    return true;
}

int esmm_run_kernel(int kernel_id, int rows, int cols, int inners, float *d_A, float *d_B, float *d_C,
                    float *h_C, const float *h_C_ref, int runs, int verify, int print_stats, int *passed,
                    float *avg_ms)
{
    return esmm_run_kernel_pattern(kernel_id, rows, cols, inners, d_A, d_B, d_C, h_C, h_C_ref, runs, verify,
                                   print_stats, nullptr, nullptr, passed, avg_ms);
}

int esmm_run_kernel_cached_b(int kernel_id, int rows, int cols, int inners, float *d_A, float *d_B, float *d_C,
                             float *h_C, const float *h_C_ref, int runs, int verify, int print_stats,
                             const uint8_t *d_b_pat_cached, int *passed, float *avg_ms)
{
    return esmm_run_kernel_pattern(kernel_id, rows, cols, inners, d_A, d_B, d_C, h_C, h_C_ref, runs, verify,
                                   print_stats, d_b_pat_cached, nullptr, passed, avg_ms);
}

int esmm_run_kernel_pattern(int kernel_id, int rows, int cols, int inners, float *d_A, float *d_B, float *d_C,
                            float *h_C, const float *h_C_ref, int runs, int verify, int print_stats,
                            const uint8_t *d_b_pat_cached, const char *pattern, int *passed, float *avg_ms)
{
    if (passed) *passed = 0;
    if (avg_ms) *avg_ms = 0.f;
    if (!esmm_kernel_id_valid(kernel_id)) return ESMM_ERR_UNSUPPORTED;
    if (!d_A || !d_B || !d_C || (verify && (!h_C || !h_C_ref))) return ESMM_ERR_NULL;
    if (rows <= 0 || cols <= 0 || inners <= 0 || runs <= 0) return ESMM_ERR_SHAPE;
    const bool single_operand = kernel_id == 14 || kernel_id == 16 || kernel_id == 17;
    const int a_tile = single_operand ? 32 : esmm::a_tile_for_kernel(kernel_id);
    if (kernel_id != 15 && a_tile == 0) return ESMM_ERR_UNSUPPORTED;
    // Id 14 takes its live k from the pattern string, not from the data: the first popcount(pattern)
    // k of every 8-slice (include/runners.cuh:47-66; the unrolled kernels exist for 1, 2, 4, 6, 8).
    int prefix = 0;
    if (kernel_id == 14) {
        const char *pat = pattern ? pattern : "11111111";
        if (strlen(pat) != 8) return ESMM_ERR_SHAPE;
        for (int i = 0; i < 8; ++i) prefix += pat[i] == '1';
    }

    cudaEvent_t start, stop;
    ESMM_CUDA_TRY(cudaEventCreate(&start));
    ESMM_CUDA_TRY(cudaEventCreate(&stop));
    int st = ESMM_OK;

    if (kernel_id == 15) {
        // run_cuBlas (include/runners.cuh:109-139): handle per call, runs back to back, one sync.
        cublasHandle_t handle;
        if (cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) {
            cudaEventDestroy(start);
            cudaEventDestroy(stop);
            return esmm::record_cuda_error_text("cublasCreate failed");
        }
        const float alpha = 1.0f, beta = 0.0f;
        cublasStatus_t cst = CUBLAS_STATUS_SUCCESS;
        cudaError_t ce = cudaEventRecord(start);
        for (int i = 0; i < runs && cst == CUBLAS_STATUS_SUCCESS; ++i)
            cst = cublasSgemm(handle, CUBLAS_OP_N, CUBLAS_OP_N, cols, rows, inners, &alpha, d_B, cols, d_A, inners,
                              &beta, d_C, cols);
        if (ce == cudaSuccess) ce = cudaDeviceSynchronize();
        if (ce == cudaSuccess) ce = cudaEventRecord(stop);
        if (ce == cudaSuccess) ce = cudaEventSynchronize(stop);
        cublasDestroy(handle);
        if (cst != CUBLAS_STATUS_SUCCESS) {
            char buf[64];
            snprintf(buf, sizeof buf, "cublasSgemm failed with status %d", (int)cst);
            st = esmm::record_cuda_error_text(buf);
        } else if (ce != cudaSuccess) {
            st = esmm::record_cuda_error(ce, "cuBLAS baseline loop");
        }
    } else {
        if (print_stats && !single_operand) {
            esmm_ab_pattern_metadata meta;
            st = esmm_preprocess_ab(d_A, d_B, rows, cols, inners, a_tile, d_b_pat_cached, &meta);
            if (st == ESMM_OK) {
                std::vector<uint8_t> ha((size_t)meta.numMBlocks * meta.numKBlocks),
                    hb((size_t)meta.numNBlocks * meta.numKBlocks);
                cudaMemcpy(ha.data(), meta.d_a_patterns, ha.size(), cudaMemcpyDeviceToHost);
                cudaMemcpy(hb.data(), meta.d_b_patterns, hb.size(), cudaMemcpyDeviceToHost);
                // the reference's CTA tile for these ids: BM = 64, BN = 128 (include/runners.cuh:830-838)
                const int wm = std::max(1, 64 / a_tile), wn = 4;
                const int cbm = meta.numMBlocks / wm, cbn = meta.numNBlocks / wn;
                if (cbm > 0 && cbn > 0) {
                    long long s[6];
                    esmm::skip_stats_host(ha.data(), hb.data(), cbm, cbn, meta.numKBlocks, wm, wn, 8, s);
                    char label[16];
                    snprintf(label, sizeof label, "K%d", kernel_id);
                    esmm::print_skip_stats(s, cbm, cbn, meta.numKBlocks, wm * wn, 8, label);
                }
                esmm_free_ab_pattern_metadata(&meta);
            }
        }
        // Ids with 32-row A patterns run the packed variant; its k-major copy of A lives in a
        // buffer allocated once per runner call (the pattern arrays are allocated per run, as
        // in the reference loop).
        float *d_packed = nullptr;
        if (a_tile == 32 && kernel_id != 14 && kernel_id != 129 && st == ESMM_OK) {
            cudaError_t e = cudaMalloc(&d_packed, esmm_a_packed_bytes(rows, inners));
            if (e != cudaSuccess) st = esmm::record_cuda_error(e, "cudaMalloc(packed A)");
        }
        const size_t a_bytes = esmm_a_pattern_bytes(rows, inners, 32), b_bytes = esmm_b_pattern_bytes(inners, cols);
        uint8_t *d_fixed_a = nullptr, *d_fixed_b = nullptr;
        if (kernel_id == 14 && st == ESMM_OK) {
            // no preprocessing inside the loop: both pattern arrays are constants of the call
            cudaError_t e = cudaMalloc(&d_fixed_a, a_bytes);
            if (e == cudaSuccess) e = cudaMalloc(&d_fixed_b, b_bytes);
            if (e == cudaSuccess) e = cudaMemset(d_fixed_a, (1 << prefix) - 1, a_bytes);
            if (e == cudaSuccess) e = cudaMemset(d_fixed_b, 0xFF, b_bytes);
            if (e != cudaSuccess) st = esmm::record_cuda_error(e, "pattern constants for id 14");
        }
        // Id 129: B is prepared once per runner call ("B offline", like a cached pattern array); the loop holds
        // what a call costs: split of A, A patterns, product.
        esmm_tf32x3_b *tf_b = nullptr;
        void *d_tf_ws = nullptr;
        if (kernel_id == 129 && st == ESMM_OK) {
            st = esmm_tf32x3_b_create(d_B, inners, cols, 1, &tf_b);
            if (st == ESMM_OK) {
                cudaError_t e = cudaMalloc(&d_tf_ws, esmm_tf32x3_workspace_bytes(rows, inners));
                if (e != cudaSuccess) st = esmm::record_cuda_error(e, "cudaMalloc(3xTF32 workspace)");
            }
        }
        // (the tiled kernel's once-per-device set-up is not part of a run)
        if (d_packed && st == ESMM_OK) st = esmm::gemm_ab_packed_prepare();
        cudaEventRecord(start);
        for (int i = 0; i < runs && st == ESMM_OK; ++i) {
            cudaMemset(d_C, 0, (size_t)rows * cols * sizeof(float));
            if (kernel_id == 129) {
                st = esmm_sgemm_joint_tf32x3(rows, d_A, tf_b, d_C, d_tf_ws, nullptr);
                cudaDeviceSynchronize();
                continue;
            }
            if (kernel_id == 14) {
                // the reference launches nothing for other counts and leaves C zeroed
                if (prefix == 1 || prefix == 2 || prefix == 4 || prefix == 6 || prefix == 8)
                    st = esmm::gemm_ab_launch(rows, cols, inners, d_A, d_B, d_C, d_fixed_a, d_fixed_b, 32, 0);
                continue;
            }
            if (kernel_id == 16 || kernel_id == 17) {
                // One operand's patterns per run (analyze_sparsity_pattern_gpu / analyze_b_sparsity_warp_
                // granularity + free, include/runners.cuh:172-178, 236-242); the other operand counts as
                // all live.  For id 17 the packing pass still leaves out 32-row blocks of A that are all
                // zero at some k; that drops only terms that are exactly zero.
                uint8_t *d_ap = nullptr, *d_bp = nullptr;
                cudaError_t e = cudaMalloc(&d_ap, a_bytes);
                if (e == cudaSuccess) e = cudaMalloc(&d_bp, b_bytes);
                if (e != cudaSuccess) st = esmm::record_cuda_error(e, "cudaMalloc(patterns)");
                if (st == ESMM_OK) {
                    if (kernel_id == 16) {
                        e = cudaMemsetAsync(d_bp, 0xFF, b_bytes, 0);
                        if (e != cudaSuccess) st = esmm::record_cuda_error(e, "cudaMemsetAsync(B patterns)");
                    } else {
                        st = esmm_preprocess_b(d_B, inners, cols, d_bp, 0);
                    }
                }
                if (st == ESMM_OK) st = esmm::preprocess_a_pack_launch(d_A, rows, inners, d_ap, d_packed, 0);
                if (st == ESMM_OK)
                    st = esmm::gemm_ab_packed_launch(rows, cols, inners, d_packed, d_B, d_C, d_ap, d_bp, 0);
                cudaDeviceSynchronize();
                cudaFree(d_ap);
                cudaFree(d_bp);
                continue;
            }
            esmm_ab_pattern_metadata meta;
            st = esmm_preprocess_ab(d_A, d_B, rows, cols, inners, a_tile, d_b_pat_cached, &meta);
            if (st != ESMM_OK) break;
            if (d_packed) {
                st = esmm::preprocess_a_pack_launch(d_A, rows, inners, meta.d_a_patterns, d_packed, 0);
                if (st == ESMM_OK)
                    st = esmm::gemm_ab_packed_launch(rows, cols, inners, d_packed, d_B, d_C, meta.d_a_patterns,
                                                     meta.d_b_patterns, 0);
            } else {
                st = esmm::gemm_ab_launch(rows, cols, inners, d_A, d_B, d_C, meta.d_a_patterns,
                                          meta.d_b_patterns, a_tile, 0);
            }
            cudaDeviceSynchronize();
            esmm_free_ab_pattern_metadata(&meta);
        }
        cudaEventRecord(stop);
        cudaEventSynchronize(stop);
        if (d_packed) cudaFree(d_packed);
        esmm_tf32x3_b_destroy(tf_b);
        if (d_tf_ws) cudaFree(d_tf_ws);
        if (d_fixed_a) cudaFree(d_fixed_a);
        if (d_fixed_b) cudaFree(d_fixed_b);
    }

    float ms = 0.f;
    cudaEventElapsedTime(&ms, start, stop);
    cudaEventDestroy(start);
    cudaEventDestroy(stop);
    printf("Kernel time: %.3f ms (avg: %.3f ms)\n", ms, ms / runs);
    if (kernel_id == 129)
        printf("  (id 129: B is split and its patterns are prepared once, outside the timed loop; ids 20-30 recompute\n"
               "   B's patterns in every run unless cached patterns are supplied)\n");
    if (avg_ms) *avg_ms = ms / runs;

    if (st != ESMM_OK) {
        printf("ESMM error: %s %s\n", esmm_strerror(st), esmm_last_cuda_error());
        return st;
    }
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        printf("CUDA error: %s\n", cudaGetErrorString(err));
        return esmm::record_cuda_error(err, "after kernel runs");
    }
    if (kernel_id != 15) {
        st = esmm_device_status(nullptr);
        if (st != ESMM_OK) {
            printf("ESMM error: %s\n", esmm_strerror(st));
            return st;
        }
    }
    bool ok = true;
    if (kernel_id == 15) {
        if (h_C) cudaMemcpy(h_C, d_C, (size_t)rows * cols * sizeof(float), cudaMemcpyDeviceToHost);
    } else if (verify) {
        cudaMemcpy(h_C, d_C, (size_t)rows * cols * sizeof(float), cudaMemcpyDeviceToHost);
        ok = verify_results_host(h_C, h_C_ref, (long)rows * cols, 1e-2f, cols);
    }
    if (passed) *passed = ok ? 1 : 0;
    fflush(stdout);
    return ok ? ESMM_OK : ESMM_ERR_VERIFY;
}

}  // extern "C"
