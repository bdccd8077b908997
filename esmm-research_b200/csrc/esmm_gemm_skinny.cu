// Joint-sparse FP32 SGEMM for sm_100a, few rows: M <= 32 (one 32-row pattern block of A).
//
// Same arithmetic as the packed kernel (esmm_gemm_packed.cu) and as esmm_ab_optimized_v3 of the
// reference (src/kernels/esmm_ab_optimized_v3.cu:157, 183-203): for every output one FMA chain in
// ascending k over the k whose joint bit is set.  With a single row block of A the large kernel has
// M / 128 x N / 128 = N / 128 tiles, runs half of its consumer warps on rows that do not exist and
// leaves a third of the SMs idle (N = 11008: 86 tiles).  Here the work is cut the other way:
//
//   * one CTA per 32-column strip of C (N / 32 CTAs, several resident per SM).  A strip is exactly one
//     pattern block of B, so its live k are a_pat[0][kb] & b_pat[strip][kb]: every listed row is live
//     for the whole CTA, there are no per-warp masks and no index lists in the inner loop;
//   * all threads first build the strip's list of live k; then stages of 32 rows travel through a ring
//     as 16-byte asynchronous copies (cp.async, one commit group per stage), every thread moving 4 of a
//     stage's 512 pieces: per row 128 bytes of packed A (rows 0-31 of the first panel) and 128 of B;
//   * four warps, one per SM sub-partition, hold 32 rows x 8 columns each, 4 rows x 2 columns per thread:
//     per k a 16-byte and an 8-byte load and 4 two-wide FMAs (fma.rn.f32x2, 2 x 2 blocks as in the packed
//     kernel).
//
// Variants measured on M = 16, N = 11008, K = 4096 (819 live k per strip): a tensor-copy producer warp
// with two computing warps, a cp.async producer warp with four, one warp per strip with 8 x 4 outputs per
// thread - all between 33 and 45 us against 55 us for the tiled kernel; this form is the simplest of the
// fast ones.  The only waits are cp.async.wait_group and __syncthreads with a trip count common to all
// threads: no flag or barrier that another agent has to signal, nothing that can wait forever.
#include <cstring>

#include "esmm_gemm_shared.cuh"

namespace esmm {

constexpr int SK_COLS = 32;                     // columns of a strip = one B pattern block
constexpr int SK_ROWS = 32;                     // rows of C handled (M <= 32)
constexpr int SK_STAGE_ROWS = 32;               // k per stage
constexpr int SK_ROW_BYTES = 128;               // one k of either operand in shared memory
constexpr int SK_HALF = SK_STAGE_ROWS * SK_ROW_BYTES;   // 4096: A rows, then B rows
constexpr int SK_STAGE_BYTES = 2 * SK_HALF;     // 8192
constexpr int SK_STAGES = 6;
constexpr int SK_WARPS = 4;                      // one per SM sub-partition
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_MAX_KP = 16384;                // longest K the row list is sized for

// Optional timeline for tuning (build with -DESMM_TRACE), as in the packed kernel.
#ifdef ESMM_TRACE
__device__ unsigned long long g_sk_trace[1024];
#define SK_STAMP(idx)                                                                                \
    do {                                                                                             \
        if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && (idx) < 1024) g_sk_trace[(idx)] = global_timer_ns();     \
    } while (0)
#else
#define SK_STAMP(idx) \
    do {              \
    } while (0)
#endif

struct SkinnyParams {
    int M, N, K, nKB, kp, cap;
    const uint8_t *a_pat;   // row block 0 of the A patterns
    const uint8_t *b_pat;
    const float *a_packed;  // [k][128]: rows 0-31 of the first panel are read
    const float *B;
    float *C;
    int *status;
};

// 16-byte asynchronous copy global -> shared; src_bytes = 0 writes zeros instead
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src, int src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

__device__ __forceinline__ void cp_async_commit()
{
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// returns when at most N of this thread's copy groups are still in flight
template <int N>
__device__ __forceinline__ void cp_async_wait_group()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ int sk_scan(int v, int lane)
{
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xFFFFFFFFu, v, d);
        if (lane >= d) v += t;
    }
    return v;
}

__global__ void __launch_bounds__(SK_THREADS)
esmm_joint_sgemm_skinny_kernel(const SkinnyParams p)
{
    extern __shared__ __align__(1024) char smem[];
    // layout: ring | krow (u16 x cap) | warp sums
    uint16_t *krow = reinterpret_cast<uint16_t *>(smem + SK_STAGES * SK_STAGE_BYTES);
    volatile int *wsum = reinterpret_cast<volatile int *>(smem + SK_STAGES * SK_STAGE_BYTES + ((p.cap * 2 + 15) & ~15));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int strip = blockIdx.x;
    SK_STAMP(0);

    // ---------------- the strip's list of live k ----------------
    // Thread t owns the K blocks t * per .. t * per + per - 1 (consecutive threads, ascending k): count,
    // prefix over the CTA, write.
    {
        const uint8_t *bp = p.b_pat + (size_t)strip * p.nKB;
        const int per = (p.nKB + SK_THREADS - 1) / SK_THREADS;
        const int kb_lo = min((int)threadIdx.x * per, p.nKB), kb_hi = min(kb_lo + per, p.nKB);
        int c = 0;
        for (int kb = kb_lo; kb < kb_hi; ++kb) c += __popc((unsigned)(p.a_pat[kb] & bp[kb]));
        const int incl = sk_scan(c, lane);
        if (lane == 31) wsum[warp] = incl;
        __syncthreads();
        int q = incl - c;
        for (int w = 0; w < warp; ++w) q += wsum[w];
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
            unsigned live = (unsigned)(p.a_pat[kb] & bp[kb]);
            while (live) {
                krow[q++] = (uint16_t)(kb * BK + __ffs((int)live) - 1);
                live &= live - 1u;
            }
        }
        __syncthreads();
    }
    int n = 0;
#pragma unroll
    for (int w = 0; w < SK_WARPS; ++w) n += wsum[w];
    const int num_stages = (n + SK_STAGE_ROWS - 1) / SK_STAGE_ROWS;
    SK_STAMP(1);

    // ---------------- copies: every thread moves 4 of a stage's 512 sixteen-byte pieces ----------------
    // (Rows of 128 bytes are too short for the tensor copy engine, which spends about as long on a row of
    // 128 bytes as on one of 512: measured, one row per ~17 cycles per SM.)
    const int col0 = strip * SK_COLS, chunk = threadIdx.x & 7, sub = threadIdx.x >> 3;   // sub: 0 .. 15
    const bool col_ok = col0 + chunk * 4 < p.N;
    auto issue = [&](int stage) {
        if (stage < num_stages) {
            const int r0 = stage * SK_STAGE_ROWS, cnt = min(SK_STAGE_ROWS, n - r0);
            const uint32_t sa = smem_u32(smem) + (uint32_t)(stage % SK_STAGES) * SK_STAGE_BYTES + (uint32_t)chunk * 16;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = i * 16 + sub;
                if (r < cnt) {
                    const int k = krow[r0 + r];
                    cp_async_16(sa + r * SK_ROW_BYTES, p.a_packed + (size_t)k * TILE_M + chunk * 4, 16);
                    const bool b_ok = col_ok && k < p.K;   // outside B: zero fill
                    cp_async_16(sa + SK_HALF + r * SK_ROW_BYTES, b_ok ? p.B + (size_t)k * p.N + col0 + chunk * 4 : p.B,
                                b_ok ? 16 : 0);
                }
            }
        }
        cp_async_commit();   // one group per stage, empty past the end: the wait below counts groups
    };

    // ---------------- 32 rows x 8 columns per warp, 4 x 2 per thread ----------------
    // every 4 consecutive lanes touch 2 row groups x 2 column pairs (few distinct bytes per load)
    const int rg = ((lane >> 1) & 3) | ((lane >> 4) << 2);       // group of 4 rows
    const int cp = (lane & 1) | (((lane >> 3) & 1) << 1);        // pair of columns within the warp's 8
    const char *tA = smem + rg * 16;
    const char *tB = smem + SK_HALF + warp * 32 + cp * 8;
    // rows 2p, 2p+1 x the column pair: diag[p] = (c[2p][0], c[2p+1][1]), anti[p] = (c[2p][1], c[2p+1][0])
    float2 diag[2], anti[2];
    diag[0] = diag[1] = anti[0] = anti[1] = make_float2(0.0f, 0.0f);

#pragma unroll
    for (int s = 0; s < SK_STAGES - 1; ++s) issue(s);
    for (int s = 0; s < num_stages; ++s) {
        cp_async_wait_group<SK_STAGES - 2>();   // this thread's pieces of stage s have landed ...
        __syncthreads();                        // ... everybody's have, and stage s - 1 has been read by all
        issue(s + SK_STAGES - 1);               // into the slot of stage s - 1
        if (warp == 0) SK_STAMP(10 + s);
        const int cnt = min(SK_STAGE_ROWS, n - s * SK_STAGE_ROWS);
        const char *sA = tA + (size_t)(s % SK_STAGES) * SK_STAGE_BYTES;
        const char *sB = tB + (size_t)(s % SK_STAGES) * SK_STAGE_BYTES;
        auto row = [&](int r) {
            const float4 a = *reinterpret_cast<const float4 *>(sA + r * SK_ROW_BYTES);
            const float2 b = *reinterpret_cast<const float2 *>(sB + r * SK_ROW_BYTES);
            const float2 a01 = make_float2(a.x, a.y), a23 = make_float2(a.z, a.w), bs = make_float2(b.y, b.x);
            diag[0] = __ffma2_rn(a01, b, diag[0]);
            anti[0] = __ffma2_rn(a01, bs, anti[0]);
            diag[1] = __ffma2_rn(a23, b, diag[1]);
            anti[1] = __ffma2_rn(a23, bs, anti[1]);
        };
        if (cnt == SK_STAGE_ROWS) {
#pragma unroll 16
            for (int r = 0; r < SK_STAGE_ROWS; ++r) row(r);
        } else {
            for (int r = 0; r < cnt; ++r) row(r);
        }
        if (warp == 0) SK_STAMP(200 + s);
    }
    cp_async_wait_group<0>();   // nothing of this thread is in flight when it leaves
    SK_STAMP(5);

    // C is overwritten (beta = 0); un-scramble the 2 x 2 blocks into rows
    const int col = strip * SK_COLS + warp * 8 + cp * 2;
#pragma unroll
    for (int pr = 0; pr < 2; ++pr)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int r = rg * 4 + 2 * pr + e;
            const float2 v = e == 0 ? make_float2(diag[pr].x, anti[pr].x) : make_float2(anti[pr].y, diag[pr].y);
            if (r < p.M && col < p.N) *reinterpret_cast<float2 *>(p.C + (size_t)r * p.N + col) = v;
        }
}

#ifdef ESMM_TRACE
extern "C" int esmm_sk_trace_read(unsigned long long *host, int n)
{
    return (int)cudaMemcpyFromSymbol(host, g_sk_trace, sizeof(unsigned long long) * (n < 1024 ? n : 1024));
}
#endif

// Whether the few-rows kernel takes a problem (otherwise the packed kernel does).
bool gemm_ab_skinny_applies(int M, int N, int K)
{
    const int kp = ceil_div(K, BK) * BK;
    return M <= SK_ROWS && kp <= SK_MAX_KP && N >= 4 * SK_COLS && tuning_get("NO_SKINNY", 0) == 0;
}

int gemm_ab_skinny_launch(int M, int N, int K, const float *d_a_packed, const float *d_B, float *d_C,
                          const uint8_t *d_a_pat, const uint8_t *d_b_pat, cudaStream_t stream)
{
    SkinnyParams p;
    memset(&p, 0, sizeof p);
    p.M = M;
    p.N = N;
    p.K = K;
    p.nKB = ceil_div(K, BK);
    p.kp = p.nKB * BK;
    p.cap = p.kp + 32;
    p.a_pat = d_a_pat;
    p.b_pat = d_b_pat;
    p.a_packed = d_a_packed;
    p.B = d_B;
    p.C = d_C;
    p.status = device_status_ptr();
    if (!p.status) return ESMM_ERR_CUDA;
    // ring, row list, one int per warp
    const size_t smem = (size_t)SK_STAGES * SK_STAGE_BYTES + ((p.cap * 2 + 15) & ~15) + (SK_WARPS * 4 + 15) / 16 * 16;
    ESMM_CUDA_TRY(cudaFuncSetAttribute(esmm_joint_sgemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem));
    esmm_joint_sgemm_skinny_kernel<<<ceil_div(N, SK_COLS), SK_THREADS, smem, stream>>>(p);
    ESMM_CUDA_TRY(cudaGetLastError());
    return ESMM_OK;
}

}  // namespace esmm
