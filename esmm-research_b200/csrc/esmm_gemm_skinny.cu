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
//   * all threads first build the strip's list of live k (pattern bytes read as 32-bit words); then stages of
//     32 rows travel through a ring as 16-byte asynchronous copies (cp.async, one commit group per stage): per
//     row 128 bytes of B and 128 bytes of packed A (rows 0-31 of the first panel), or only 64 bytes of A (rows
//     0-15) when M <= 16 - the 16-row variant moves and multiplies half as much of A;
//   * four warps, one per SM sub-partition, hold ROWS rows x 8 columns each, (ROWS / 8) rows x 2 columns per
//     thread, as 2 x 2 blocks of two-wide FMAs (fma.rn.f32x2) like the packed kernel.  The operands of four rows
//     are loaded (volatile, so that they stay put) one batch ahead of the multiply-adds that use them, two
//     register sets in ping-pong: without that the compiler sank every load to its first use and a row cost a
//     shared-memory round trip (36 cycles per row and warp measured; 26 with the batches).
//
// Measured on M = 16, N = 11008, K = 4096 (819 live k per strip, 344 CTAs on 148 SMs), kernel alone, back to back:
// 24.8 us (35.5 us before the 16-row variant and the batched loads; tiled kernel 49 us; cuBLAS 110 us).  What is
// left: an SM holds 2 or 3 strips, i.e. 8-12 warps, and every asynchronous-copy or shared-load instruction costs its
// warp tens of cycles of issue whatever its width (a warp-wide 16-byte cp.async: about 26 cycles, measured), so the
// row rate is set by the number of such instructions, not by bytes.  Variants measured and dropped: a tensor-copy
// producer warp with two computing warps, a cp.async producer warp with four, one warp per strip with 8 x 4 outputs per
// thread (33-45 us, before batching); two warps per strip, 16 columns and (ROWS / 8) x 4 outputs per thread each, with
// private rings and no barrier in the main loop (28.2 us at M = 16, 49.3 us at M = 32: twice the copy instructions per
// warp) or on one shared ring (28.9 / 37.4 us).
// The only waits are cp.async.wait_group and __syncthreads with a trip count common to all threads: no flag or
// barrier that another agent has to signal, nothing that can wait forever.
#include <cstring>

#include "esmm_gemm_shared.cuh"

namespace esmm {

constexpr int SK_COLS = 32;                     // columns of a strip = one B pattern block
constexpr int SK_ROWS = 32;                     // rows of C handled (M <= 32)
constexpr int SK_STAGE_ROWS = 32;               // k per stage
constexpr int SK_ROW_BYTES = 128;               // one k of either operand in shared memory
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

// ROWS = 32: rows 0-31 of the first panel (any M <= 32).  ROWS = 16 (M <= 16): only rows 0-15 are fetched and
// multiplied - half the shared-memory traffic of A and half the multiply-adds.
template <int ROWS>
__global__ void __launch_bounds__(SK_THREADS)
esmm_joint_sgemm_skinny_kernel(const SkinnyParams p)
{
    constexpr int A_ROW_BYTES = ROWS * 4;                           // one k of A in shared memory
    constexpr int A_CHUNKS = A_ROW_BYTES / 16;                      // 16-byte pieces per A row
    constexpr int A_HALF = SK_STAGE_ROWS * A_ROW_BYTES;             // A rows, then B rows
    constexpr int STAGE_BYTES = A_HALF + SK_STAGE_ROWS * SK_ROW_BYTES;
    constexpr int BATCH = 4;                                        // rows per register set of operands
    extern __shared__ __align__(1024) char smem[];
    // layout: ring | krow (u16 x cap) | warp sums
    uint16_t *krow = reinterpret_cast<uint16_t *>(smem + SK_STAGES * STAGE_BYTES);
    volatile int *wsum = reinterpret_cast<volatile int *>(smem + SK_STAGES * STAGE_BYTES + ((p.cap * 2 + 15) & ~15));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int strip = blockIdx.x;
    SK_STAMP(0);
    grid_dependency_wait();   // (the A patterns and the packed copy come from the kernel before this one)

    // ---------------- the strip's list of live k ----------------
    // Thread t owns the K blocks t * per .. t * per + per - 1 (consecutive threads, ascending k; per a multiple
    // of 4 so that a thread's pattern bytes are whole 32-bit words where the arrays allow): count, prefix over
    // the CTA, write.
    {
        constexpr int MAX_WORDS = SK_MAX_KP / BK / SK_THREADS / 4;   // 4 words of 4 K blocks per thread at most
        const uint8_t *bp = p.b_pat + (size_t)strip * p.nKB;
        const int per = ((p.nKB + SK_THREADS - 1) / SK_THREADS + 3) & ~3;
        const int kb_lo = min((int)threadIdx.x * per, p.nKB), kb_hi = min(kb_lo + per, p.nKB);
        const bool words = (p.nKB & 3) == 0 && ((reinterpret_cast<uintptr_t>(p.a_pat) | reinterpret_cast<uintptr_t>(bp)) & 3) == 0;
        unsigned live[MAX_WORDS];
        int c = 0;
#pragma unroll
        for (int w = 0; w < MAX_WORDS; ++w) {
            const int kb = kb_lo + 4 * w;
            unsigned v = 0u;
            if (kb < kb_hi) {
                if (words) {
                    v = *reinterpret_cast<const unsigned *>(p.a_pat + kb) & *reinterpret_cast<const unsigned *>(bp + kb);
                } else {
                    for (int j = 0; j < 4 && kb + j < kb_hi; ++j) v |= (unsigned)(p.a_pat[kb + j] & bp[kb + j]) << (8 * j);
                }
            }
            live[w] = v;
            c += __popc(v);
        }
        const int incl = sk_scan(c, lane);
        if (lane == 31) wsum[warp] = incl;
        __syncthreads();
        int q = incl - c;
        for (int w = 0; w < warp; ++w) q += wsum[w];
#pragma unroll
        for (int w = 0; w < MAX_WORDS; ++w) {
            unsigned v = live[w];
            while (v) {
                const int bit = __ffs((int)v) - 1;                   // bit 8 j + kk: K block kb_lo + 4 w + j, offset kk
                if (bounds_ok(q < p.cap, p.status, 30)) krow[q] = (uint16_t)((kb_lo + 4 * w) * BK + bit);   // checked build: site 30
                ++q;
                v &= v - 1u;
            }
        }
        __syncthreads();
    }
    int n = 0;
#pragma unroll
    for (int w = 0; w < SK_WARPS; ++w) n += wsum[w];
    const int num_stages = (n + SK_STAGE_ROWS - 1) / SK_STAGE_ROWS;
    SK_STAMP(1);

    // ---------------- copies: every thread moves up to 4 of a stage's sixteen-byte pieces ----------------
    // (Rows of 128 bytes are too short for the tensor copy engine, which spends about as long on a row of
    // 128 bytes as on one of 512: measured, one row per ~17 cycles per SM.)
    const int col0 = strip * SK_COLS, chunk = threadIdx.x & 7, sub = threadIdx.x >> 3;   // sub: 0 .. 15
    const bool col_ok = col0 + chunk * 4 < p.N;
    auto issue = [&](int stage) {
        if (stage < num_stages) {
            const int r0 = stage * SK_STAGE_ROWS, cnt = min(SK_STAGE_ROWS, n - r0);
            const uint32_t s0 = smem_u32(smem) + (uint32_t)(stage % SK_STAGES) * STAGE_BYTES + (uint32_t)chunk * 16;
#pragma unroll
            for (int i = 0; i < SK_STAGE_ROWS / 16; ++i) {
                const int r = i * 16 + sub;
                if (r < cnt && bounds_ok(r0 + r < p.cap, p.status, 31)) {
                    const int k = krow[r0 + r];
                    if (!bounds_ok(k >= 0 && k < p.kp, p.status, 32)) continue;   // site 32: a k outside the packed panel / B
                    if (chunk < A_CHUNKS)
                        cp_async_16(s0 + r * A_ROW_BYTES, p.a_packed + (size_t)k * TILE_M + chunk * 4, 16);
                    const bool b_ok = col_ok && k < p.K;   // outside B: zero fill
                    cp_async_16(s0 + A_HALF + r * SK_ROW_BYTES, b_ok ? p.B + (size_t)k * p.N + col0 + chunk * 4 : p.B,
                                b_ok ? 16 : 0);
                }
            }
        }
        cp_async_commit();   // one group per stage, empty past the end: the wait below counts groups
    };

    // ---------------- per warp ROWS rows x 8 columns; per thread (ROWS / 8) rows x 2 columns ----------------
    // every 4 consecutive lanes touch 2 row groups x 2 column pairs (few distinct bytes per load)
    const int rg = ((lane >> 1) & 3) | ((lane >> 4) << 2);       // group of ROWS / 8 consecutive rows
    const int cp = (lane & 1) | (((lane >> 3) & 1) << 1);        // pair of columns within the warp's 8
    const uint32_t tA = smem_u32(smem) + rg * (ROWS / 2);
    const uint32_t tB = smem_u32(smem) + A_HALF + warp * 32 + cp * 8;
    // rows 2p, 2p+1 x the column pair: diag[p] = (c[2p][0], c[2p+1][1]), anti[p] = (c[2p][1], c[2p+1][0])
    constexpr int RP = ROWS / 16;                                 // row pairs per thread
    float2 diag[RP], anti[RP];
#pragma unroll
    for (int i = 0; i < RP; ++i) diag[i] = anti[i] = make_float2(0.0f, 0.0f);

    // Operands of BATCH consecutive rows of a stage.  The loop below loads the next batch before it multiplies
    // the current one (two register sets, ping-pong), so that a load has a whole batch of multiply-adds to land
    // under; the loads are volatile so that they stay where they are written.
    struct Ops {
        float2 a[BATCH][RP], b[BATCH];
    };
    auto load_rows = [&](Ops &o, uint32_t sA, uint32_t sB, int r) {
#pragma unroll
        for (int i = 0; i < BATCH; ++i) {
            const uint32_t pa = sA + (uint32_t)((r + i) * A_ROW_BYTES), pb = sB + (uint32_t)((r + i) * SK_ROW_BYTES);
            if (RP == 2)
                asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                             : "=f"(o.a[i][0].x), "=f"(o.a[i][0].y), "=f"(o.a[i][RP - 1].x), "=f"(o.a[i][RP - 1].y) : "r"(pa));
            else
                asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(o.a[i][0].x), "=f"(o.a[i][0].y) : "r"(pa));
            asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(o.b[i].x), "=f"(o.b[i].y) : "r"(pb));
        }
    };
    auto fma_rows = [&](const Ops &o, int count) {
#pragma unroll
        for (int i = 0; i < BATCH; ++i) {
            if (i < count) {
                const float2 bs = make_float2(o.b[i].y, o.b[i].x);
#pragma unroll
                for (int pr = 0; pr < RP; ++pr) {
                    diag[pr] = __ffma2_rn(o.a[i][pr], o.b[i], diag[pr]);
                    anti[pr] = __ffma2_rn(o.a[i][pr], bs, anti[pr]);
                }
            }
        }
    };

#pragma unroll
    for (int s = 0; s < SK_STAGES - 1; ++s) issue(s);
    for (int s = 0; s < num_stages; ++s) {
        cp_async_wait_group<SK_STAGES - 2>();   // this thread's pieces of stage s have landed ...
        __syncthreads();                        // ... everybody's have, and stage s - 1 has been read by all
        issue(s + SK_STAGES - 1);               // into the slot of stage s - 1
        if (warp == 0) SK_STAMP(10 + s);
        const int cnt = min(SK_STAGE_ROWS, n - s * SK_STAGE_ROWS);
        const uint32_t sA = tA + (uint32_t)(s % SK_STAGES) * STAGE_BYTES;
        const uint32_t sB = tB + (uint32_t)(s % SK_STAGES) * STAGE_BYTES;
        // (a batch loaded past the stage's last row reads the next slot or the row list: in bounds, never multiplied)
        Ops x, y;
        load_rows(x, sA, sB, 0);
        if (cnt == SK_STAGE_ROWS) {
#pragma unroll 1
            for (int r = 0; r < SK_STAGE_ROWS; r += 2 * BATCH) {
                load_rows(y, sA, sB, r + BATCH);
                fma_rows(x, BATCH);
                load_rows(x, sA, sB, r + 2 * BATCH);
                fma_rows(y, BATCH);
            }
        } else {
#pragma unroll 1
            for (int r = 0; r < cnt; r += BATCH) {
                fma_rows(x, min(BATCH, cnt - r));
                load_rows(x, sA, sB, r + BATCH);
            }
        }
        if (warp == 0) SK_STAMP(200 + s);
    }
    cp_async_wait_group<0>();   // nothing of this thread is in flight when it leaves
    SK_STAMP(5);

    // C is overwritten (beta = 0); un-scramble the 2 x 2 blocks into rows
    const int col = strip * SK_COLS + warp * 8 + cp * 2;
#pragma unroll
    for (int pr = 0; pr < RP; ++pr)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int r = rg * (ROWS / 8) + 2 * pr + e;
            const float2 v = e == 0 ? make_float2(diag[pr].x, anti[pr].x) : make_float2(anti[pr].y, diag[pr].y);
            if (r < p.M && col < p.N && bounds_ok((size_t)r * p.N + col + 2 <= (size_t)p.M * p.N, p.status, 33))
                *reinterpret_cast<float2 *>(p.C + (size_t)r * p.N + col) = v;
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
    const bool rows16 = M <= 16 && tuning_get("SKINNY_ROWS", 0) != 32;
    // ring, row list, one int per warp
    const size_t stage_bytes = (size_t)SK_STAGE_ROWS * ((rows16 ? 16 : 32) * 4 + SK_ROW_BYTES);
    const size_t smem = (size_t)SK_STAGES * stage_bytes + ((p.cap * 2 + 15) & ~15) + (SK_WARPS * 4 + 15) / 16 * 16;
    if (rows16) {
        ESMM_CUDA_TRY(cudaFuncSetAttribute(esmm_joint_sgemm_skinny_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem));
        ESMM_CUDA_TRY(launch_dependent(esmm_joint_sgemm_skinny_kernel<16>, dim3(ceil_div(N, SK_COLS)), dim3(SK_THREADS), smem, stream, p));
    } else {
        ESMM_CUDA_TRY(cudaFuncSetAttribute(esmm_joint_sgemm_skinny_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem));
        ESMM_CUDA_TRY(launch_dependent(esmm_joint_sgemm_skinny_kernel<32>, dim3(ceil_div(N, SK_COLS)), dim3(SK_THREADS), smem, stream, p));
    }
    ESMM_CUDA_TRY(cudaGetLastError());
    return ESMM_OK;
}

}  // namespace esmm
