// Joint-sparse FP32 SGEMM for sm_100a: C = A * B over the k whose joint pattern bit is set.
//
// Stands in for esmm_ab_optimized_v3 and dispatch_v3 of the reference
// (src/kernels/esmm_ab_optimized_v3.cu:18-235, include/runners.cuh:801-825) with the same
// arithmetic - one FFMA chain per output, ascending k, live k only, C overwritten - and a
// different machine mapping:
//
//   * persistent CTAs, one per SM, each walking 128 x 128 tiles of C;
//   * 16 consumer warps, each owning one 32 x 32 block of the tile, i.e. exactly one
//     (A pattern row, B pattern row) pair, so every skip decision is warp-uniform;
//   * one TMA warp that streams K blocks (A box 128 rows x 8 k, 32-byte swizzled; B box
//     8 k x 128 columns, or single live k rows when few are live) into a ring of stages
//     guarded by full/empty mbarriers, and never issues a copy for a K block whose joint
//     mask is zero for the whole tile;
//   * one mask warp that, one tile ahead, joins the A and B pattern bytes of the tile into
//     a compacted list of live K blocks with their per-warp-row / per-warp-column masks.
//
// Every wait is bounded; a wait that expires raises the device status word and the CTA
// leaves after waiting (bounded again) for its copies in flight.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "esmm_common.cuh"

namespace esmm {

constexpr int TILE_M = 128;
constexpr int TILE_N = 128;
constexpr int KB_PER_STAGE = 4;                      // live K blocks per pipeline stage
constexpr int A_SUB_BYTES = TILE_M * BK * 4;         // 4096: one K block of the A tile
constexpr int B_ROW_BYTES = TILE_N * 4;              // 512: one k row of the B tile
constexpr int B_SUB_BYTES = BK * B_ROW_BYTES;        // 4096
constexpr int STAGE_A_BYTES = KB_PER_STAGE * A_SUB_BYTES;
constexpr int STAGE_BYTES = KB_PER_STAGE * (A_SUB_BYTES + B_SUB_BYTES);  // 32768
constexpr int CONSUMER_WARPS = 16;
constexpr int TMA_WARP = CONSUMER_WARPS;
constexpr int MASK_WARP = CONSUMER_WARPS + 1;
constexpr int GEMM_THREADS = (CONSUMER_WARPS + 2) * 32;  // 576
constexpr int MAX_STAGES = 6;
constexpr int GROUP_M = 8;                           // tile rows per raster group
constexpr int SMEM_LIMIT = 232448;                   // 227 KB per CTA on sm_100

struct GemmParams {
    int M, N, K;
    int nKB;         // ceil(K / 8)
    int nKBpad;      // capacity of the per-tile live lists (multiple of 4)
    int a_rows;      // rows of the A pattern array
    int b_rows;      // rows of the B pattern array (ceil(N / 32))
    int a_div;       // 32-row block mb uses A pattern rows (mb / a_div) * a_mul + [0, a_mul)
    int a_mul;
    int tiles_m, tiles_n, num_tiles;
    int stages;
    int swizzle;     // 1: A boxes are 32-byte swizzled
    int brow_bits;   // B rows are fetched one by one when a K block has at most this many live k
    const uint8_t *a_pat;
    const uint8_t *b_pat;
    float *C;
    int *status;
};

struct SmemLayout {
    uint32_t stage_off, cmask_off, cmask_stride, klist_off, klist_stride, bar_off, misc_off, total;
};

__host__ __device__ inline SmemLayout smem_layout(int stages, int nKBpad)
{
    SmemLayout L;
    uint32_t o = 0;
    L.stage_off = o;
    o += (uint32_t)stages * STAGE_BYTES;
    L.cmask_off = o;  // two buffers of (A word, B word) per live K block
    L.cmask_stride = (uint32_t)nKBpad * 8;
    o += 2 * L.cmask_stride;
    L.klist_off = o;  // two buffers of live K block indices
    L.klist_stride = (uint32_t)nKBpad * 2;
    o += 2 * L.klist_stride;
    o = (o + 15u) & ~15u;
    L.bar_off = o;  // full[MAX_STAGES], empty[MAX_STAGES], mask_full[2], mask_empty[2]
    o += (2 * MAX_STAGES + 4) * 8;
    L.misc_off = o;  // nlive[2], abort
    o += 16;
    L.total = o;
    return L;
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int &tm, int &tn)
{
    const int per_group = GROUP_M * tiles_n;
    const int group = tile / per_group;
    const int first_m = group * GROUP_M;
    const int gsize = min(tiles_m - first_m, GROUP_M);
    const int r = tile - group * per_group;
    tm = first_m + r % gsize;
    tn = r / gsize;
}

__device__ __forceinline__ void fma8(float (&acc)[8], float a, const float4 &b0, const float4 &b1)
{
    acc[0] = fmaf(a, b0.x, acc[0]);
    acc[1] = fmaf(a, b0.y, acc[1]);
    acc[2] = fmaf(a, b0.z, acc[2]);
    acc[3] = fmaf(a, b0.w, acc[3]);
    acc[4] = fmaf(a, b1.x, acc[4]);
    acc[5] = fmaf(a, b1.y, acc[5]);
    acc[6] = fmaf(a, b1.z, acc[6]);
    acc[7] = fmaf(a, b1.w, acc[7]);
}

// Four consecutive k (4H .. 4H+3) of one K block, all live: A comes in as one 16-byte load
// per row (the 32-byte swizzle keeps the 8 rows of a warp on distinct banks).
template <int H>
__device__ __forceinline__ void dense_half(float (&acc)[4][8], const char *sA, const char *sB,
                                           int swoff)
{
    const char *ap = sA + ((H << 4) ^ swoff);
    float a[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 v = *reinterpret_cast<const float4 *>(ap + i * 256);
        a[i][0] = v.x;
        a[i][1] = v.y;
        a[i][2] = v.z;
        a[i][3] = v.w;
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
        const char *bp = sB + (4 * H + kk) * B_ROW_BYTES;
        const float4 b0 = *reinterpret_cast<const float4 *>(bp);
        const float4 b1 = *reinterpret_cast<const float4 *>(bp + 64);
#pragma unroll
        for (int i = 0; i < 4; ++i) fma8(acc[i], a[i][kk], b0, b1);
    }
}

// The live k of one nibble (bits of `nib` are k offsets 4H .. 4H+3), one at a time, ascending.
template <int H>
__device__ __forceinline__ void sparse_half(float (&acc)[4][8], const char *sA, const char *sB,
                                            int swoff, unsigned nib)
{
    const char *ap = sA + ((H << 4) ^ swoff);
    const char *bp0 = sB + 4 * H * B_ROW_BYTES;
#pragma unroll 1
    while (nib) {
        const int kk = __ffs(nib) - 1;
        nib &= nib - 1;
        const char *bp = bp0 + kk * B_ROW_BYTES;
        const float4 b0 = *reinterpret_cast<const float4 *>(bp);
        const float4 b1 = *reinterpret_cast<const float4 *>(bp + 64);
        const char *akp = ap + kk * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) fma8(acc[i], *reinterpret_cast<const float *>(akp + i * 256), b0, b1);
    }
}

__device__ __forceinline__ void compute_kblock(float (&acc)[4][8], const char *sA, const char *sB,
                                               int swoff, unsigned joint)
{
    const unsigned lo = joint & 0xFu, hi = joint >> 4;
    if (lo == 0xFu) dense_half<0>(acc, sA, sB, swoff);
    else if (lo) sparse_half<0>(acc, sA, sB, swoff, lo);
    if (hi == 0xFu) dense_half<1>(acc, sA, sB, swoff);
    else if (hi) sparse_half<1>(acc, sA, sB, swoff, hi);
}

__global__ void __launch_bounds__(GEMM_THREADS, 1)
esmm_joint_sgemm_kernel(const __grid_constant__ CUtensorMap map_a,
                        const __grid_constant__ CUtensorMap map_b_box,
                        const __grid_constant__ CUtensorMap map_b_row,
                        const GemmParams p)
{
    extern __shared__ __align__(1024) char smem[];
    const SmemLayout L = smem_layout(p.stages, p.nKBpad);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L.bar_off);
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = smem_u32(bars + MAX_STAGES);
    const uint32_t mfull0 = smem_u32(bars + 2 * MAX_STAGES);
    const uint32_t mempty0 = smem_u32(bars + 2 * MAX_STAGES + 2);
    volatile int *nlive = reinterpret_cast<volatile int *>(smem + L.misc_off);
    volatile int *abort_flag = nlive + 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, CONSUMER_WARPS);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(mfull0 + 8 * b, 1);
            mbar_init(mempty0 + 8 * b, CONSUMER_WARPS + 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();

    bool ok = true;

    if (warp == MASK_WARP) {
        // ---------------- mask warp: live K-block list of each tile ----------------
        const unsigned lt_mask = (1u << lane) - 1u;
        int it = 0;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            ok = mbar_wait(mempty0 + 8 * buf, ((it >> 1) & 1) ^ 1, abort_flag);
            if (!ok) break;
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            uint2 *cmask = reinterpret_cast<uint2 *>(smem + L.cmask_off + buf * L.cmask_stride);
            uint16_t *klist = reinterpret_cast<uint16_t *>(smem + L.klist_off + buf * L.klist_stride);
            int base = 0;
            for (int kb0 = 0; kb0 < p.nKB; kb0 += 32) {
                const int kb = kb0 + lane;
                unsigned aw = 0, bw = 0;
                if (kb < p.nKB) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int mb = tm * 4 + i;  // 32-row block of C
                        unsigned v = 0;
                        const int r0 = (mb / p.a_div) * p.a_mul;
                        for (int t = 0; t < p.a_mul; ++t)
                            if (r0 + t < p.a_rows) v |= p.a_pat[(size_t)(r0 + t) * p.nKB + kb];
                        aw |= v << (8 * i);
                        const int nb = tn * 4 + i;
                        if (nb < p.b_rows) bw |= (unsigned)p.b_pat[(size_t)nb * p.nKB + kb] << (8 * i);
                    }
                }
                unsigned au = aw | (aw >> 16), bu = bw | (bw >> 16);
                au = (au | (au >> 8)) & 0xFFu;
                bu = (bu | (bu >> 8)) & 0xFFu;
                const bool live = (au & bu) != 0;
                const unsigned bal = __ballot_sync(0xFFFFFFFFu, live);
                if (live) {
                    const int pos = base + __popc(bal & lt_mask);
                    cmask[pos] = make_uint2(aw, bw);
                    klist[pos] = (uint16_t)kb;
                }
                base += __popc(bal);
            }
            // zero the tail of the last stage so that its unused K-block slots read as dead
            if (lane < 4) {
                const int pos = base + lane;
                if (pos < ((base + 3) & ~3)) {
                    cmask[pos] = make_uint2(0u, 0u);
                    klist[pos] = 0;
                }
            }
            if (lane == 0) nlive[buf] = base;
            __syncwarp();
            if (lane == 0) mbar_arrive(mfull0 + 8 * buf);
        }
    } else if (warp == TMA_WARP) {
        // ---------------- TMA warp: stream live K blocks into the ring ----------------
        if (lane == 0) {
            tma_prefetch_descriptor(&map_a);
            tma_prefetch_descriptor(&map_b_box);
            tma_prefetch_descriptor(&map_b_row);
            int slot = 0;
            uint32_t phase = 0;
            uint32_t issued_bits = 0, parity_bits = 0;  // per slot: ever issued / parity of last issue
            int it = 0;
            for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++it) {
                const int buf = it & 1;
                ok = mbar_wait(mfull0 + 8 * buf, (it >> 1) & 1, abort_flag);
                if (!ok) break;
                int tm, tn;
                tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
                const uint2 *cmask = reinterpret_cast<const uint2 *>(smem + L.cmask_off + buf * L.cmask_stride);
                const uint16_t *klist = reinterpret_cast<const uint16_t *>(smem + L.klist_off + buf * L.klist_stride);
                const int n = nlive[buf];
                for (int i0 = 0; i0 < n; i0 += KB_PER_STAGE) {
                    ok = mbar_wait(empty0 + 8 * slot, phase ^ 1, abort_flag);
                    if (!ok) break;
                    const int cnt = min(KB_PER_STAGE, n - i0);
                    unsigned live[KB_PER_STAGE];
                    uint32_t bytes = 0;
#pragma unroll
                    for (int j = 0; j < KB_PER_STAGE; ++j) {
                        live[j] = 0;
                        if (j < cnt) {
                            const uint2 m = cmask[i0 + j];
                            unsigned au = m.x | (m.x >> 16), bu = m.y | (m.y >> 16);
                            au = (au | (au >> 8)) & 0xFFu;
                            bu = (bu | (bu >> 8)) & 0xFFu;
                            live[j] = au & bu;
                            const int bits = __popc(live[j]);
                            bytes += A_SUB_BYTES + (bits <= p.brow_bits ? bits * B_ROW_BYTES : B_SUB_BYTES);
                        }
                    }
                    const uint32_t full = full0 + 8 * slot;
                    mbar_arrive_expect_tx(full, bytes);
                    const uint32_t sbase = smem_u32(smem + L.stage_off) + (uint32_t)slot * STAGE_BYTES;
#pragma unroll
                    for (int j = 0; j < KB_PER_STAGE; ++j) {
                        if (j < cnt) {
                            const int k0 = (int)klist[i0 + j] * BK;
                            tma_load_2d(sbase + j * A_SUB_BYTES, &map_a, k0, tm * TILE_M, full);
                            const uint32_t sb = sbase + STAGE_A_BYTES + j * B_SUB_BYTES;
                            unsigned m = live[j];
                            if (__popc(m) <= p.brow_bits) {
                                while (m) {
                                    const int kk = __ffs(m) - 1;
                                    m &= m - 1;
                                    tma_load_2d(sb + kk * B_ROW_BYTES, &map_b_row, tn * TILE_N, k0 + kk, full);
                                }
                            } else {
                                tma_load_2d(sb, &map_b_box, tn * TILE_N, k0, full);
                            }
                        }
                    }
                    issued_bits |= 1u << slot;
                    parity_bits = (parity_bits & ~(1u << slot)) | (phase << slot);
                    if (++slot == p.stages) {
                        slot = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                mbar_arrive(mempty0 + 8 * buf);
            }
            if (!ok) {
                // leave only after the copies already issued have landed (bounded)
                for (int s = 0; s < p.stages; ++s) {
                    if (!(issued_bits & (1u << s))) continue;
                    const uint32_t par = (parity_bits >> s) & 1u;
                    for (int tries = 0; tries < (1 << 16); ++tries)
                        if (mbar_try_wait(full0 + 8 * s, par)) break;
                }
            }
        }
    } else {
        // ---------------- consumer warps: 32 x 32 block of the tile each ----------------
        const int wm = warp >> 2, wn = warp & 3;
        const int lm = lane >> 2, ln = lane & 3;
        const int swoff = p.swizzle ? ((lm >> 2) & 1) << 4 : 0;
        const uint32_t a_thr = (uint32_t)(wm * 32 + lm) * 32;               // row offset in an A sub-slot
        const uint32_t b_thr = STAGE_A_BYTES + (uint32_t)(wn * 32 + ln * 4) * 4;  // column offset in a B sub-slot
        const int ash = 8 * wm, bsh = 8 * wn;
        int slot = 0;
        uint32_t phase = 0;
        int it = 0;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            ok = mbar_wait(mfull0 + 8 * buf, (it >> 1) & 1, abort_flag);
            if (!ok) break;
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            const uint4 *cmask4 = reinterpret_cast<const uint4 *>(smem + L.cmask_off + buf * L.cmask_stride);
            const int n = nlive[buf];

            float acc[4][8];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

            for (int i0 = 0; i0 < n; i0 += KB_PER_STAGE) {
                const uint4 m01 = cmask4[(i0 >> 1)];
                const uint4 m23 = cmask4[(i0 >> 1) + 1];
                const unsigned j0 = ((m01.x >> ash) & (m01.y >> bsh)) & 0xFFu;
                const unsigned j1 = ((m01.z >> ash) & (m01.w >> bsh)) & 0xFFu;
                const unsigned j2 = ((m23.x >> ash) & (m23.y >> bsh)) & 0xFFu;
                const unsigned j3 = ((m23.z >> ash) & (m23.w >> bsh)) & 0xFFu;
                ok = mbar_wait(full0 + 8 * slot, phase, abort_flag);
                if (!ok) break;
                const char *sbase = smem + L.stage_off + (size_t)slot * STAGE_BYTES;
                const char *sA = sbase + a_thr;
                const char *sB = sbase + b_thr;
                if (j0) compute_kblock(acc, sA, sB, swoff, j0);
                if (j1) compute_kblock(acc, sA + A_SUB_BYTES, sB + B_SUB_BYTES, swoff, j1);
                if (j2) compute_kblock(acc, sA + 2 * A_SUB_BYTES, sB + 2 * B_SUB_BYTES, swoff, j2);
                if (j3) compute_kblock(acc, sA + 3 * A_SUB_BYTES, sB + 3 * B_SUB_BYTES, swoff, j3);
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * slot);
                if (++slot == p.stages) {
                    slot = 0;
                    phase ^= 1;
                }
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(mempty0 + 8 * buf);

            // epilogue: C is overwritten (beta = 0)
            const int row0 = tm * TILE_M + wm * 32 + lm;
            const int col0 = tn * TILE_N + wn * 32 + ln * 4;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = row0 + 8 * i;
                if (row < p.M) {
                    float *c = p.C + (size_t)row * p.N + col0;
                    if (col0 < p.N)
                        *reinterpret_cast<float4 *>(c) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
                    if (col0 + 16 < p.N)
                        *reinterpret_cast<float4 *>(c + 16) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
                }
            }
        }
    }

    if (!ok && lane == 0) atomicExch(p.status, (int)ESMM_ERR_TIMEOUT);
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// Row-major FP32 matrix of `outer` rows x `inner` columns, box = box_outer x box_inner.
static int make_map_2d(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer,
                       uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz,
                       CUtensorMapL2promotion l2)
{
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return record_cuda_error_text("cuTensorMapEncodeTiled entry point not available");
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * 4};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base), dims, strides,
                     box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, l2, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char buf[96];
        snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return record_cuda_error_text(buf);
    }
    return ESMM_OK;
}

static int env_int(const char *name, int dflt)
{
    const char *s = getenv(name);
    return (s && *s) ? atoi(s) : dflt;
}

int gemm_ab_launch(int M, int N, int K, const float *d_A, const float *d_B, float *d_C,
                   const uint8_t *d_a_pat, const uint8_t *d_b_pat, int a_tile_m, cudaStream_t stream)
{
    if (!d_A || !d_B || !d_C || !d_a_pat || !d_b_pat) return ESMM_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || (K & 3) || (N & 3)) return ESMM_ERR_SHAPE;
    if (a_tile_m <= 0 || (a_tile_m < 32 ? (32 % a_tile_m) : (a_tile_m % 32))) return ESMM_ERR_UNSUPPORTED;
    if (((uintptr_t)d_A | (uintptr_t)d_B | (uintptr_t)d_C) & 15) return ESMM_ERR_ALIGN;

    GemmParams p;
    memset(&p, 0, sizeof p);
    p.M = M;
    p.N = N;
    p.K = K;
    p.nKB = ceil_div(K, BK);
    p.nKBpad = ((p.nKB + 3) & ~3) + 4;
    p.a_rows = ceil_div(M, a_tile_m);
    p.b_rows = ceil_div(N, PAT_N);
    p.a_div = a_tile_m >= 32 ? a_tile_m / 32 : 1;
    p.a_mul = a_tile_m >= 32 ? 1 : 32 / a_tile_m;
    p.tiles_m = ceil_div(M, TILE_M);
    p.tiles_n = ceil_div(N, TILE_N);
    p.num_tiles = p.tiles_m * p.tiles_n;
    p.swizzle = env_int("ESMM_SWIZZLE", 1) ? 1 : 0;
    p.brow_bits = env_int("ESMM_BROW_BITS", 2);
    if (p.brow_bits < 0) p.brow_bits = 0;
    if (p.brow_bits > 8) p.brow_bits = 8;
    p.a_pat = d_a_pat;
    p.b_pat = d_b_pat;
    p.C = d_C;
    if (p.nKB > 65535) return ESMM_ERR_TOO_LARGE;

    int stages = env_int("ESMM_STAGES", MAX_STAGES);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) stages = 2;
    while (stages > 2 && smem_layout(stages, p.nKBpad).total > SMEM_LIMIT) --stages;
    const SmemLayout L = smem_layout(stages, p.nKBpad);
    if (L.total > SMEM_LIMIT) return ESMM_ERR_TOO_LARGE;
    p.stages = stages;

    int dev = 0, sms = 0;
    ESMM_CUDA_TRY(cudaGetDevice(&dev));
    ESMM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    p.status = device_status_ptr();
    if (!p.status) return ESMM_ERR_CUDA;

    CUtensorMap map_a, map_b_box, map_b_row;
    int st = make_map_2d(&map_a, d_A, (uint64_t)K, (uint64_t)M, BK, TILE_M,
                         p.swizzle ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    if (st) return st;
    // Boxes keep the full tile shape on every matrix: elements outside the matrix are
    // zero-filled by the copy engine and still counted in the stage's byte total.
    st = make_map_2d(&map_b_box, d_B, (uint64_t)N, (uint64_t)K, TILE_N, BK, CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (st) return st;
    st = make_map_2d(&map_b_row, d_B, (uint64_t)N, (uint64_t)K, TILE_N, 1, CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (st) return st;

    ESMM_CUDA_TRY(cudaFuncSetAttribute(esmm_joint_sgemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)L.total));
    int grid = env_int("ESMM_GRID", sms);
    if (grid > p.num_tiles) grid = p.num_tiles;
    if (grid < 1) grid = 1;
    esmm_joint_sgemm_kernel<<<grid, GEMM_THREADS, L.total, stream>>>(map_a, map_b_box, map_b_row, p);
    ESMM_CUDA_TRY(cudaGetLastError());
    return ESMM_OK;
}

}  // namespace esmm

extern "C" int esmm_gemm_ab(int M, int N, int K, const float *d_A, const float *d_B, float *d_C,
                            const uint8_t *d_a_pat, const uint8_t *d_b_pat, int a_tile_m, void *stream)
{
    return esmm::gemm_ab_launch(M, N, K, d_A, d_B, d_C, d_a_pat, d_b_pat, a_tile_m, (cudaStream_t)stream);
}
