// Joint-sparse FP32 SGEMM for sm_100a: C = A * B over the k whose joint pattern bit is set.
//
// Stands in for esmm_ab_optimized_v3 and dispatch_v3 of the reference
// (src/kernels/esmm_ab_optimized_v3.cu:18-235, include/runners.cuh:801-825) with the same
// arithmetic - one FFMA chain per output, ascending k, live k only, C overwritten - and a
// different machine mapping:
//
//   * persistent CTAs, one per SM, each walking 128 x 128 tiles of C;
//   * 8 consumer warps, each owning 64 rows x 32 columns of the tile, i.e. two A pattern
//     rows ("top" and "bottom" 32-row block) and one B pattern row; a thread holds 8 x 8
//     outputs, 4 rows in each block, so the two joint masks are applied separately and the
//     executed multiply-adds are exactly those of the reference's 32 x 32 warp tiles;
//   * lanes are laid out so that every group of 4 consecutive lanes touches 2 rows x 2
//     column chunks: on this GPU a 16-byte shared load costs 2 wavefronts when each such
//     group reads at most 32 distinct bytes and 4 otherwise;
//   * one TMA warp that streams K blocks (A box 128 rows x 8 k, 32-byte swizzled; B box
//     8 k x 128 columns, or single live k rows when few are live) into a ring of stages of
//     4 live K blocks guarded by full/empty mbarriers, and never issues a copy for a K block
//     whose joint mask is zero for the whole tile;
//   * one mask warp that, one tile ahead, joins the A and B pattern bytes of the tile into
//     a compacted list of live K blocks with per-stage 32-bit masks (one byte per K block of
//     the stage) for each 32-row and 32-column block of the tile.
//
// Every wait is bounded; a wait that expires raises the device status word and the CTA
// leaves after waiting (bounded again) for its copies in flight.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "esmm_gemm_shared.cuh"

namespace esmm {

constexpr int KB_PER_STAGE = 4;                      // live K blocks per pipeline stage
constexpr int A_SUB_BYTES = TILE_M * BK * 4;         // 4096: one K block of the A tile
constexpr int B_ROW_BYTES = TILE_N * 4;              // 512: one k row of the B tile
constexpr int B_SUB_BYTES = BK * B_ROW_BYTES;        // 4096
constexpr int STAGE_A_BYTES = KB_PER_STAGE * A_SUB_BYTES;
constexpr int STAGE_BYTES = KB_PER_STAGE * (A_SUB_BYTES + B_SUB_BYTES);  // 32768
constexpr int CONSUMER_WARPS = 8;
constexpr int TMA_WARP = CONSUMER_WARPS;
constexpr int MASK_WARP = CONSUMER_WARPS + 1;
constexpr int GEMM_THREADS = (CONSUMER_WARPS + 2) * 32;  // 320
constexpr int MAX_STAGES = 6;
constexpr int MASK_STAGE_BYTES = 32;                 // 4 A words + 4 B words per stage
#ifndef ESMM_DENSE_UNROLL
#define ESMM_DENSE_UNROLL 1
#endif
constexpr int DENSE_UNROLL = ESMM_DENSE_UNROLL;      // K blocks of a dense stage unrolled together

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
    L.cmask_off = o;  // two buffers; per stage of 4 live K blocks: A words [4], B words [4]
    L.cmask_stride = (uint32_t)(nKBpad / KB_PER_STAGE) * MASK_STAGE_BYTES;
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

// Four consecutive k of one K block, live for both 32-row blocks of the warp: each of the
// thread's 8 rows comes in as one 16-byte load (4 k), each k of B as two.
__device__ __forceinline__ void dense_nibble(float (&acc)[8][8], const char *ap, const char *bp)
{
    float a[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 v = *reinterpret_cast<const float4 *>(ap + i * 256);
        a[i][0] = v.x;
        a[i][1] = v.y;
        a[i][2] = v.z;
        a[i][3] = v.w;
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
        const float4 b0 = *reinterpret_cast<const float4 *>(bp + kk * B_ROW_BYTES);
        const float4 b1 = *reinterpret_cast<const float4 *>(bp + kk * B_ROW_BYTES + 64);
#pragma unroll
        for (int i = 0; i < 8; ++i) fma8(acc[i], a[i][kk], b0, b1);
    }
}

// The live k of one nibble, one at a time, ascending; `tn` / `bn` are the nibble's joint bits
// for the warp's top / bottom 32-row block.
__device__ __forceinline__ void sparse_nibble(float (&acc)[8][8], const char *ap, const char *bp,
                                              unsigned tn, unsigned bn)
{
    unsigned u = tn | bn;
#pragma unroll 1
    while (u) {
        const int kk = __ffs(u) - 1;
        u &= u - 1;
        const float4 b0 = *reinterpret_cast<const float4 *>(bp + kk * B_ROW_BYTES);
        const float4 b1 = *reinterpret_cast<const float4 *>(bp + kk * B_ROW_BYTES + 64);
        const char *akp = ap + kk * 4;
        float a[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = *reinterpret_cast<const float *>(akp + i * 256);
        if ((tn >> kk) & 1u) {
#pragma unroll
            for (int i = 0; i < 4; ++i) fma8(acc[i], a[i], b0, b1);
        }
        if ((bn >> kk) & 1u) {
#pragma unroll
            for (int i = 4; i < 8; ++i) fma8(acc[i], a[i], b0, b1);
        }
    }
}

// A stage whose 32 k are all live for both row blocks: straight-line code, so that the
// compiler can issue the loads of a nibble under the multiply-adds of the one before.
__device__ __forceinline__ void dense_stage(float (&acc)[8][8], const char *sA, const char *sB, int swoff)
{
    const char *ap0 = sA + swoff;         // k 0..3 of each K block
    const char *ap1 = sA + (16 ^ swoff);  // k 4..7
#pragma unroll DENSE_UNROLL
    for (int j = 0; j < KB_PER_STAGE; ++j) {
        dense_nibble(acc, ap0 + j * A_SUB_BYTES, sB + j * B_SUB_BYTES);
        dense_nibble(acc, ap1 + j * A_SUB_BYTES, sB + j * B_SUB_BYTES + 4 * B_ROW_BYTES);
    }
}

// A stage without any fully live nibble: its live k (bits of jt | jb, bit = 8 * K block + k)
// are taken four at a time, ascending; all loads of a batch are issued before its
// multiply-adds so that their latency overlaps.
__device__ __forceinline__ void sparse_stage(float (&acc)[8][8], const char *sA, const char *sB, int swoff,
                                             unsigned jt, unsigned jb)
{
    unsigned u = jt | jb;
#pragma unroll 1
    while (u) {
        int bi[4];
        bool valid[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            valid[j] = u != 0;
            bi[j] = valid[j] ? __ffs(u) - 1 : bi[0];
            u &= u - 1;
        }
        float a[4][8];
        float4 b0[4], b1[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int b = bi[j];
            const char *ap = sA + ((b >> 3) << 12) + ((((b >> 2) & 1) << 4) ^ swoff) + ((b & 3) << 2);
            const char *bp = sB + (b << 9);
            b0[j] = *reinterpret_cast<const float4 *>(bp);
            b1[j] = *reinterpret_cast<const float4 *>(bp + 64);
#pragma unroll
            for (int i = 0; i < 8; ++i) a[j][i] = *reinterpret_cast<const float *>(ap + i * 256);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (valid[j]) {
                if ((jt >> bi[j]) & 1u) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) fma8(acc[i], a[j][i], b0[j], b1[j]);
                }
                if ((jb >> bi[j]) & 1u) {
#pragma unroll
                    for (int i = 4; i < 8; ++i) fma8(acc[i], a[j][i], b0[j], b1[j]);
                }
            }
        }
    }
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
            uint8_t *cmask = reinterpret_cast<uint8_t *>(smem + L.cmask_off + buf * L.cmask_stride);
            uint16_t *klist = reinterpret_cast<uint16_t *>(smem + L.klist_off + buf * L.klist_stride);
            int base = 0;
            for (int kb0 = 0; kb0 < p.nKB; kb0 += 32) {
                const int kb = kb0 + lane;
                unsigned aw = 0, bw = 0;  // byte i: pattern of the tile's i-th 32-row / 32-column block
                if (kb < p.nKB) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int mb = tm * 4 + i;
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
                    uint8_t *m = cmask + (pos >> 2) * MASK_STAGE_BYTES + (pos & 3);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        m[4 * i] = (uint8_t)(aw >> (8 * i));
                        m[16 + 4 * i] = (uint8_t)(bw >> (8 * i));
                    }
                    if (bounds_ok(pos < p.nKBpad, p.status, 40)) klist[pos] = (uint16_t)kb;   // checked build: site 40
                }
                base += __popc(bal);
            }
            // zero the tail of the last stage so that its unused K-block slots read as dead
            if (lane < 4) {
                const int pos = base + lane;
                if (pos < ((base + 3) & ~3)) {
                    uint8_t *m = cmask + (pos >> 2) * MASK_STAGE_BYTES + (pos & 3);
#pragma unroll
                    for (int i = 0; i < 8; ++i) m[4 * i] = 0;
                    if (bounds_ok(pos < p.nKBpad, p.status, 40)) klist[pos] = 0;
                }
            }
            if (lane == 0) nlive[buf] = base;
            __syncwarp();
            if (lane == 0) mbar_arrive(mfull0 + 8 * buf);
        }
    } else if (warp == TMA_WARP) {
        // ---------------- TMA warp: stream live K blocks into the ring ----------------
        // All 32 lanes work: lane = 8 * j + kk looks after k row kk of the stage's j-th K block,
        // so the copies of a stage go out in one or two warp instructions instead of a long
        // single-thread sequence.
        if (lane == 0) {
            tma_prefetch_descriptor(&map_a);
            tma_prefetch_descriptor(&map_b_box);
            tma_prefetch_descriptor(&map_b_row);
        }
        const int j = lane >> 3, kk = lane & 7;
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
            const uint4 *cmask = reinterpret_cast<const uint4 *>(smem + L.cmask_off + buf * L.cmask_stride);
            const uint16_t *klist = reinterpret_cast<const uint16_t *>(smem + L.klist_off + buf * L.klist_stride);
            const int n = nlive[buf];
            for (int i0 = 0; i0 < n; i0 += KB_PER_STAGE) {
                const uint4 ma = cmask[(i0 >> 2) * 2], mb = cmask[(i0 >> 2) * 2 + 1];
                // byte j: live k of the stage's j-th K block for the tile as a whole
                const unsigned live = (ma.x | ma.y | ma.z | ma.w) & (mb.x | mb.y | mb.z | mb.w);
                const bool valid = i0 + j < n;
                const unsigned mj = (live >> (8 * j)) & 0xFFu;
                const bool by_row = __popc(mj) <= p.brow_bits;
                const bool my_row = valid && by_row && ((mj >> kk) & 1u);
                const bool my_box = valid && !by_row && kk == 0;
                const int k0 = valid ? (int)klist[i0 + j] * BK : 0;
                uint32_t my_bytes = (my_row ? B_ROW_BYTES : 0) + (my_box ? B_SUB_BYTES : 0);
                if (valid && kk == 0) my_bytes += A_SUB_BYTES;
                const uint32_t bytes = __reduce_add_sync(0xFFFFFFFFu, my_bytes);
                ok = mbar_wait(empty0 + 8 * slot, phase ^ 1, abort_flag);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                const uint32_t full = full0 + 8 * slot;
                if (lane == 0) mbar_arrive_expect_tx(full, bytes);
                __syncwarp();
                const uint32_t sa = smem_u32(smem + L.stage_off) + (uint32_t)slot * STAGE_BYTES + j * A_SUB_BYTES;
                const uint32_t sb = sa + STAGE_A_BYTES;
                if (valid && kk == 0) tma_load_2d(sa, &map_a, k0, tm * TILE_M, full);
                if (my_row) tma_load_2d(sb + kk * B_ROW_BYTES, &map_b_row, tn * TILE_N, k0 + kk, full);
                if (my_box) tma_load_2d(sb, &map_b_box, tn * TILE_N, k0, full);
                issued_bits |= 1u << slot;
                parity_bits = (parity_bits & ~(1u << slot)) | (phase << slot);
                if (++slot == p.stages) {
                    slot = 0;
                    phase ^= 1;
                }
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(mempty0 + 8 * buf);
        }
        if (!ok && lane == 0) {
            // leave only after the copies already issued have landed (bounded)
            for (int s = 0; s < p.stages; ++s) {
                if (!(issued_bits & (1u << s))) continue;
                const uint32_t par = (parity_bits >> s) & 1u;
                for (int tries = 0; tries < (1 << 16); ++tries)
                    if (mbar_try_wait(full0 + 8 * s, par)) break;
            }
        }
    } else {
        // ---------------- consumer warps: 64 rows x 32 columns of the tile each ----------------
        const int wm = warp >> 2, wn = warp & 3;              // 2 x 4 warps
        const int lm = (lane >> 1) & 7;                       // row (group) within the warp's 32-row blocks
        const int ln = (lane & 1) | ((lane >> 4) << 1);       // 16-byte column chunk
        const int swoff = p.swizzle ? ((lm >> 2) & 1) << 4 : 0;
        // the thread owns rows lm + 8 i of the warp's 64; a row of an A sub-slot is 32 bytes
        const uint32_t a_thr = (uint32_t)(wm * 64 + lm) * 32;
        const uint32_t b_thr = STAGE_A_BYTES + (uint32_t)(wn * 32 + ln * 4) * 4;  // column offset in a B sub-slot
        int slot = 0;
        uint32_t phase = 0;
        int it = 0;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            ok = mbar_wait(mfull0 + 8 * buf, (it >> 1) & 1, abort_flag);
            if (!ok) break;
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            const char *cmask = smem + L.cmask_off + buf * L.cmask_stride;
            const int n = nlive[buf];

            float acc[8][8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

            for (int i0 = 0; i0 < n; i0 += KB_PER_STAGE) {
                const char *ms = cmask + (i0 >> 2) * MASK_STAGE_BYTES;
                const uint2 am = *reinterpret_cast<const uint2 *>(ms + 8 * wm);   // top, bottom 32-row block
                const unsigned bm = *reinterpret_cast<const unsigned *>(ms + 16 + 4 * wn);
                const unsigned jt = am.x & bm, jb = am.y & bm;   // byte j: joint mask of the stage's j-th K block
                ok = mbar_wait(full0 + 8 * slot, phase, abort_flag);
                if (!ok) break;
                const char *sA = smem + L.stage_off + (size_t)slot * STAGE_BYTES + a_thr;
                const char *sB = smem + L.stage_off + (size_t)slot * STAGE_BYTES + b_thr;
                const unsigned both = jt & jb;
                unsigned dn = both & (both >> 1);   // bit 4n: nibble n is live for both row blocks
                dn &= dn >> 2;
                dn &= 0x11111111u;
                if (dn == 0x11111111u) {
                    dense_stage(acc, sA, sB, swoff);
                } else if (dn == 0u) {
                    sparse_stage(acc, sA, sB, swoff, jt, jb);
                } else {
                    // mixed: nibble by nibble, skipping the dead ones
                    unsigned z = jt | jb;
                    z |= z >> 1;
                    z |= z >> 2;
                    z &= 0x11111111u;
#pragma unroll 1
                    while (z) {
                        const int nb = (__ffs(z) - 1) >> 2;   // K block nb >> 1, half nb & 1
                        z &= z - 1;
                        const unsigned tnib = (jt >> (4 * nb)) & 0xFu, bnib = (jb >> (4 * nb)) & 0xFu;
                        const char *ap = sA + (nb >> 1) * A_SUB_BYTES + (((nb & 1) << 4) ^ swoff);
                        const char *bp = sB + nb * (4 * B_ROW_BYTES);
                        if ((tnib & bnib) == 0xFu) dense_nibble(acc, ap, bp);
                        else sparse_nibble(acc, ap, bp, tnib, bnib);
                    }
                }
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
            const int row0 = tm * TILE_M + wm * 64 + lm;
            const int col0 = tn * TILE_N + wn * 32 + ln * 4;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int row = row0 + 8 * i;
                if (row < p.M) {
                    float *c = p.C + (size_t)row * p.N + col0;
                    const size_t c_floats = (size_t)p.M * p.N, off = (size_t)row * p.N + col0;   // checked build: site 41
                    if (col0 < p.N && bounds_ok(off + 4 <= c_floats, p.status, 41))
                        *reinterpret_cast<float4 *>(c) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
                    if (col0 + 16 < p.N && bounds_ok(off + 20 <= c_floats, p.status, 41))
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
    p.swizzle = tuning_get("SWIZZLE", 1) ? 1 : 0;
    p.brow_bits = tuning_get("BROW_BITS", 2);
    if (p.brow_bits < 0) p.brow_bits = 0;
    if (p.brow_bits > 8) p.brow_bits = 8;
    p.a_pat = d_a_pat;
    p.b_pat = d_b_pat;
    p.C = d_C;
    if (p.nKB > 65535) return ESMM_ERR_TOO_LARGE;

    int stages = tuning_get("STAGES", MAX_STAGES);
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

    // Boxes keep the full tile shape on every matrix: elements outside the matrix are
    // zero-filled by the copy engine and still counted in the stage's byte total.
    CUtensorMap map_a, map_b_box, map_b_row;
    int st = make_map_2d(&map_a, d_A, (uint64_t)K, (uint64_t)M, BK, TILE_M,
                         p.swizzle ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    if (st) return st;
    st = make_map_2d(&map_b_box, d_B, (uint64_t)N, (uint64_t)K, TILE_N, BK, CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (st) return st;
    st = make_map_2d(&map_b_row, d_B, (uint64_t)N, (uint64_t)K, TILE_N, 1, CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (st) return st;

    ESMM_CUDA_TRY(cudaFuncSetAttribute(esmm_joint_sgemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)L.total));
    int grid = tuning_get("GRID", sms);
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
