// Joint-sparse FP32 SGEMM for sm_100a on the packed (k-major) copy of A.
//
// Same arithmetic as esmm_ab_optimized_v3 of the reference
// (src/kernels/esmm_ab_optimized_v3.cu:18-235): for every output one FFMA chain in ascending
// k over the k whose joint bit (A pattern of its 32-row block AND B pattern of its 32-column
// block) is set; C is overwritten.  What differs is where the skipping happens.
//
// A comes from the packing preprocessor as [128-row tile][k][128 rows]; B is the caller's
// row-major matrix, i.e. [k][N].  So one k of a 128 x 128 tile of C needs one 512-byte row
// of each operand, and the pipeline moves exactly such rows:
//
//   * a mask warp walks the tile's K blocks one tile ahead and appends, for every K block,
//     the k rows that are live for the tile as a whole (the OR over its four 32-row blocks
//     AND the OR over its four 32-column blocks) to a row list, with one byte per row saying
//     for which row blocks and which column blocks the row is live.  On a tile whose K
//     blocks do not all share one live byte, K blocks with more than `brow_bits` live k are
//     appended whole (8 rows), so that they can be fetched as one box;
//   * three producer warps cut the row list into stages of 32 rows and fetch each stage's rows into
//     a ring slot ([32][512 B] of A, [32][512 B] of B), guarded by full / empty mbarriers.
//     Both operands are also described to the copy engine as 3-D tensors (column, k % 8,
//     k / 8), so a stage whose rows are "the same c consecutive k offsets of 32 / c
//     consecutive K blocks" (c = 1, 2, 4, 8: what uniform patterns such as 10000000,
//     11000000, 11110000 and 11111111 produce) is ONE box per operand, landing in ascending
//     k.  Other stages: the list is ascending, and rows with consecutive k are consecutive rows
//     of both operands, so every run of them goes as boxes of 8, 4, 2 and 1 rows, issued by the
//     lane at the box's first row, the boxes of a stage shared out among the producer warps (a
//     copy costs its warp about 50 cycles of issue, and warps issue in parallel).  A k that is
//     dead for the whole tile costs neither a copy nor shared memory nor a slot in any loop;
//   * a tile all of whose K blocks hold the same run of 1, 2, 4 or 8 consecutive live k, live for all
//     of its row and column blocks (what uniform patterns, and dense inputs, give), needs no row
//     list at all: its stages are computed arithmetically and are all-live;
//   * where 128 x 128 tiles would leave most of the GPU idle (small M x N), the same kernel runs
//     with 64 x 128 tiles: a 64-row tile reads the left or right half of a 128-row panel of A, a
//     consumer warp owns 32 x 32 outputs;
//   * 8 consumer warps own 64 rows x 32 columns of the tile each (two A pattern rows, one B
//     pattern row; a thread holds 8 x 8 outputs, 4 rows in each 32-row block).  Per stage a
//     warp forms its two 32-bit joint masks with two ballots.  If every row of the stage is
//     live for both row blocks - always the case for uniform patterns, at any density - it
//     runs straight-line code (4 sixteen-byte loads and 32 two-wide FMAs per k).  Otherwise it
//     walks the set bits of its masks, loading the next live row under the multiply-adds of
//     the current one.
//
// Lanes are laid out so that every group of 4 consecutive lanes touches 2 row chunks x 2
// column chunks: on this GPU a 16-byte shared load costs 2 wavefronts when each such group
// reads at most 32 distinct bytes and 4 otherwise.
//
// Every wait is bounded; a wait that expires raises the device status word and the CTA
// leaves after waiting (bounded again) for its copies in flight.
#include <atomic>
#include <cstring>
#include <mutex>

#include "esmm_gemm_shared.cuh"

namespace esmm {

constexpr int ROW_BYTES = TILE_N * 4;            // 512: one k of an operand tile
constexpr int ROWS_PER_STAGE = 32;
constexpr int STAGE_HALF_BYTES = ROWS_PER_STAGE * ROW_BYTES;   // 16384: A rows, then B rows
constexpr int PSTAGE_BYTES = 2 * STAGE_HALF_BYTES;             // 32768
constexpr int P_CONSUMER_WARPS = 8;
// Issuing a copy costs the issuing warp about 50 cycles per copy, whatever the mechanism (2-D tensor copy of one row
// or of an 8-row box, untiled bulk copy, or a warp-wide 16-byte cp.async per row: 3300 cycles for the 64 copies of a
// row-by-row stage from one warp, 1270 from three, 970 from four - measured), and different warps issue in parallel.
// So the rows of a stage are shared out among several producer warps.
//   3 producer warps: 8 consumer + 3 producer + 1 mask warp = 12 warps, 3 per SM sub-partition, every thread with
//     the 168 registers a 384-thread CTA allows (the consumers need about 150).
//   7 producer warps: 16 warps.  A 512-thread CTA starts with 128 registers per thread; the two warp groups of
//     consumers raise their allowance to 160 and the two warp groups of producers / mask warp lower theirs to 96
//     (setmaxnreg).  Each CTA's first tile decides whether all 7 copy (tiles of scattered single rows with little
//     work per consumer warp: a stage is then posted every 0.92 us instead of 1.19) or 3 do and 4 sleep.  Measured
//     at 4096^3 against the 12-warp form: independent 32-granular patterns at 0.2 / 0.2 0.369 -> 0.322 ms, but
//     dense and uniform patterns 0.5 % slower.  A launch takes this form when the launch before it on the device
//     noted such tiles (see gemm_ab_packed_launch_form); esmm_tuning_set("PRODUCER_WARPS", 3 | 7 | 0) pins one.
constexpr int P_TMA_WARP = P_CONSUMER_WARPS;                   // first producer warp
constexpr int P_MAX_STAGES = 6;

// Optional timeline for tuning (build with -DESMM_TRACE): CTA 0 stamps %globaltimer at a few points
// into a device array that esmm_trace_read copies out.  Not part of the product build or of the ABI.
#ifdef ESMM_TRACE
__device__ unsigned long long g_esmm_trace[1024];
#define ESMM_STAMP(idx)                                                                   \
    do {                                                                                  \
        if (blockIdx.x == 0 && lane == 0 && (idx) < 1024) g_esmm_trace[(idx)] = global_timer_ns(); \
    } while (0)
#else
#define ESMM_STAMP(idx) \
    do {                \
    } while (0)
#endif

struct PackedParams {
    int M, N, K;
    int nKB;         // ceil(K / 8)
    int kp;          // rows of the packed A matrix per 128-row tile (nKB * 8)
    int cap;         // capacity of a tile's row list (multiple of 32)
    int a_rows;      // rows of the A pattern array (ceil(M / 32))
    int b_rows;      // rows of the B pattern array (ceil(N / 32))
    int tiles_m, tiles_n, num_tiles;
    int group_m;     // tile rows per raster group
    int stages;
    int brow_bits;   // K blocks with more live k than this are fetched whole
    int row_density; // ... on tiles with at most this many live k per K block on average; denser tiles
                     // fetch every live K block whole
    int b_runs_ok;   // K % 8 == 0: the 3-D view of B stays inside the matrix
    int force_listed;  // tuning aid: take the index-list path even for all-live stages
    int no_run_tiles;  // tuning aid: build the row list even for tiles that need none
    int vec_patterns;  // K blocks per lane and load in the mask warp: 16, 4 (alignment permitting) or 0 = bytes
    int adaptive;      // 16-warp form: the CTA's first tile decides whether 3 or all 7 producer warps copy
    int *form_hint;    // host-mapped word, or null: CTA 0 notes whether its first tile wanted 7 producers
    const uint8_t *a_pat;
    const uint8_t *b_pat;
    float *C;
    int *status;
};

// Tensor maps of one launch.  *_box[i]: 2-D, 1 << i rows (1, 2, 4, 8) of 128 columns.  *_run[i]: 3-D
// (column, k % 8, k / 8) boxes of 128 x c x 32/c with c = 1 << i.
struct PackedMaps {
    CUtensorMap a_box[4], a_run[4];
    CUtensorMap b_box[4], b_run[4];
};

constexpr int RUN_TILE = 0x100;
constexpr int RUNS_LIKELY = 0x200;   // a listed tile whose stages may be whole runs of K blocks: the producers look for them

struct PackedSmem {
    uint32_t stage_off, krow_off, krow_stride, rmask_off, rmask_stride, wlist_off, bar_off, misc_off, total;
};

__host__ __device__ inline PackedSmem packed_smem_layout(int stages, int cap)
{
    PackedSmem L;
    uint32_t o = 0;
    L.stage_off = o;
    o += (uint32_t)stages * PSTAGE_BYTES;
    L.krow_off = o;   // two buffers: k index of every listed row
    L.krow_stride = (uint32_t)cap * 2;
    o += 2 * L.krow_stride;
    L.rmask_off = o;  // two buffers: per row, bits 0-3 live row blocks, bits 4-7 live column blocks
    L.rmask_stride = (uint32_t)cap;
    o += 2 * L.rmask_stride;
    o = (o + 15u) & ~15u;
    L.wlist_off = o;  // per consumer warp: offsets of the live rows of its top and its bottom block
    o += P_CONSUMER_WARPS * 2 * 96;  // two lists of WLIST_BYTES per warp
    L.bar_off = o;    // full[P_MAX_STAGES], empty[P_MAX_STAGES], list_full[2], list_empty[2]
    o += (2 * P_MAX_STAGES + 4) * 8;
    L.misc_off = o;   // nrows[2], abort, n_producers, runinfo[2]
    o += 32;
    L.total = o;
    return L;
}

// One k of the tile for one thread: its 4 rows of the top block, 4 rows of the bottom block
// and 2 x 4 columns are one 16-byte load each.
struct KFrag {
    float4 at, ab, b0, b1;
};

// WMB = 32-row blocks per consumer warp: 2 in the 128 x 128 tiling, 1 in the 64 x 128 tiling (where a
// thread holds 4 x 8 outputs and the "bottom" half of everything below is compiled out).
template <int WMB>
__device__ __forceinline__ KFrag load_kfrag(const char *pa, const char *pb)
{
    KFrag f;
    f.at = *reinterpret_cast<const float4 *>(pa);
    if (WMB == 2) f.ab = *reinterpret_cast<const float4 *>(pa + 128);
    f.b0 = *reinterpret_cast<const float4 *>(pb);
    f.b1 = *reinterpret_cast<const float4 *>(pb + 64);
    return f;
}

// The thread's 8 x 8 outputs are held as 2 x 2 blocks for the packed FP32 multiply-add of sm_100
// (fma.rn.f32x2: two independent IEEE FMAs per instruction, half the issue slots of scalar FFMA).
// Block (p, q) covers rows 2p, 2p+1 and columns 2q, 2q+1 of the thread tile:
//   diag[p][q] = (c[2p][2q],   c[2p+1][2q+1])        anti[p][q] = (c[2p][2q+1], c[2p+1][2q])
// so both use the row pair (a[2p], a[2p+1]) as it comes from shared memory, with the column pair
// (b[2q], b[2q+1]) as loaded for diag and swapped for anti.  Row pairs 0, 1 are the top 32-row
// block, 2, 3 the bottom one.  Every output still sees one FMA per live k, in ascending k.
struct Acc {
    float2 diag[4][4], anti[4][4];
};

// One 2 x 2 block: the diagonal pair and the anti-diagonal pair, one two-wide FMA each (the second on the swapped column
// pair).  (The anti-diagonal pair as two scalar FMAs instead - no swapped operands, 48 instead of 32 multiply-add
// instructions per row - was measured 23 % slower on the dense path.)
__device__ __forceinline__ void fma_block(float2 &diag, float2 &anti, float2 ar, float bx, float by)
{
    diag = __ffma2_rn(ar, make_float2(bx, by), diag);
    anti = __ffma2_rn(ar, make_float2(by, bx), anti);
}

__device__ __forceinline__ void fma_pair_row(Acc &c, int p, float2 ar, const KFrag &f)
{
    fma_block(c.diag[p][0], c.anti[p][0], ar, f.b0.x, f.b0.y);
    fma_block(c.diag[p][1], c.anti[p][1], ar, f.b0.z, f.b0.w);
    fma_block(c.diag[p][2], c.anti[p][2], ar, f.b1.x, f.b1.y);
    fma_block(c.diag[p][3], c.anti[p][3], ar, f.b1.z, f.b1.w);
}

__device__ __forceinline__ void fma_top(Acc &c, const KFrag &f)
{
    fma_pair_row(c, 0, make_float2(f.at.x, f.at.y), f);
    fma_pair_row(c, 1, make_float2(f.at.z, f.at.w), f);
}

__device__ __forceinline__ void fma_bottom(Acc &c, const KFrag &f)
{
    fma_pair_row(c, 2, make_float2(f.ab.x, f.ab.y), f);
    fma_pair_row(c, 3, make_float2(f.ab.z, f.ab.w), f);
}

// A stage whose 32 rows are all live for both row blocks: 16 rows of straight-line code per
// loop trip (measured: 4 rows 1 % slower than 8, 16 rows 1.6 % faster, 32 no better than 16),
// so that the compiler can issue the loads of a row under the multiply-adds of the row before.
template <int WMB>
__device__ __forceinline__ void dense_rows(Acc &acc, const char *sA, const char *sB)
{
    constexpr int A_ROW = 256 * WMB;   // bytes of one k of the A tile
    // (Measured and dropped: a rolling prefetch across the loop's back edge; a non-blocking look at the next stage's
    // barrier under the last multiply-adds of this one, so that the wait at the stage change is skipped - no gain.)
#ifndef ESMM_DENSE_UNROLL
#define ESMM_DENSE_UNROLL 16
#endif
#pragma unroll 1
    for (int r0 = 0; r0 < ROWS_PER_STAGE; r0 += ESMM_DENSE_UNROLL) {
#pragma unroll
        for (int r = 0; r < ESMM_DENSE_UNROLL; ++r) {
            const KFrag f = load_kfrag<WMB>(sA + (r0 + r) * A_ROW, sB + (r0 + r) * ROW_BYTES);
            fma_top(acc, f);
            if (WMB == 2) fma_bottom(acc, f);
        }
    }
}

// ---- stages that are not all-live ------------------------------------------------------------------
// When the warp's two 32-row blocks have the same live rows (jt == jb) every live row goes into all
// 8 x 8 outputs (mode BOTH): the set bits of the mask, a warp-uniform value, are walked in ascending
// order with find-first-set, one row loaded ahead under the 32 two-wide FMAs of the row before.
// Otherwise the top and the bottom block are processed one after the other (modes TOP, BOTTOM): each
// accumulator still sees its own live k in ascending order, no multiply-add is predicated, and the
// only price is that B rows live for both blocks are read from shared memory twice.  A row then
// feeds only 16 two-wide FMAs, too few to hide a find-first-set chain and a load behind: the lanes
// first write the rows' offsets as a list (in parallel, while the stage may still be in flight) and
// the loop takes two rows per step from it.  (Measured on random 32-granular patterns: one pass over
// jt | jb with warp-uniform branches per block is 20 % slower than the two passes, bit walking in
// the half modes 3-5 % slower than lists, lists in mode BOTH 4 % slower than bit walking, a switch
// per nibble of the mask into straight-line code 38 % slower.  For masks made of bytes 0x00 / 0xFF
// (block-pruned operands) a walk in groups of 8 rows with one three-way choice per group gained nothing
// on a pruned-MLP shape - there the spread of live rows between the 8 warps of a stage is what costs -
// and made the other paths 1-5 % slower; preparing masks and lists one stage ahead (two list buffers)
// was 2-5 % slower on every workload.)
enum { MODE_BOTH = 0, MODE_TOP = 1, MODE_BOTTOM = 2 };

template <int MODE, int WMB>
__device__ __forceinline__ KFrag load_entry(const char *sA, const char *sB, unsigned off)
{
    KFrag f;
    const unsigned a_off = WMB == 2 ? off : off >> 1;   // A rows are 512 or 256 bytes apart
    if (MODE != MODE_BOTTOM) f.at = *reinterpret_cast<const float4 *>(sA + a_off);
    if (MODE != MODE_TOP) f.ab = *reinterpret_cast<const float4 *>(sA + a_off + 128);
    f.b0 = *reinterpret_cast<const float4 *>(sB + off);
    f.b1 = *reinterpret_cast<const float4 *>(sB + off + 64);
    return f;
}

template <int MODE>
__device__ __forceinline__ void fma_entry(Acc &acc, const KFrag &f)
{
    if (MODE != MODE_BOTTOM) fma_top(acc, f);
    if (MODE != MODE_TOP) fma_bottom(acc, f);
}

// byte offset in the stage's B rows of the lowest live row of m, which is removed from m
__device__ __forceinline__ unsigned pop_row(unsigned &m)
{
    const unsigned r = (unsigned)__ffs((int)m) - 1u;
    m &= m - 1u;
    return r << 9;
}

// (128-row tiling only: in the 64-row tiling every stage that is not all-live takes the list.)
__device__ __forceinline__ void masked_rows_both(Acc &acc, const char *sA, const char *sB, unsigned m)
{
    if (m == 0u) return;
    KFrag f0 = load_entry<MODE_BOTH, 2>(sA, sB, pop_row(m)), f1;
#pragma unroll 1
    while (true) {
        if (m == 0u) {
            fma_entry<MODE_BOTH>(acc, f0);
            break;
        }
        f1 = load_entry<MODE_BOTH, 2>(sA, sB, pop_row(m));
        fma_entry<MODE_BOTH>(acc, f0);
        if (m == 0u) {
            fma_entry<MODE_BOTH>(acc, f1);
            break;
        }
        f0 = load_entry<MODE_BOTH, 2>(sA, sB, pop_row(m));
        fma_entry<MODE_BOTH>(acc, f1);
    }
}

// A list holds, ascending, the byte offset in the stage (row * 512, 16 bits) of every row that is
// live for one of the warp's blocks, padded with 8 zero entries so that look-ahead loads need no
// bounds checks.
constexpr int WLIST_ENTRIES = ROWS_PER_STAGE + 8;
constexpr int WLIST_BYTES = 96;   // WLIST_ENTRIES * 2, rounded up to a multiple of 16
static_assert(WLIST_ENTRIES * 2 <= WLIST_BYTES, "per-warp list does not fit");

__device__ __forceinline__ unsigned entry_of(const uint2 &w, int j)
{
    const unsigned word = (j & 2) ? w.y : w.x;
    return (j & 1) ? (word >> 16) : (word & 0xFFFFu);
}

// Two rows per step, the next pair loaded before the current pair is multiplied.
template <int MODE, int WMB>
__device__ __forceinline__ void listed_rows(Acc &acc, const char *sA, const char *sB, const uint16_t *list, int cnt)
{
    const int n4 = cnt & ~3;
    uint2 ew = *reinterpret_cast<const uint2 *>(list);   // entries 0..3
    KFrag f0 = load_entry<MODE, WMB>(sA, sB, entry_of(ew, 0));
    KFrag f1 = load_entry<MODE, WMB>(sA, sB, entry_of(ew, 1));
#pragma unroll 1
    for (int i = 0; i < n4; i += 4) {
        const KFrag g0 = load_entry<MODE, WMB>(sA, sB, entry_of(ew, 2));
        const KFrag g1 = load_entry<MODE, WMB>(sA, sB, entry_of(ew, 3));
        fma_entry<MODE>(acc, f0);
        fma_entry<MODE>(acc, f1);
        ew = *reinterpret_cast<const uint2 *>(list + i + 4);   // padded: always readable
        f0 = load_entry<MODE, WMB>(sA, sB, entry_of(ew, 0));
        f1 = load_entry<MODE, WMB>(sA, sB, entry_of(ew, 1));
        fma_entry<MODE>(acc, g0);
        fma_entry<MODE>(acc, g1);
    }
    // up to three rows are left; f0, f1 already hold the first two of them (or padding)
    const int rem = cnt - n4;
    if (rem >= 1) fma_entry<MODE>(acc, f0);
    if (rem >= 2) fma_entry<MODE>(acc, f1);
    if (rem == 3) fma_entry<MODE>(acc, load_entry<MODE, WMB>(sA, sB, entry_of(ew, 2)));
}

// Lanes write the list of the rows whose bit is set in `m`; returns the count.
__device__ __forceinline__ int build_list(uint16_t *list, unsigned m, int lane, int *status)
{
    const int cnt = __popc(m);
    const int mine = __popc(m & ((1u << lane) - 1u));
    if (((m >> lane) & 1u) && bounds_ok(mine < WLIST_ENTRIES, status, 25)) list[mine] = (uint16_t)(lane << 9);
    if (lane < 8 && bounds_ok(cnt + lane < WLIST_ENTRIES, status, 25)) list[cnt + lane] = 0;
    return cnt;
}

// ---- mask warp helpers ---------------------------------------------------------------------------
// Pattern bytes of KPL (16 or 4) consecutive K blocks kb0 .. kb0 + KPL - 1, all inside the matrix, for the
// tile's RB 32-row blocks and four 32-column blocks: one 16-byte or 4-byte load per pattern row.  aw[j] /
// bw[j] get the four bytes of K block kb0 + j (byte i = block i).  Long K takes 16 per lane; shorter K
// takes 4, so that all lanes have work.
template <int RB, int KPL>
__device__ __forceinline__ void load_patterns(const PackedParams &p, int tm, int tn, int kb0, bool valid,
                                              unsigned (&aw)[KPL], unsigned (&bw)[KPL])
{
    constexpr int W = KPL / 4;   // 32-bit words per pattern row
    unsigned ra[4][W], rb[4][W];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int mb = tm * RB + i, nb = tn * 4 + i;
#pragma unroll
        for (int w = 0; w < W; ++w) ra[i][w] = rb[i][w] = 0u;
        if (valid && i < RB && mb < p.a_rows && bounds_ok(kb0 >= 0 && kb0 + KPL <= p.nKB, p.status, 21)) {
            const uint8_t *src = p.a_pat + (size_t)mb * p.nKB + kb0;
            if (KPL == 16) {
                const uint4 v = *reinterpret_cast<const uint4 *>(src);
                ra[i][0] = v.x, ra[i][W > 1 ? 1 : 0] = v.y, ra[i][W > 2 ? 2 : 0] = v.z, ra[i][W > 3 ? 3 : 0] = v.w;
            } else {
                ra[i][0] = *reinterpret_cast<const unsigned *>(src);
            }
        }
        if (valid && nb < p.b_rows && bounds_ok(kb0 >= 0 && kb0 + KPL <= p.nKB, p.status, 21)) {
            const uint8_t *src = p.b_pat + (size_t)nb * p.nKB + kb0;
            if (KPL == 16) {
                const uint4 v = *reinterpret_cast<const uint4 *>(src);
                rb[i][0] = v.x, rb[i][W > 1 ? 1 : 0] = v.y, rb[i][W > 2 ? 2 : 0] = v.z, rb[i][W > 3 ? 3 : 0] = v.w;
            } else {
                rb[i][0] = *reinterpret_cast<const unsigned *>(src);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < KPL; ++j) {
        const int sh = 8 * (j & 3);
        unsigned a = 0, b = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            a |= ((ra[i][j >> 2] >> sh) & 0xFFu) << (8 * i);
            b |= ((rb[i][j >> 2] >> sh) & 0xFFu) << (8 * i);
        }
        aw[j] = a;
        bw[j] = b;
    }
}

// k offsets of one K block that are live for the tile as a whole: (OR of the A bytes) & (OR of the B bytes)
__device__ __forceinline__ unsigned tile_live(unsigned aw, unsigned bw)
{
    unsigned au = aw | (aw >> 16), bu = bw | (bw >> 16);
    au = (au | (au >> 8)) & 0xFFu;
    bu = (bu | (bu >> 8)) & 0xFFu;
    return au & bu;
}

// Appends the listed rows of one K block at position q; returns the new position.
__device__ __forceinline__ int append_rows(uint16_t *krow, uint8_t *rmask, int q, int kb, unsigned rows,
                                           unsigned aw, unsigned bw, int cap, int *status)
{
    while (rows) {
        const int kk = __ffs(rows) - 1;
        rows &= rows - 1;
        const unsigned as = aw >> kk, bs = bw >> kk;
        const unsigned abits = (as & 1u) | ((as >> 7) & 2u) | ((as >> 14) & 4u) | ((as >> 21) & 8u);
        const unsigned bbits = (bs & 1u) | ((bs >> 7) & 2u) | ((bs >> 14) & 4u) | ((bs >> 21) & 8u);
        if (bounds_ok(q < cap, status, 20)) {
            krow[q] = (uint16_t)(kb * BK + kk);
            rmask[q] = (uint8_t)(abits | (bbits << 4));
        }
        ++q;
    }
    return q;
}

__device__ __forceinline__ int warp_inclusive_scan(int v, int lane)
{
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xFFFFFFFFu, v, d);
        if (lane >= d) v += t;
    }
    return v;
}

// First pass of the mask warp over a tile's pattern bytes: the live byte of its first K block, whether all
// K blocks share it, the number of live k, and how many of those lie in K blocks with at most brow_bits live k.
// whether the live k of a K block are live for each of the tile's RB row blocks and 4 column blocks
template <int RB>
__device__ __forceinline__ bool blocks_cover(unsigned aw, unsigned bw, unsigned live)
{
    const unsigned l4 = live * 0x01010101u, am = RB == 4 ? 0xFFFFFFFFu : 0x0000FFFFu;
    return ((aw & l4 & am) == (l4 & am)) && ((bw & l4) == l4);
}

template <int RB, int KPL>
__device__ __forceinline__ void tile_scan(const PackedParams &p, int tm, int tn, int lane, unsigned &live_first,
                                          bool &uniform, bool &full, int &live_total, int &live_small)
{
    for (int c0 = 0; c0 < p.nKB; c0 += 32 * KPL) {
        const int kb0 = c0 + KPL * lane;
        unsigned aw[KPL], bw[KPL];
        load_patterns<RB, KPL>(p, tm, tn, kb0, kb0 < p.nKB, aw, bw);
        if (c0 == 0) live_first = __shfl_sync(0xFFFFFFFFu, tile_live(aw[0], bw[0]), 0);
        bool same = true, cover = true;
        int cnt = 0, small = 0;
#pragma unroll
        for (int j = 0; j < KPL; ++j) {
            const unsigned live = tile_live(aw[j], bw[j]);
            same = same && live == live_first;
            cover = cover && blocks_cover<RB>(aw[j], bw[j], live);
            cnt += __popc(live);
            small += __popc(live) <= p.brow_bits ? __popc(live) : 0;
        }
        uniform = uniform && __all_sync(0xFFFFFFFFu, kb0 >= p.nKB || same);
        full = full && __all_sync(0xFFFFFFFFu, kb0 >= p.nKB || cover);
        live_total += __reduce_add_sync(0xFFFFFFFFu, cnt);
        live_small += __reduce_add_sync(0xFFFFFFFFu, small);
    }
}

// Second pass: the row list.  Lane l owns K blocks c0 + KPL l .. c0 + KPL l + KPL - 1 (consecutive lanes,
// consecutive K); K blocks with more than whole_above live k are listed whole.  Returns the row count.
template <int RB, int KPL>
__device__ __forceinline__ int tile_list(const PackedParams &p, int tm, int tn, int lane, int whole_above,
                                         uint16_t *krow, uint8_t *rmask)
{
    int pos = 0;
    for (int c0 = 0; c0 < p.nKB; c0 += 32 * KPL) {
        const int kb0 = c0 + KPL * lane;
        unsigned aw[KPL], bw[KPL];
        load_patterns<RB, KPL>(p, tm, tn, kb0, kb0 < p.nKB, aw, bw);
        unsigned rows[KPL];
        int c = 0;
#pragma unroll
        for (int j = 0; j < KPL; ++j) {
            const unsigned live = tile_live(aw[j], bw[j]);
            rows[j] = live == 0u ? 0u : (__popc(live) > whole_above ? 0xFFu : live);
            c += __popc(rows[j]);
        }
        const int incl = warp_inclusive_scan(c, lane);
        int q = pos + incl - c;
#pragma unroll
        for (int j = 0; j < KPL; ++j) q = append_rows(krow, rmask, q, kb0 + j, rows[j], aw[j], bw[j], p.cap, p.status);
        pos += __shfl_sync(0xFFFFFFFFu, incl, 31);
    }
    return pos;
}

#ifndef ESMM_CONS_REGS
#define ESMM_CONS_REGS 160
#define ESMM_PROD_REGS 96
#endif

// Sum over a tile's listed rows of the number of consumer warps (of 8) the row is live for.  (A call rather than
// inline code: it runs once per CTA, and the kernel's register allocation stays that of the code without it.)
template <int WMB>
__device__ __noinline__ int listed_warp_rows(const uint8_t *rmask, int n, int lane)
{
    int warp_rows = 0;
    for (int r = lane; r < n; r += 32) {
        const unsigned m = rmask[r], a = m & 15u, b = m >> 4;
        const int na = WMB == 2 ? ((a & 3u) != 0u) + ((a & 12u) != 0u) : __popc(a & 3u);
        warp_rows += na * __popc(b);
    }
    return __reduce_add_sync(0xFFFFFFFFu, warp_rows);
}

template <int WMB, int NPW>
__global__ void __launch_bounds__((P_CONSUMER_WARPS + NPW + 1) * 32, 1)
esmm_joint_sgemm_packed_kernel(const __grid_constant__ PackedMaps maps, const PackedParams p)
{
    static_assert(NPW == 3 || NPW == 7, "consumers, producers and the mask warp fill whole warp groups");
    constexpr int P_TMA_WARPS = NPW;
    constexpr int P_MASK_WARP = P_CONSUMER_WARPS + NPW;
    constexpr bool P_REBALANCE_REGS = NPW == 7;
    constexpr int TM_ROWS = 64 * WMB;                  // rows of a tile of C: 128 or 64
    constexpr int RB = 2 * WMB;                        // 32-row blocks per tile
    constexpr int A_ROW = TM_ROWS * 4;                 // bytes of one k of the A tile in shared memory
    constexpr uint32_t STAGE_ROW_BYTES = A_ROW + ROW_BYTES;
    extern __shared__ __align__(1024) char smem[];
    const PackedSmem L = packed_smem_layout(p.stages, p.cap);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L.bar_off);
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = smem_u32(bars + P_MAX_STAGES);
    const uint32_t lfull0 = smem_u32(bars + 2 * P_MAX_STAGES);
    const uint32_t lempty0 = smem_u32(bars + 2 * P_MAX_STAGES + 2);
    volatile int *nrows = reinterpret_cast<volatile int *>(smem + L.misc_off);
    volatile int *abort_flag = nrows + 2;
    volatile int *n_producers = nrows + 3;   // 16-warp form: producer warps that copy (set with the first tile's list)
    // per list buffer: 0, or RUN_TILE | log2(c) | kk0 << 4 for a tile whose every K block has the same c = 1, 2,
    // 4 or 8 consecutive live k (kk0 .. kk0 + c - 1), live for all of the tile's row and column blocks.  Such
    // a tile needs no row list: stage s is the 3-D box of K blocks 32 s / c .. and every stage is all-live.
    volatile int *runinfo = nrows + 4;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, P_CONSUMER_WARPS);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(lfull0 + 8 * b, 1);
            mbar_init(lempty0 + 8 * b, P_CONSUMER_WARPS + P_TMA_WARPS);
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();
    grid_dependency_wait();   // (patterns and the packed copy of A come from the kernel before this one)

    bool ok = true;
    if (warp == 0) ESMM_STAMP(0);

    // (16-warp form: registers move from the producer / mask warp groups to the consumer warp groups; 8 x 32 x 160 +
    // 8 x 32 x 96 = 65536, all the CTA starts with.  Each instruction heads its own side's code.)
    if (warp == P_MASK_WARP) {
        if (P_REBALANCE_REGS) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(ESMM_PROD_REGS));
        // ---------------- mask warp: the tile's list of live k rows ----------------
        int it = 0;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            ok = mbar_wait(lempty0 + 8 * buf, ((it >> 1) & 1) ^ 1, abort_flag);
            if (!ok) break;
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn, p.group_m);
            uint16_t *krow = reinterpret_cast<uint16_t *>(smem + L.krow_off + buf * L.krow_stride);
            uint8_t *rmask = reinterpret_cast<uint8_t *>(smem + L.rmask_off + buf * L.rmask_stride);
            // A first pass over the tile's pattern bytes decides the listing policy.
            unsigned live_first = 0;
            bool uniform = true, full = true;
            int live_total = 0, live_small = 0;
            if (p.vec_patterns == 16) {
                tile_scan<RB, 16>(p, tm, tn, lane, live_first, uniform, full, live_total, live_small);
            } else if (p.vec_patterns == 4) {
                tile_scan<RB, 4>(p, tm, tn, lane, live_first, uniform, full, live_total, live_small);
            } else {
                for (int kb0 = 0; kb0 < p.nKB; kb0 += 32) {
                    const int kb = kb0 + lane;
                    unsigned au = 0, bu = 0;
                    if (kb < p.nKB) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int mb = tm * RB + i, nb = tn * 4 + i;
                            if (i < RB && mb < p.a_rows) au |= p.a_pat[(size_t)mb * p.nKB + kb];
                            if (nb < p.b_rows) bu |= p.b_pat[(size_t)nb * p.nKB + kb];
                        }
                    }
                    const unsigned live = au & bu;
                    if (kb0 == 0) live_first = __shfl_sync(0xFFFFFFFFu, live, 0);
                    uniform = uniform && __all_sync(0xFFFFFFFFu, kb >= p.nKB || live == live_first);
                    full = false;   // the byte-wise path keeps the general listing
                    live_total += __reduce_add_sync(0xFFFFFFFFu, __popc(live));
                    live_small += __reduce_add_sync(0xFFFFFFFFu, __popc(live) <= p.brow_bits ? __popc(live) : 0);
                }
            }
            // uniform tile: list live k only.  Otherwise the policy is two numbers: K blocks with more than brow_bits
            // live k are listed whole, on tiles with at most row_density live k per K block on average; denser
            // tiles list every live K block whole.  With the producers fetching runs of consecutive rows as boxes,
            // listing exactly the live k is best at every density measured (brow_bits 7, row_density 8: a K
            // block is then listed whole only when it is whole; 6 / 6 was 2-4 % slower on independent
            // 32-granular patterns at 0.5 / 0.5 and 0.3 / 0.7).
            const int whole_above = uniform ? BK : (live_total <= p.row_density * p.nKB ? p.brow_bits : 0);
            // a run tile?  c = 1, 2, 4 or 8 consecutive live k, whole stages only, 3-D view of B valid
            int run_code = 0;
            {
                const int c = __popc(live_first);
                const int kk0 = __ffs((int)live_first) - 1;
                if (uniform && full && live_first != 0u && (c & (c - 1)) == 0 &&
                    (live_first >> kk0) == (1u << c) - 1u && (p.nKB * c) % ROWS_PER_STAGE == 0 && p.b_runs_ok &&
                    !p.force_listed && !p.no_run_tiles)
                    run_code = RUN_TILE | (31 - __clz(c)) | (kk0 << 4);
            }
            int pos = 0;
            if (run_code) {
                pos = p.nKB * __popc(live_first);
            } else if (p.vec_patterns == 16) {
                pos = tile_list<RB, 16>(p, tm, tn, lane, whole_above, krow, rmask);
            } else if (p.vec_patterns == 4) {
                pos = tile_list<RB, 4>(p, tm, tn, lane, whole_above, krow, rmask);
            } else {
                for (int kb0 = 0; kb0 < p.nKB; kb0 += 32) {
                    const int kb = kb0 + lane;
                    unsigned aw = 0, bw = 0;  // byte i: pattern of the tile's i-th 32-row / 32-column block
                    if (kb < p.nKB) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int mb = tm * RB + i, nb = tn * 4 + i;
                            if (i < RB && mb < p.a_rows) aw |= (unsigned)p.a_pat[(size_t)mb * p.nKB + kb] << (8 * i);
                            if (nb < p.b_rows) bw |= (unsigned)p.b_pat[(size_t)nb * p.nKB + kb] << (8 * i);
                        }
                    }
                    const unsigned live = tile_live(aw, bw);            // k live for the tile as a whole
                    const unsigned rows = live == 0u ? 0u : (__popc(live) > whole_above ? 0xFFu : live);
                    const int c = __popc(rows);
                    const int incl = warp_inclusive_scan(c, lane);
                    append_rows(krow, rmask, pos + incl - c, kb, rows, aw, bw, p.cap, p.status);
                    pos += __shfl_sync(0xFFFFFFFFu, incl, 31);
                }
            }
            // rows past the end of the last stage read as dead
            if (!run_code) {
                const int q = pos + lane;
                if (q < ((pos + 31) & ~31) && bounds_ok(q < p.cap, p.status, 22)) {
                    krow[q] = 0;
                    rmask[q] = 0;
                }
            }
            // a tile of mostly single rows: no stage of it is a run of whole K blocks, bar a rare coincidence
            const bool sparse_rows = !run_code && !uniform && whole_above == p.brow_bits && 2 * live_small >= pos;
            if (it == 0 && (NPW == 7 || (blockIdx.x == 0 && p.form_hint != nullptr))) {
                // 16-warp form: how many producer warps copy.  A row-by-row stage costs its producers the same 64
                // copies whatever the patterns, and its consumers one pass per row that is live for their own
                // 64 (32) rows x 32 columns.  Where the CTA's first tile is mostly such rows and a consumer warp
                // works on 12 of a stage's 32 rows or fewer, three producers cannot keep up and all seven copy;
                // otherwise three do and four stay idle.
                bool wants7 = false;
                if (sparse_rows) {
                    __syncwarp();
                    wants7 = listed_warp_rows<WMB>(rmask, min(pos, p.cap), lane) <= 3 * pos;
                }
                if (lane == 0) {
                    *n_producers = !p.adaptive || wants7 ? 7 : 3;
                    // (either form computes the same C; the note only steers the shape of the next launch)
                    if (blockIdx.x == 0 && p.form_hint != nullptr) *p.form_hint = wants7 ? 1 : 0;
                }
            }
            if (lane == 0) {
                nrows[buf] = pos;
                runinfo[buf] = run_code | (sparse_rows ? 0 : RUNS_LIKELY);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(lfull0 + 8 * buf);
            if (it == 0) ESMM_STAMP(1);
        }
    } else if (warp >= P_TMA_WARP) {
        if (P_REBALANCE_REGS) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(ESMM_PROD_REGS));
        // ---------------- producer warps: one lane per row of the stage ----------------
        // All of them walk the row list and take the same decisions; producer q issues the copies of
        // rows 32 q / P .. of each stage, producer 0 also the stage's byte count and whole-stage boxes.
        // (A copy may complete before producer 0 has posted the byte count: the barrier's transaction
        // count then goes negative for a moment, which it is allowed to, and the phase cannot complete
        // before producer 0's arrival.)
        const int q = warp - P_TMA_WARP;
        if (q == 0 && lane < 16) tma_prefetch_descriptor(&maps.a_box[0] + lane);
        int slot = 0;
        uint32_t phase = 0;
        uint32_t issued_bits = 0, parity_bits = 0;  // per slot: ever issued / parity of last issue
        int it = 0;
        int copying = P_TMA_WARPS;   // producer warps that share the copies out
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            ok = NPW == 7 && q >= copying ? mbar_wait_idle(lfull0 + 8 * buf, (it >> 1) & 1, abort_flag)
                                          : mbar_wait(lfull0 + 8 * buf, (it >> 1) & 1, abort_flag);
            if (!ok) break;
            if (NPW == 7 && it == 0) copying = *n_producers;
            if (NPW == 7 && q >= copying) {
                // an idle producer: it only hands the list buffer back, once per tile
                __syncwarp();
                if (lane == 0) mbar_arrive(lempty0 + 8 * buf);
                continue;
            }
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn, p.group_m);
            const uint16_t *krow = reinterpret_cast<const uint16_t *>(smem + L.krow_off + buf * L.krow_stride);
            const int n = nrows[buf];
            const int run_code = runinfo[buf] & (RUN_TILE | 0xFF);
            const bool look_for_runs = (runinfo[buf] & RUNS_LIKELY) != 0 && p.b_runs_ok;
            // packed A is stored in panels of 128 rows: a 64-row tile is the left or right half of one
            const int panel = WMB == 2 ? tm : tm >> 1;
            const int a_x = WMB == 2 ? 0 : (tm & 1) * TM_ROWS;
            const int a_row0 = panel * p.kp, b_col0 = tn * TILE_N;
            if (run_code) {
                // a run tile: whole stages, each one box per operand, no row list
                const int lc = run_code & 15, kk0 = (run_code >> 4) & 7;
                for (int r0 = 0; r0 < n; r0 += ROWS_PER_STAGE) {
                    // (every producer waits for every stage's slot, also where it has nothing to copy: a
                    // parity wait only tells "this phase" from "the one before", so no producer may get
                    // more than one lap of the ring ahead of the consumers)
                    ok = mbar_wait(empty0 + 8 * slot, phase ^ 1, abort_flag);
                    if (!ok) break;
                    const uint32_t full = full0 + 8 * slot;
                    if (q == 0 && lane == 0) {
                        mbar_arrive_expect_tx(full, (uint32_t)ROWS_PER_STAGE * STAGE_ROW_BYTES);
                        const uint32_t s0 = smem_u32(smem + L.stage_off) + (uint32_t)slot * PSTAGE_BYTES;
                        const int kb0 = r0 >> lc;
                        tma_load_3d(s0, &maps.a_run[lc], a_x, kk0, panel * p.nKB + kb0, full);
                        tma_load_3d(s0 + STAGE_HALF_BYTES, &maps.b_run[lc], b_col0, kk0, kb0, full);
                    }
                    if (q == 0) {
                        issued_bits |= 1u << slot;
                        parity_bits = (parity_bits & ~(1u << slot)) | (phase << slot);
                    }
                    if (it == 0 && q == 0) ESMM_STAMP(400 + r0 / ROWS_PER_STAGE);
                    if (++slot == p.stages) {
                        slot = 0;
                        phase ^= 1;
                    }
                }
            }
            // (the k of a stage's rows are read one stage ahead, under the copies of the stage before)
            int k_next = !run_code && lane < n && bounds_ok(lane < p.cap, p.status, 27) ? (int)krow[lane] : -1;
            for (int r0 = 0; r0 < n && !run_code; r0 += ROWS_PER_STAGE) {
                const int cnt = min(ROWS_PER_STAGE, n - r0);
                const bool valid = lane < cnt;
                if (it == 0 && q == 0 && r0 < 80 * ROWS_PER_STAGE) ESMM_STAMP(700 + 4 * (r0 / ROWS_PER_STAGE));
                const int k = k_next;
                {
                    const int rn = r0 + ROWS_PER_STAGE + lane;
                    k_next = rn < n && bounds_ok(rn < p.cap, p.status, 27) ? (int)krow[rn] : -1;
                }
                // a uniform run?  rows = k offsets kk0 .. kk0 + c - 1 of 32 / c consecutive K blocks
                const int k_first = __shfl_sync(0xFFFFFFFFu, k, 0);
                const int kb0 = k_first >> 3, kk0 = k_first & 7;
                int run = -1;  // log2(c)
                if (cnt == ROWS_PER_STAGE && look_for_runs) {
#pragma unroll
                    for (int lc = 3; lc >= 0; --lc) {
                        const int c = 1 << lc;
                        const int expect = ((kb0 + (lane >> lc)) << 3) + kk0 + (lane & (c - 1));
                        if (run < 0 && kk0 + c <= BK && __all_sync(0xFFFFFFFFu, k == expect)) run = lc;
                    }
                }
                // otherwise: the list is ascending, and rows with consecutive k are consecutive rows of packed A and of
                // B alike, so a run of L such rows is fetched in boxes of 8, 4, 2 and 1 rows (L = 8 a + 4 b + 2 c +
                // d, largest first): fewer copies for the same bytes.  The lane at a box's first row issues it.
                const int k_prev = __shfl_up_sync(0xFFFFFFFFu, k, 1);
                const unsigned starts = __ballot_sync(0xFFFFFFFFu, valid && (lane == 0 || k != k_prev + 1));
                int box_log = -1;   // log2 of the height of the box this lane issues
                if (valid && run < 0) {
                    const int first = 31 - __clz((int)(starts & (0xFFFFFFFFu >> (31 - lane))));   // my run's first lane
                    const unsigned later = lane == 31 ? 0u : (starts >> (first + 1)) << (first + 1);
                    const int len = (later ? __ffs((int)later) - 1 : cnt) - first;
                    const int o = lane - first;
                    const int full8 = len & ~7;
                    if (o < full8) box_log = (o & 7) == 0 ? 3 : -1;
                    else if ((len & 4) && o == full8) box_log = 2;
                    else if ((len & 2) && o == full8 + (len & 4)) box_log = 1;
                    else if ((len & 1) && o == len - 1) box_log = 0;
                }
                // my share of the stage: the boxes that start in my lane group
                if (((lane * copying) >> 5) != q) box_log = -1;
                if (it == 0 && q == 0 && r0 < 80 * ROWS_PER_STAGE) ESMM_STAMP(701 + 4 * (r0 / ROWS_PER_STAGE));
                ok = mbar_wait(empty0 + 8 * slot, phase ^ 1, abort_flag);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                if (it == 0 && q == 0 && r0 < 80 * ROWS_PER_STAGE) ESMM_STAMP(702 + 4 * (r0 / ROWS_PER_STAGE));
                {
                    const uint32_t full = full0 + 8 * slot;
                    const uint32_t s0 = smem_u32(smem + L.stage_off) + (uint32_t)slot * PSTAGE_BYTES;
                    const uint32_t sa = s0 + lane * A_ROW;
                    const uint32_t sb = s0 + STAGE_HALF_BYTES + lane * ROW_BYTES;
                    if (run >= 0) {
                        if (q == 0 && lane == 0) {
                            tma_load_3d(sa, &maps.a_run[run], a_x, kk0, panel * p.nKB + kb0, full);
                            tma_load_3d(sb, &maps.b_run[run], b_col0, kk0, kb0, full);
                        }
                    } else if (box_log >= 0) {
                        tma_load_2d(sa, &maps.a_box[box_log], a_x, a_row0 + k, full);
                        tma_load_2d(sb, &maps.b_box[box_log], b_col0, k, full);
                    }
                    if (q == 0 && lane == 0) mbar_arrive_expect_tx(full, (uint32_t)cnt * STAGE_ROW_BYTES);
                    issued_bits |= 1u << slot;
                    parity_bits = (parity_bits & ~(1u << slot)) | (phase << slot);
                }
                if (it == 0 && q == 0) ESMM_STAMP(400 + r0 / ROWS_PER_STAGE);
                if (it == 0 && q == 0 && r0 < 80 * ROWS_PER_STAGE) ESMM_STAMP(703 + 4 * (r0 / ROWS_PER_STAGE));
                if (++slot == p.stages) {
                    slot = 0;
                    phase ^= 1;
                }
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(lempty0 + 8 * buf);
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
        if (P_REBALANCE_REGS) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(ESMM_CONS_REGS));
        // ---------------- consumer warps: 32 WMB rows x 32 columns of the tile each ----------------
        const int wm = warp >> 2, wn = warp & 3;              // 2 x 4 warps
        const int lm = (lane >> 1) & 7;                       // group of 4 rows within a 32-row block
        const int ln = (lane & 1) | ((lane >> 4) << 1);       // 16-byte column chunk
        const uint32_t a_thr = (uint32_t)(wm * 32 * WMB + lm * 4) * 4;                // within a row of A
        const uint32_t b_thr = STAGE_HALF_BYTES + (uint32_t)(wn * 32 + ln * 4) * 4;  // within a row of B
        const int t_shift = WMB * wm, b_shift = 4 + wn;
        uint16_t *wlist_t = reinterpret_cast<uint16_t *>(smem + L.wlist_off + warp * 2 * WLIST_BYTES);
        uint16_t *wlist_b = wlist_t + WLIST_BYTES / 2;
        int slot = 0;
        uint32_t phase = 0;
        int it = 0;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            ok = mbar_wait(lfull0 + 8 * buf, (it >> 1) & 1, abort_flag);
            if (!ok) break;
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn, p.group_m);
            const uint8_t *rmask = reinterpret_cast<const uint8_t *>(smem + L.rmask_off + buf * L.rmask_stride);
            const int n = nrows[buf];
            const bool run_tile = (runinfo[buf] & RUN_TILE) != 0;
            if (warp == 0) ESMM_STAMP(600 + 4 * it);

            Acc acc;
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc.diag[i][j] = make_float2(0.0f, 0.0f);
                    acc.anti[i][j] = make_float2(0.0f, 0.0f);
                }

            // joint masks of a stage: bit r = row r is live for (top | bottom) block x my columns.  The
            // masks of the next stage are formed under the multiply-adds of the current one (the list's
            // buffer is padded by one stage, so reading one stage past the end is harmless).
            unsigned rm = run_tile ? 0xFFu : rmask[lane];   // (cap >= 64: the first stage is always inside the list)
            for (int r0 = 0; r0 < n; r0 += ROWS_PER_STAGE) {
                unsigned jt = 0xFFFFFFFFu, jb = 0xFFFFFFFFu;   // a run tile: every row live for every block
                if (!run_tile) {
                    const unsigned colb = (rm >> b_shift) & 1u;
                    jt = __ballot_sync(0xFFFFFFFFu, ((rm >> t_shift) & colb) != 0u);
                    jb = WMB == 2 ? __ballot_sync(0xFFFFFFFFu, ((rm >> (t_shift + 1)) & colb) != 0u) : jt;
                    rm = bounds_ok(r0 + ROWS_PER_STAGE + lane < p.cap, p.status, 23) ? rmask[r0 + ROWS_PER_STAGE + lane] : 0u;
                }
                const bool dense = (jt & jb) == 0xFFFFFFFFu && !p.force_listed;
                // in the 64-row tiling a row feeds 16 two-wide FMAs, as in the half modes: lists there too
                int cnt_t = 0, cnt_b = 0;
                if (WMB == 1 ? !dense : jt != jb) {
                    cnt_t = build_list(wlist_t, jt, lane, p.status);
                    if (WMB == 2) cnt_b = build_list(wlist_b, jb, lane, p.status);
                    __syncwarp();
                }
                ok = mbar_wait(full0 + 8 * slot, phase, abort_flag);
                if (!ok) break;
                if (!bounds_ok(slot >= 0 && slot < p.stages && L.stage_off + (uint32_t)(slot + 1) * PSTAGE_BYTES <= L.krow_off,
                               p.status, 24)) {
                    ok = false;   // a stage outside the ring: leave through the time-out path rather than read it
                    break;
                }
                const char *sA = smem + L.stage_off + (size_t)slot * PSTAGE_BYTES + a_thr;
                const char *sB = smem + L.stage_off + (size_t)slot * PSTAGE_BYTES + b_thr;
                if (warp == 0 && it == 0) ESMM_STAMP(10 + r0 / ROWS_PER_STAGE);
                if (dense) {
                    dense_rows<WMB>(acc, sA, sB);
                } else if (WMB == 1) {
                    listed_rows<MODE_TOP, 1>(acc, sA, sB, wlist_t, cnt_t);
                } else if (jt == jb) {
                    masked_rows_both(acc, sA, sB, jt);
                } else {
                    listed_rows<MODE_TOP, 2>(acc, sA, sB, wlist_t, cnt_t);
                    listed_rows<MODE_BOTTOM, 2>(acc, sA, sB, wlist_b, cnt_b);
                }
                if (warp == 0 && it == 0) ESMM_STAMP(200 + r0 / ROWS_PER_STAGE);
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * slot);
                if (++slot == p.stages) {
                    slot = 0;
                    phase ^= 1;
                }
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(lempty0 + 8 * buf);
            if (warp == 0) ESMM_STAMP(601 + 4 * it);

            // epilogue: C is overwritten (beta = 0); un-scramble the 2 x 2 blocks into rows
            const int row0 = tm * TM_ROWS + wm * 32 * WMB + lm * 4;
            const int col0 = tn * TILE_N + wn * 32 + ln * 4;
#pragma unroll
            for (int pr = 0; pr < 2 * WMB; ++pr) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int i = 2 * pr + e;                        // row of the thread tile
                    const int row = row0 + (i & 3) + 32 * (i >> 2);
                    float v[8];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        v[2 * q] = e == 0 ? acc.diag[pr][q].x : acc.anti[pr][q].y;
                        v[2 * q + 1] = e == 0 ? acc.anti[pr][q].x : acc.diag[pr][q].y;
                    }
                    if (row < p.M) {
                        float *c = p.C + (size_t)row * p.N + col0;
                        const size_t c_floats = (size_t)p.M * p.N, off = (size_t)row * p.N + col0;
                        if (col0 < p.N && bounds_ok(off + 4 <= c_floats, p.status, 26))
                            *reinterpret_cast<float4 *>(c) = make_float4(v[0], v[1], v[2], v[3]);
                        if (col0 + 16 < p.N && bounds_ok(off + 20 <= c_floats, p.status, 26))
                            *reinterpret_cast<float4 *>(c + 16) = make_float4(v[4], v[5], v[6], v[7]);
                    }
                }
            }
            if (warp == 0) ESMM_STAMP(602 + 4 * it);
        }
    }

    if (warp == 0) ESMM_STAMP(5);
    if (!ok && lane == 0) atomicExch(p.status, (int)ESMM_ERR_TIMEOUT);
}

#ifdef ESMM_TRACE
extern "C" int esmm_trace_read(unsigned long long *host, int n)
{
    return (int)cudaMemcpyFromSymbol(host, g_esmm_trace, sizeof(unsigned long long) * (n < 1024 ? n : 1024));
}
#endif

// esmm_gemm_skinny.cu: the kernel for M <= 32
bool gemm_ab_skinny_applies(int M, int N, int K);
int gemm_ab_skinny_launch(int M, int N, int K, const float *d_a_packed, const float *d_B, float *d_C,
                          const uint8_t *d_a_pat, const uint8_t *d_b_pat, cudaStream_t stream);

// The launch shape follows the operands: the 16-warp form pays on tiles of scattered single rows and costs about
// half a percent elsewhere, and which kind the operands are is known on the device only.  So CTA 0 of every
// launch notes what its first tile would have wanted in a word of host-mapped memory (one per device, set up at
// the first launch), and the next launch on that device reads the word, without waiting for anything: repeated
// products of like operands - what a benchmark loop or a layer with fixed weights issues - get the right
// shape from the second call on, and a stale or missing note only costs that difference.  The results are
// bit-identical in both shapes.  esmm_tuning_set("PRODUCER_WARPS", 3 | 7 | 0) pins the shape instead.
static std::atomic<int> g_last_tiled_warps[64];   // per device: warps per CTA of the last launch of the tiled kernel

struct FormHint {
    volatile int *host = nullptr;   // what the host reads
    int *device = nullptr;          // the same word as the kernels address it
};

static FormHint form_hint_word(int dev)
{
    static std::mutex mu;
    static FormHint words[64];
    if (dev < 0 || dev >= 64) return FormHint();
    std::lock_guard<std::mutex> lock(mu);
    if (!words[dev].host) {
        void *h = nullptr, *d = nullptr;
        if (cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess ||
            cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) {
            (void)cudaGetLastError();   // no note then: the 12-warp form is launched
            if (h) (void)cudaFreeHost(h);
            return FormHint();
        }
        memset(h, 0, 64);
        words[dev].host = static_cast<volatile int *>(h);
        words[dev].device = static_cast<int *>(d);
    }
    return words[dev];
}

// Once per device: the SM count, and the shared-memory allowance of all four forms of the kernel raised to the device's
// maximum.  (Raising it also loads the forms' code, so that the first launch in the other shape does not pay for that.)
static int prepare_device(int dev, int *sms)
{
    static std::mutex mu;
    static int sm_count[64] = {0};
    if (dev < 0 || dev >= 64) return ESMM_ERR_CUDA;
    std::lock_guard<std::mutex> lock(mu);
    if (!sm_count[dev]) {
        int n = 0, smem = 0;
        ESMM_CUDA_TRY(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
        ESMM_CUDA_TRY(cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        ESMM_CUDA_TRY(cudaFuncSetAttribute(esmm_joint_sgemm_packed_kernel<1, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        ESMM_CUDA_TRY(cudaFuncSetAttribute(esmm_joint_sgemm_packed_kernel<2, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        ESMM_CUDA_TRY(cudaFuncSetAttribute(esmm_joint_sgemm_packed_kernel<1, 7>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        ESMM_CUDA_TRY(cudaFuncSetAttribute(esmm_joint_sgemm_packed_kernel<2, 7>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        sm_count[dev] = n;
    }
    *sms = sm_count[dev];
    return ESMM_OK;
}

int gemm_ab_packed_launch_form(int M, int N, int K, const float *d_a_packed, const float *d_B, float *d_C,
                               const uint8_t *d_a_pat, const uint8_t *d_b_pat, cudaStream_t stream, bool follow_hint);

// The once-per-device set-up of the tiled kernel on the current device, for callers that want it outside a timed region.
int gemm_ab_packed_prepare()
{
    int dev = 0, sms = 0;
    ESMM_CUDA_TRY(cudaGetDevice(&dev));
    const int st = prepare_device(dev, &sms);
    if (st == ESMM_OK && tuning_get("PRODUCER_WARPS", -1) < 0) (void)form_hint_word(dev);
    return st;
}

int gemm_ab_packed_launch(int M, int N, int K, const float *d_a_packed, const float *d_B, float *d_C,
                          const uint8_t *d_a_pat, const uint8_t *d_b_pat, cudaStream_t stream)
{
    return gemm_ab_packed_launch_form(M, N, K, d_a_packed, d_B, d_C, d_a_pat, d_b_pat, stream, true);
}

// follow_hint = false: the 12-warp form unless PRODUCER_WARPS says otherwise, and no host-mapped word (for the
// entry point that may not allocate).
int gemm_ab_packed_launch_form(int M, int N, int K, const float *d_a_packed, const float *d_B, float *d_C,
                               const uint8_t *d_a_pat, const uint8_t *d_b_pat, cudaStream_t stream, bool follow_hint)
{
    if (!d_a_packed || !d_B || !d_C || !d_a_pat || !d_b_pat) return ESMM_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || (K & 3) || (N & 3)) return ESMM_ERR_SHAPE;
    if (((uintptr_t)d_a_packed | (uintptr_t)d_B | (uintptr_t)d_C) & 15) return ESMM_ERR_ALIGN;
    if (gemm_ab_skinny_applies(M, N, K))
        return gemm_ab_skinny_launch(M, N, K, d_a_packed, d_B, d_C, d_a_pat, d_b_pat, stream);

    PackedParams p;
    memset(&p, 0, sizeof p);
    p.M = M;
    p.N = N;
    p.K = K;
    p.nKB = ceil_div(K, BK);
    p.kp = p.nKB * BK;
    if (p.kp > 65535) return ESMM_ERR_TOO_LARGE;  // row list entries are 16-bit k indices
    p.cap = ((p.kp + 31) & ~31) + 32;
    p.a_rows = ceil_div(M, 32);
    p.b_rows = ceil_div(N, PAT_N);
    int dev = 0, sms = 0;
    ESMM_CUDA_TRY(cudaGetDevice(&dev));
    {
        const int pst = prepare_device(dev, &sms);
        if (pst != ESMM_OK) return pst;
    }
    // Tile height: 128 rows, or 64 where that fills the GPU better.  Rounds of tiles per SM, a 64-row
    // tile counted as 0.55 of a 128-row one (it does half the multiply-adds at a worse ratio of
    // shared-memory loads).  ESMM_TILE_M = 64 | 128 overrides.
    p.tiles_n = ceil_div(N, TILE_N);
    const int panels = ceil_div(M, TILE_M);
    const long t128 = (long)panels * p.tiles_n, t64 = (long)ceil_div(M, 64) * p.tiles_n;
    const double cost128 = (double)((t128 + sms - 1) / sms), cost64 = 0.55 * (double)((t64 + sms - 1) / sms);
    int tile_rows = cost64 < cost128 ? 64 : TILE_M;
    const int forced_rows = tuning_get("TILE_M", 0);
    if (forced_rows == 64 || forced_rows == TILE_M) tile_rows = forced_rows;
    p.tiles_m = ceil_div(M, tile_rows);
    p.num_tiles = p.tiles_m * p.tiles_n;
    p.group_m = tuning_get("GROUP_M", GROUP_M);
    if (p.group_m < 1) p.group_m = 1;
    p.brow_bits = tuning_get("BROW_BITS", 7);
    if (p.brow_bits < 0) p.brow_bits = 0;
    if (p.brow_bits > 8) p.brow_bits = 8;
    p.row_density = tuning_get("ROW_DENSITY", 8);
    p.force_listed = tuning_get("FORCE_LISTED", 0);
    p.no_run_tiles = tuning_get("NO_RUN_TILES", 0);
    const uintptr_t pat_bits = (uintptr_t)d_a_pat | (uintptr_t)d_b_pat;
    p.vec_patterns = 0;
    if (p.nKB % 4 == 0 && (pat_bits & 3) == 0) p.vec_patterns = 4;
    if (p.nKB % 16 == 0 && (pat_bits & 15) == 0 && p.nKB >= 512) p.vec_patterns = 16;
    const int forced_vec = tuning_get("VEC_PATTERNS", -1);   // 0, 4, 16: tuning and tests
    if (forced_vec == 0 || (forced_vec == 4 && p.vec_patterns >= 4) ||
        (forced_vec == 16 && p.nKB % 16 == 0 && (pat_bits & 15) == 0))
        p.vec_patterns = forced_vec;
    p.a_pat = d_a_pat;
    p.b_pat = d_b_pat;
    p.C = d_C;

    int stages = tuning_get("STAGES", P_MAX_STAGES);
    if (stages > P_MAX_STAGES) stages = P_MAX_STAGES;
    if (stages < 2) stages = 2;
    while (stages > 2 && packed_smem_layout(stages, p.cap).total > SMEM_LIMIT) --stages;
    const PackedSmem L = packed_smem_layout(stages, p.cap);
    if (L.total > SMEM_LIMIT) return ESMM_ERR_TOO_LARGE;
    p.stages = stages;

    p.status = device_status_ptr();
    if (!p.status) return ESMM_ERR_CUDA;

    // Packed A is a matrix of 128 columns and panels * kp rows, of which a tile reads all 128 columns
    // or the 64 of its half; B is K rows of N columns.  Rows
    // (or columns of B) outside the matrices are zero-filled by the copy engine and still counted
    // in the stage's byte total.  The 3-D views split the row index into (k % 8, k / 8); for B
    // that is only valid when K is a multiple of 8 (otherwise the view would reach past row K).
    p.b_runs_ok = (K % BK) == 0;
    PackedMaps maps;
    const uint64_t a_rows_total = (uint64_t)panels * p.kp;
    int st = 0;
    for (int i = 0; i < 4 && !st; ++i) {
        st = make_map_2d(&maps.a_box[i], d_a_packed, TILE_M, a_rows_total, tile_rows, 1u << i, CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        if (!st) st = make_map_2d(&maps.b_box[i], d_B, (uint64_t)N, (uint64_t)K, TILE_N, 1u << i, CU_TENSOR_MAP_SWIZZLE_NONE,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    }
    for (int i = 0; i < 4 && !st; ++i) {
        const uint32_t c = 1u << i;
        st = make_map_3d(&maps.a_run[i], d_a_packed, TILE_M, BK, (uint64_t)panels * p.nKB, (uint64_t)TILE_M * 4,
                         (uint64_t)TILE_M * 4 * BK, tile_rows, c, ROWS_PER_STAGE / c);
        if (!st) {
            if (p.b_runs_ok)
                st = make_map_3d(&maps.b_run[i], d_B, (uint64_t)N, BK, (uint64_t)p.nKB, (uint64_t)N * 4,
                                 (uint64_t)N * 4 * BK, TILE_N, c, ROWS_PER_STAGE / c);
            else
                maps.b_run[i] = maps.b_box[0];  // never used
        }
    }
    if (st) return st;

    int grid = tuning_get("GRID", sms);
    if (grid > p.num_tiles) grid = p.num_tiles;
    if (grid < 1) grid = 1;
    // 3 = 12 warps; 7 = 16 warps, 7 producers copying; 0 = 16 warps, 3 or 7 copying as each CTA's first tile says;
    // not set = 3 or 0 as the last launch on this device noted
    int producer_warps = tuning_get("PRODUCER_WARPS", -1);
    if (producer_warps != 3 && producer_warps != 7 && producer_warps != 0) {
        producer_warps = 3;
        if (follow_hint) {
            const FormHint hint = form_hint_word(dev);
            if (hint.host) {
                p.form_hint = hint.device;
                if (*hint.host != 0) producer_warps = 0;
            }
        }
    }
    const bool wide = producer_warps != 3;
    p.adaptive = producer_warps == 0;
    if (dev >= 0 && dev < 64) g_last_tiled_warps[dev].store(wide ? 16 : 12, std::memory_order_relaxed);
    auto launch = [&](auto kernel, int threads) -> int {
        ESMM_CUDA_TRY(launch_dependent(kernel, dim3(grid), dim3(threads), L.total, stream, maps, p));
        return ESMM_OK;
    };
    const int threads = (P_CONSUMER_WARPS + (wide ? 7 : 3) + 1) * 32;
    int lst;
    if (tile_rows == 64) lst = wide ? launch(esmm_joint_sgemm_packed_kernel<1, 7>, threads) : launch(esmm_joint_sgemm_packed_kernel<1, 3>, threads);
    else lst = wide ? launch(esmm_joint_sgemm_packed_kernel<2, 7>, threads) : launch(esmm_joint_sgemm_packed_kernel<2, 3>, threads);
    if (lst != ESMM_OK) return lst;
    ESMM_CUDA_TRY(cudaGetLastError());
    return ESMM_OK;
}

int last_tiled_warps()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    return g_last_tiled_warps[dev].load(std::memory_order_relaxed);
}

}  // namespace esmm

extern "C" int esmm_last_tiled_kernel_warps(void) { return esmm::last_tiled_warps(); }

extern "C" int esmm_gemm_ab_packed(int M, int N, int K, const float *d_a_packed, const float *d_B, float *d_C,
                                   const uint8_t *d_a_pat, const uint8_t *d_b_pat, void *stream)
{
    return esmm::gemm_ab_packed_launch(M, N, K, d_a_packed, d_B, d_C, d_a_pat, d_b_pat, (cudaStream_t)stream);
}
