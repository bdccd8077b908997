// Optional tensor-core variant of the joint-sparse SGEMM: 3xTF32 on tcgen05 (sm_100a), accumulators in TMEM.
//
// Every FP32 operand is split into two TF32 parts, x = hi + lo (hi = x rounded to TF32, lo = (x - hi) rounded
// to TF32), and a product is taken as  a_hi b_hi + a_hi b_lo + a_lo b_hi  with FP32 accumulation: three
// tensor-core MMAs per K step instead of 64 FP32 multiply-adds per thread.  The dropped a_lo b_lo term and the
// rounding of lo are of relative size 2^-22, far inside the 1e-4 relative tolerance the results are held to;
// the result is NOT bit-identical to the FP32 FMA kernels, which is why this is a separate entry point.
//
// Skipping happens at two levels.  (1) When B is prepared, every k whose row of B is all zero is dropped from both
// operands (the split of A gathers the kept columns), so patterns that repeat in every K block, the reference's
// benchmark patterns, shrink K itself.  (2) Of what is left, a K block (8 k, the K extent of one kind::tf32 MMA)
// of a tile is multiplied only if some k in it is live for the tile (OR of the A pattern bytes of the tile's row
// blocks AND OR of the B pattern bytes of its column blocks), and a group of four K blocks is fetched only if one is.
// Everything skipped multiplies exact zeros, so the sum is the one the reference's masked FMA chain forms
// (src/kernels/esmm_ab_optimized_v3.cu:157, 183-203) up to rounding.
//
// Rounding: the tensor core's own FP32 accumulation loses accuracy linearly in the number of MMAs (3e-5 of
// max |C| at K = 4096 when a whole tile is accumulated in one run), so a run is limited to T_CHUNK groups
// (256 k) and the epilogue warps add the runs in registers with round-to-nearest: 2e-6 at K = 4096 and 16384.
//
// Layouts: both operands K-major.  A_hi, A_lo: M x Kc row-major, written per call by the split kernel.
// Bt_hi, Bt_lo: N x Kc row-major (B transposed), written once per B ("B offline").  A group of four K blocks of
// one operand part is one TMA box of 32 floats x 128 rows with the 128-byte swizzle (16 KB), the canonical
// K-major shared-memory layout; the MMA of K block j of the group reads it through a descriptor that starts
// 32 j bytes into the swizzled row.  (Boxes of one K block with the 32-byte swizzle were measured first: 1.6 x
// slower, the copy engine handles about one box row per cycle whatever its width.)
//
// Kernels.  All persistent, one CTA per SM, warp-specialised: a mask warp lists the live groups of the next tile, a
// producer warp fetches one group per ring stage, one thread issues the MMAs and commits them to the ring's and
// the accumulator's mbarriers, epilogue warps drain one of two TMEM accumulators while the other is being filled.
// Every wait is bounded, as in the other kernels, and the tensor memory is freed on every path out.
//   esmm_joint_sgemm_tf32x3_pair_kernel<256>  large problems (the host picks the kernel by an estimate of the time per
//       SM: see esmm_sgemm_joint_tf32x3; ESMM_TF32_PAIR = 0 | 128 | 256 overrides).  Two CTAs of a cluster share a
//       256 x 256 tile (cta_group::2 MMAs, M 256, N 256): each CTA fetches its 128 rows of A and its 128 columns of
//       B, 16 KB per K block for two 128 x 128 tiles' worth of MMA work.  12 warps; the eight epilogue warps take
//       registers over from the other four (setmaxnreg) for their 128-column rows of run sums.
//   esmm_joint_sgemm_tf32x3_pair_kernel<128>  256 x 128 per pair: problems with too few 256 x 256 tiles to fill the GPU.
//   esmm_joint_sgemm_tf32x3_kernel            one CTA per 128 x 128 tile: M < 192, and where it fills its waves best.
//
// What was measured on the way (one B200, 4096^3 dense, cycles per group of four K blocks on one SM):
//   * 128 x 128 tiles need 64 KB per group and the SM takes in about 64 bytes per clock from L2: 1024 cycles, more
//     than the 813 cycles its twelve MMAs (128 x 128 x 8, 67.8 cycles each at the TF32 rate) take.  The single-CTA
//     kernel runs at 1082.  Pulling groups into L2 ahead of the ring changes nothing (DRAM is not the limit).
//   * The issuing thread's own instructions count: building two 64-bit descriptors per MMA cost 77 cycles per MMA
//     (more than the MMA); with one precomputed word per operand it is 57.  A wait on a data barrier costs about
//     170 cycles even when the data is there, so the next group's barrier is polled while the pipe has work.
//   * 256 x 256 on a CTA pair: 64 KB per group feed 12 MMAs of 128 x 256 x 8 per SM; measured 1588 cycles per
//     group in steady state, the tensor pipe's own time.  256 tiles on 74 pairs are 3.46 waves: the 34 tiles of
//     the last wave are computed as two halves of K by 68 pairs (they add into a zeroed C), 3.5 waves instead of
//     4.  In a long loop the GPU sits at its 1000 W power cap (SM clock 1.6-1.7 GHz, sw_power_cap the only reason).
// Whole call (split of A with its patterns + product), bursts of 20 calls: 0.51 ms dense against 2.35 ms for the
// FP32 kernel.
#include <algorithm>
#include <cstring>
#include <vector>

#include "esmm_gemm_shared.cuh"

namespace esmm {

constexpr int T_GROUP_KB = 4;                // K blocks per fetch group: 32 floats = one 128-byte swizzle row
constexpr int T_PART_BYTES = 128 * 128;      // one operand part of a group: 128 rows x 32 floats
constexpr int T_STAGE_BYTES = 4 * T_PART_BYTES;   // A_hi, A_lo, B_hi, B_lo: 65536
constexpr int T_STAGES = 3;
constexpr int T_CHUNK = 8;                   // groups (256 k) accumulated in tensor memory before the epilogue adds them up
constexpr int T_THREADS = 256;               // warps: 0 producer, 1 MMA, 2 mask, 3 idle, 4-7 epilogue
constexpr int T_TMEM_COLS = 256;             // two accumulators of 128 columns

struct Tf32Params {
    int M, N, K, nKB, cap;
    int stage_off;                           // byte offset of the epilogue's staging squares in shared memory, 0: none
    int num_items, split_first;              // pair kernels: work items; tiles >= split_first are two items (halves of K)
    int a_rows, b_rows, tiles_m, tiles_n, num_tiles;
    const uint8_t *a_pat;
    const uint8_t *b_pat;
    float *C;
    int *status;
};

struct Tf32Maps {
    CUtensorMap a_hi, a_lo, b_hi, b_lo;      // boxes of 32 floats x 128 rows, 128-byte swizzle
};

// Shared-memory matrix descriptor of a K-major TF32 operand inside a 128-byte-swizzled tile of rows x 32 floats:
// rows of 128 bytes, groups of 8 rows 1024 bytes apart (stride byte offset 64 at bit 32), descriptor version 1
// (bit 46), layout type 2 (bits 61-63), leading byte offset 1 (bit 16), start address >> 4 in the low 14 bits.
// K block j of the tile starts 32 j bytes into the row; the swizzle is a function of the address.
// The descriptor as two words: only the low one (start address, leading byte offset) changes from MMA to MMA; the
// K block j of a tile adds 2 j to it (32 j bytes >> 4).  The issuing thread's own instructions are on the critical
// path (one MMA of K = 8 keeps the tensor pipe busy for only about 65 cycles), so the 64-bit descriptor is put
// together inside the asm block from one precomputed word and a constant.
constexpr uint32_t UMMA_DESC_HI_K128 = 64u | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }

// instruction descriptor: D = F32 (bit 4), A = B = TF32 (bits 7, 10), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
constexpr uint32_t UMMA_IDESC_TF32_128x128 = (1u << 4) | (2u << 7) | (2u << 10) | (16u << 17) | (8u << 24);

template <bool PAIR, uint32_t IDESC>
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t accumulate)
{
    if constexpr (PAIR) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::tf32 [%0], da, db, %3, {%6, %6, %6, %6, %6, %6, %6, %6}, p;\n\t}\n" ::"r"(tmem_d),
            "r"(a_lo), "r"(b_lo), "r"(IDESC), "r"(accumulate), "r"(UMMA_DESC_HI_K128), "r"(0u)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %3, {%6, %6, %6, %6}, p;\n\t}\n" ::"r"(tmem_d),
            "r"(a_lo), "r"(b_lo), "r"(IDESC), "r"(accumulate), "r"(UMMA_DESC_HI_K128), "r"(0u)
            : "memory");
    }
}

// the three products of K block j of a group: small terms first
template <bool PAIR, uint32_t IDESC>
__device__ __forceinline__ void umma_kblock(uint32_t d, uint32_t ah, uint32_t al, uint32_t bh, uint32_t bl, uint32_t j,
                                            uint32_t accumulate)
{
    umma_tf32<PAIR, IDESC>(d, al + 2u * j, bh + 2u * j, accumulate);
    umma_tf32<PAIR, IDESC>(d, ah + 2u * j, bl + 2u * j, 1u);
    umma_tf32<PAIR, IDESC>(d, ah + 2u * j, bh + 2u * j, 1u);
}

// All live K blocks of a group (live: 4-bit mask, not 0); the dense case is unrolled with constant offsets.
// A wait on a data barrier costs the issuing thread about 170 cycles even when the data is there, more than
// two MMAs take, and the tensor pipe runs dry meanwhile.  So the next group's barrier is polled (one
// non-blocking test) right after this group's first K block is issued, while the pipe has work queued; the
// caller skips its wait when the poll said "landed".
template <bool PAIR, uint32_t IDESC>
__device__ __forceinline__ bool umma_group(uint32_t d, uint32_t ah, uint32_t al, uint32_t bh, uint32_t bl, unsigned live,
                                           uint32_t &accumulate, uint32_t next_bar, uint32_t next_parity)
{
    bool next_ready;
    if (live == 0xFu) {
        umma_kblock<PAIR, IDESC>(d, ah, al, bh, bl, 0u, accumulate);
        next_ready = mbar_test_wait(next_bar, next_parity);
        umma_kblock<PAIR, IDESC>(d, ah, al, bh, bl, 1u, 1u);
        umma_kblock<PAIR, IDESC>(d, ah, al, bh, bl, 2u, 1u);
        umma_kblock<PAIR, IDESC>(d, ah, al, bh, bl, 3u, 1u);
    } else {
        uint32_t j = (uint32_t)(__ffs(live) - 1);
        live &= live - 1;
        umma_kblock<PAIR, IDESC>(d, ah, al, bh, bl, j, accumulate);
        next_ready = mbar_test_wait(next_bar, next_parity);
        while (live) {
            j = (uint32_t)(__ffs(live) - 1);
            live &= live - 1;
            umma_kblock<PAIR, IDESC>(d, ah, al, bh, bl, j, 1u);
        }
    }
    accumulate = 1u;
    return next_ready;
}

__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld_32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// x = hi + lo with both parts representable in TF32 (low 13 mantissa bits clear)
__device__ __forceinline__ void split_tf32(float x, float &hi, float &lo)
{
    uint32_t h, l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    hi = __uint_as_float(h);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(x - hi));
    lo = __uint_as_float(l);
}

// A (M x K, row-major) -> A_hi, A_lo (M x Kc, row-major) and the A pattern bytes of the result, in one pass.
// klist == nullptr: Kc == K, the same columns.  Otherwise column j of the output is column klist[j] of A
// (ascending; -1: a zero column of padding).  A value whose TF32 hi part is zero has a zero lo part too and
// contributes nothing, so the pattern bit of (32-row block, k) is "some hi part is nonzero": the byte layout is the
// one of esmm_preprocess_a (src/preprocessors/ab_preprocessor.cu:122-187), a_pat[mb * (Kc / 8) + kb], bit k.
// One warp per 32 rows x 64 output columns: half-warp h takes the rows of parity h, lane c its float4 column.
// Rows of blocks past the last 32-row block of A zero the C tiles that the product kernel computes as two halves
// (ZeroJob; count 0: none): the pass is in the stream anyway and a launch of its own would cost more than the work.
struct ZeroJob {
    float *C;
    int N, tiles_m, tiles_n, nb, first, count;    // nb: tile width; tiles first .. first + count - 1, 256 rows each
};

__global__ void __launch_bounds__(256)
esmm_tf32_split_pattern_kernel(const float *__restrict__ A, int M, int K, const int *__restrict__ klist, int Kc,
                               float *__restrict__ hi, float *__restrict__ lo, uint8_t *__restrict__ a_pat,
                               const ZeroJob zj)
{
    const int a_blocks = (M + 31) >> 5;
    if ((int)blockIdx.y >= a_blocks) {
        if (blockIdx.x != 0) return;
        const int z = (int)blockIdx.y - a_blocks;                 // (tile, 32-row band)
        int tm, tn;
        tile_coords(zj.first + (z >> 3), zj.tiles_m, zj.tiles_n, tm, tn);
        const int row0 = tm * 256 + (z & 7) * 32, col0 = tn * zj.nb, q = zj.nb >> 2;
        for (int i = threadIdx.x; i < 32 * q; i += blockDim.x) {
            const int row = row0 + i / q, col = col0 + (i % q) * 4;
            if (row < M && col < zj.N)
                *reinterpret_cast<float4 *>(zj.C + (size_t)row * zj.N + col) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mb = blockIdx.y, col = (blockIdx.x * 8 + warp) * 64 + (lane & 15) * 4, h = lane >> 4;
    if ((blockIdx.x * 8 + warp) * 64 >= Kc) return;               // the whole warp is past the last column
    const bool in_cols = col < Kc;                                // Kc is a multiple of 8: a float4 is in or out
    int4 k = make_int4(col, col + 1, col + 2, col + 3);
    if (klist != nullptr && in_cols) k = __ldg(reinterpret_cast<const int4 *>(klist + col));
    float4 v[16];
#pragma unroll
    for (int rr = 0; rr < 16; ++rr) {
        const int row = mb * 32 + 2 * rr + h;
        v[rr] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (in_cols && row < M) {
            const float *a = A + (size_t)row * K;
            if (klist == nullptr) {
                v[rr] = __ldg(reinterpret_cast<const float4 *>(a + col));
            } else {
                v[rr].x = k.x >= 0 ? __ldg(a + k.x) : 0.0f;
                v[rr].y = k.y >= 0 ? __ldg(a + k.y) : 0.0f;
                v[rr].z = k.z >= 0 ? __ldg(a + k.z) : 0.0f;
                v[rr].w = k.w >= 0 ? __ldg(a + k.w) : 0.0f;
            }
        }
    }
    unsigned m = 0;
#pragma unroll
    for (int rr = 0; rr < 16; ++rr) {
        const int row = mb * 32 + 2 * rr + h;
        float4 hh, ll;
        split_tf32(v[rr].x, hh.x, ll.x);
        split_tf32(v[rr].y, hh.y, ll.y);
        split_tf32(v[rr].z, hh.z, ll.z);
        split_tf32(v[rr].w, hh.w, ll.w);
        m |= ((__float_as_uint(hh.x) << 1) != 0u ? 1u : 0u) | ((__float_as_uint(hh.y) << 1) != 0u ? 2u : 0u) |
             ((__float_as_uint(hh.z) << 1) != 0u ? 4u : 0u) | ((__float_as_uint(hh.w) << 1) != 0u ? 8u : 0u);
        if (in_cols && row < M) {
            *reinterpret_cast<float4 *>(hi + (size_t)row * Kc + col) = hh;
            *reinterpret_cast<float4 *>(lo + (size_t)row * Kc + col) = ll;
        }
    }
    m |= __shfl_xor_sync(0xFFFFFFFFu, m, 16);                     // both row parities
    const unsigned other = __shfl_xor_sync(0xFFFFFFFFu, m, 1);    // the K block's other four k
    if (lane < 16 && !(lane & 1) && in_cols) a_pat[(size_t)mb * (Kc >> 3) + (col >> 3)] = (uint8_t)(m | (other << 4));
}

// B (K x N, row-major) -> Bt_hi, Bt_lo (N x Kc, row-major): 32 x 32 tiles through shared memory; row j of the tile
// column is row klist[j] of B (or j itself without a list)
__global__ void esmm_tf32_split_transpose_kernel(const float *__restrict__ B, int K, int N, const int *__restrict__ klist,
                                                 int Kc, float *__restrict__ bt_hi, float *__restrict__ bt_lo)
{
    __shared__ float tile[32][33];
    const int j0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int j = j0 + r, n = n0 + threadIdx.x;
        const int k = j < Kc ? (klist ? klist[j] : j) : -1;
        tile[r][threadIdx.x] = (k >= 0 && k < K && n < N) ? B[(size_t)k * N + n] : 0.0f;
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int n = n0 + r, j = j0 + threadIdx.x;
        if (n < N && j < Kc) {
            float h, l;
            split_tf32(tile[threadIdx.x][r], h, l);
            bt_hi[(size_t)n * Kc + j] = h;
            bt_lo[(size_t)n * Kc + j] = l;
        }
    }
}

// A thread holds one C row of 128 run sums; written straight out, a warp's store touches 32 different rows (32
// sectors of 16 useful bytes), and those scattered stores were seen to hold up the ring's copies for thousands
// of cycles at every tile change.  Through a 32 x 33 float staging square per warp, every store instruction writes
// one full 128-byte line of one row instead.  stage == nullptr (no shared memory left for it): the direct form.
constexpr int T_STAGE_FLOATS = 32 * 33;
// add: the tile is computed as two halves of K by two CTA pairs; C was zeroed, both add their sums (two terms: the
// result does not depend on who comes first).
__device__ __forceinline__ void store_row_block(const float (&acc)[TILE_N], float *stage, float *C, int row0, int col0,
                                                int M, int N, int lane, bool add = false)
{
    if (stage == nullptr) {
        const int row = row0 + lane;
        if (row < M) {
            float *dst = C + (size_t)row * N + col0;
            if (add) {
#pragma unroll
                for (int j = 0; j < TILE_N; ++j)     // fully unrolled: acc must stay in registers
                    if (col0 + j < N) atomicAdd(dst + j, acc[j]);
            } else {
#pragma unroll
                for (int j = 0; j < TILE_N; j += 4)
                    if (col0 + j < N) *reinterpret_cast<float4 *>(dst + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
            }
        }
        return;
    }
#pragma unroll
    for (int cc = 0; cc < TILE_N; cc += 32) {
#pragma unroll
        for (int j = 0; j < 32; ++j) stage[lane * 33 + j] = acc[cc + j];
        __syncwarp();
        const int col = col0 + cc + lane;
        if (col < N) {
            float *dst = C + (size_t)row0 * N + col;
            const int rows = min(32, M - row0);
            if (add) {
#pragma unroll 8
                for (int r = 0; r < rows; ++r) atomicAdd(dst + (size_t)r * N, stage[r * 33 + lane]);
            } else {
#pragma unroll 8
                for (int r = 0; r < rows; ++r) dst[(size_t)r * N] = stage[r * 33 + lane];
            }
        }
        __syncwarp();
    }
}

__global__ void __launch_bounds__(T_THREADS, 1)
esmm_joint_sgemm_tf32x3_kernel(const __grid_constant__ Tf32Maps maps, const Tf32Params p)
{
    extern __shared__ __align__(1024) char smem[];
    // layout: ring (T_STAGES x 64 KB) | group lists (2 x cap u16) | barriers | misc
    const int list_stride = ((p.cap * 2 + 15) & ~15) / 2;
    uint16_t *lists = reinterpret_cast<uint16_t *>(smem + T_STAGES * T_STAGE_BYTES);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + T_STAGES * T_STAGE_BYTES + 4 * list_stride);
    // full[3], empty[3], acc_full[2], acc_empty[2], lfull[2], lempty[2]
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + 3), accf0 = smem_u32(bars + 6),
                   acce0 = smem_u32(bars + 8), lfull0 = smem_u32(bars + 10), lempty0 = smem_u32(bars + 12);
    volatile int *nlive = reinterpret_cast<volatile int *>(bars + 14);   // [2]: live groups of the listed tile
    volatile int *abort_flag = nlive + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(const_cast<int *>(nlive + 3));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < T_STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);        // one tcgen05.commit per stage
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(accf0 + 8 * b, 1);         // tcgen05.commit after the chunk's last MMA
            mbar_init(acce0 + 8 * b, 4);         // the four epilogue warps
            mbar_init(lfull0 + 8 * b, 1);
            mbar_init(lempty0 + 8 * b, 6);       // producer warp, MMA thread, four epilogue warps
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(T_TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const int nGroups = (p.nKB + T_GROUP_KB - 1) / T_GROUP_KB;
    bool ok = true;

    if (warp == 2) {
        // ---------------- mask warp: live groups of the tile (index | live K blocks << 12), one tile ahead ----------------
        int it = 0;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            ok = mbar_wait(lempty0 + 8 * buf, ((it >> 1) & 1) ^ 1, abort_flag);
            if (!ok) break;
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            uint16_t *list = lists + buf * list_stride;
            int pos = 0;
            for (int g0 = 0; g0 < nGroups; g0 += 32) {
                const int g = g0 + lane;
                unsigned live = 0;
                if (g < nGroups) {
                    // four pattern bytes per row block: one 32-bit load when the row of bytes allows it
                    unsigned au[T_GROUP_KB] = {0, 0, 0, 0}, bu[T_GROUP_KB] = {0, 0, 0, 0};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int mb = tm * 4 + i, nb = tn * 4 + i;
#pragma unroll
                        for (int j = 0; j < T_GROUP_KB; ++j) {
                            const int kb = g * T_GROUP_KB + j;
                            if (kb < p.nKB) {
                                if (mb < p.a_rows) au[j] |= p.a_pat[(size_t)mb * p.nKB + kb];
                                if (nb < p.b_rows) bu[j] |= p.b_pat[(size_t)nb * p.nKB + kb];
                            }
                        }
                    }
#pragma unroll
                    for (int j = 0; j < T_GROUP_KB; ++j) live |= ((au[j] & bu[j]) != 0u ? 1u : 0u) << j;
                }
                const unsigned m = __ballot_sync(0xFFFFFFFFu, live != 0u);
                if (live && bounds_ok(pos + __popc(m & ((1u << lane) - 1u)) < p.cap, p.status, 50))   // checked build: site 50
                    list[pos + __popc(m & ((1u << lane) - 1u))] = (uint16_t)(g | (live << 12));
                pos += __popc(m);
            }
            if (lane == 0) nlive[buf] = pos;
            __syncwarp();
            if (lane == 0) mbar_arrive(lfull0 + 8 * buf);
        }
    } else if (warp == 0) {
        // ---------------- producer: one stage per live group, lanes 0-3 fetch A_hi, A_lo, B_hi, B_lo ----------------
        if (lane < 4) tma_prefetch_descriptor(&maps.a_hi + lane);
        int slot = 0, it = 0;
        uint32_t phase = 0, issued_bits = 0, parity_bits = 0;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            ok = mbar_wait(lfull0 + 8 * buf, (it >> 1) & 1, abort_flag);
            if (!ok) break;
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            const uint16_t *list = lists + buf * list_stride;
            const int n = nlive[buf];
            const int row0 = (lane & 2) ? tn * TILE_N : tm * TILE_M;
            for (int q = 0; q < n; ++q) {
                ok = mbar_wait(empty0 + 8 * slot, phase ^ 1, abort_flag);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                const uint32_t full = full0 + 8 * slot;
                if (lane == 0) mbar_arrive_expect_tx(full, (uint32_t)T_STAGE_BYTES);
                __syncwarp();
                if (lane < 4) {
                    const int k = (int)(list[q] & 0xFFFu) * (T_GROUP_KB * BK);
                    tma_load_2d(smem_u32(smem) + (uint32_t)slot * T_STAGE_BYTES + (uint32_t)lane * T_PART_BYTES,
                                &maps.a_hi + lane, k, row0, full);
                }
                issued_bits |= 1u << slot;
                parity_bits = (parity_bits & ~(1u << slot)) | (phase << slot);
                if (++slot == T_STAGES) {
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
            for (int s = 0; s < T_STAGES; ++s) {
                if (!(issued_bits & (1u << s))) continue;
                const uint32_t par = (parity_bits >> s) & 1u;
                for (int tries = 0; tries < (1 << 16); ++tries)
                    if (mbar_try_wait(full0 + 8 * s, par)) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue: one thread; a chunk of T_CHUNK groups per accumulator ----------------
        if (lane == 0) {
            int slot = 0, it = 0;
            uint32_t phase = 0, chunk = 0;
            bool landed = false;                         // the next group's copies were seen complete by a poll
            const uint32_t ring_lo = umma_desc_lo(smem_u32(smem));
            for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++it) {
                const int buf = it & 1;
                ok = mbar_wait(lfull0 + 8 * buf, (it >> 1) & 1, abort_flag);
                if (!ok) break;
                const uint16_t *list = lists + buf * list_stride;
                const int n = nlive[buf];
                for (int c0 = 0; c0 < n && ok; c0 += T_CHUNK, ++chunk) {
                    // this chunk's accumulator: free once the epilogue has drained the chunk two before it
                    const uint32_t ab = chunk & 1u;
                    ok = mbar_wait(acce0 + 8 * ab, ((chunk >> 1) & 1u) ^ 1u, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d = tmem + ab * 128u;
                    uint32_t accumulate = 0;
                    const int c1 = min(n, c0 + T_CHUNK);
                    for (int q = c0; q < c1; ++q) {
                        if (!landed) ok = mbar_wait(full0 + 8 * slot, phase, abort_flag);
                        if (!ok) break;
                        const uint32_t ah = ring_lo + (uint32_t)slot * (T_STAGE_BYTES >> 4);
                        const int nslot = slot + 1 == T_STAGES ? 0 : slot + 1;
                        landed = umma_group<false, UMMA_IDESC_TF32_128x128>(d, ah, ah + (T_PART_BYTES >> 4), ah + 2 * (T_PART_BYTES >> 4),
                                                   ah + 3 * (T_PART_BYTES >> 4), (unsigned)list[q] >> 12, accumulate,
                                                   full0 + 8 * nslot, nslot ? phase : phase ^ 1u);
                        umma_commit(empty0 + 8 * slot);          // the slot is free when these MMAs have read it
                        if (++slot == T_STAGES) {
                            slot = 0;
                            phase ^= 1;
                        }
                    }
                    if (!ok) break;
                    umma_commit(accf0 + 8 * ab);                 // the chunk is complete when all its MMAs are
                }
                if (!ok) break;
                mbar_arrive(lempty0 + 8 * buf);
            }
        }
    } else if (warp >= 4) {
        // ---------------- epilogue: warp w owns TMEM lanes 32 (w - 4) .., one C row per thread; chunk sums are added
        // in registers with round-to-nearest, which keeps the tensor core's own accumulation runs short ----------------
        const int q = warp - 4;
        float *stage = p.stage_off ? reinterpret_cast<float *>(smem + p.stage_off) + (warp - 4) * T_STAGE_FLOATS : nullptr;
        int it = 0;
        uint32_t chunk = 0;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            ok = mbar_wait(lfull0 + 8 * buf, (it >> 1) & 1, abort_flag);
            if (!ok) break;
            const int n = nlive[buf];
            __syncwarp();
            if (lane == 0) mbar_arrive(lempty0 + 8 * buf);
            float acc[TILE_N];
#pragma unroll
            for (int j = 0; j < TILE_N; ++j) acc[j] = 0.0f;
            for (int c0 = 0; c0 < n && ok; c0 += T_CHUNK, ++chunk) {
                const uint32_t ab = chunk & 1u;
                ok = mbar_wait(accf0 + 8 * ab, (chunk >> 1) & 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int cc = 0; cc < TILE_N; cc += 32) {
                    uint32_t r[32];
                    tmem_ld_32(tmem + ((uint32_t)(q * 32) << 16) + ab * 128u + (uint32_t)cc, r);
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[cc + j] += __uint_as_float(r[j]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acce0 + 8 * ab);
            }
            if (!ok) break;
            store_row_block(acc, stage, p.C, tm * TILE_M + q * 32, tn * TILE_N, p.M, p.N, lane);
        }
    }

    if (!ok && lane == 0) atomicExch(p.status, (int)ESMM_ERR_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(T_TMEM_COLS));
}

// ---------------------------------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2): two CTAs of a cluster share one 256 x NB tile, NB = 128 or 256.  CTA r of the pair
// holds rows 128 r .. of A and columns (NB / 2) r .. of B in its own shared memory; the MMAs (M 256, N NB), issued by
// the even CTA, read both halves, and each CTA ends up with its 128 rows of the accumulator in its own tensor
// memory.  Per K block a CTA fetches 8 KB of A and NB / 32 KB of B: with NB = 256 that is the 16 KB of the
// single-CTA kernel for twice its MMA work, which is what takes operand delivery off the critical path.
// Ring: 4 stages of 48 KB (NB 128) or 3 of 64 KB (NB 256).
// Barriers: `full` lives in the even CTA and counts the bytes of both CTAs' copies (the copies carry cta_group::2
// and name the even CTA's barrier); `empty` and `acc_full` exist in both CTAs and are signalled by one
// tcgen05.commit with a CTA mask; the even CTA's `acc_empty` takes the arrivals of both CTAs' epilogue warps.
// Both CTAs build the same list of live groups from the same pattern bytes.
// ---------------------------------------------------------------------------------------------------------------
constexpr int P2_TILE_M = 256;
constexpr int P2_A_PART = 128 * 128;          // 128 rows x 32 floats
// NB: columns of the pair's tile (the N of its MMAs), 128 or 256; each CTA holds NB / 2 of them
template <int NB> struct PairCfg {
    static constexpr int B_PART = (NB / 2) * 128;                  // NB / 2 rows x 32 floats
    static constexpr int STAGE_BYTES = 2 * P2_A_PART + 2 * B_PART; // 48 KB or 64 KB
    static constexpr int STAGES = NB == 128 ? 4 : 3;
    static constexpr int EPI_WARPS = 4 * (NB / 128);               // a set of four warps per 128 columns
    static constexpr int THREADS = (4 + EPI_WARPS) * 32;
    static constexpr int TMEM_COLS = 2 * NB;                       // two accumulators
    static constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(NB >> 3) << 17) | (16u << 24);
};
struct Tf32PairMaps {
    CUtensorMap a_hi, a_lo;                   // boxes of 32 floats x 128 rows, 128-byte swizzle
    CUtensorMap b_hi, b_lo;                   // boxes of 32 floats x NB / 2 rows
};

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// the address, in the cluster's shared window, of this CTA's shared address `addr` in CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// copy into this CTA's shared memory, bytes counted on a barrier that may live in the pair's other CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// arrives on the barrier at this shared offset in both CTAs of the pair once the MMAs issued so far are complete
__device__ __forceinline__ void umma_commit_pair(uint32_t bar)
{
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"(mask)
                 : "memory");
}

struct PairItem {
    int tile, half;
    bool split;
};

// Work items of the pair kernels: whole tiles first, then the tiles of the last, partly filled wave as two items each
// (halves of the tile's live groups), so that the wave costs half a tile instead of a whole one.  Their part of C
// is zeroed by the split pass (ZeroJob) and both items add their sums.
__device__ __forceinline__ PairItem pair_item(const Tf32Params &p, int item)
{
    PairItem w;
    if (item < p.split_first) {
        w.tile = item;
        w.half = 0;
        w.split = false;
    } else {
        w.tile = p.split_first + ((item - p.split_first) >> 1);
        w.half = (item - p.split_first) & 1;
        w.split = true;
    }
    return w;
}

template <int NB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg<NB>::THREADS, 1)
esmm_joint_sgemm_tf32x3_pair_kernel(const __grid_constant__ Tf32PairMaps maps, const Tf32Params p)
{
    using Cfg = PairCfg<NB>;
    extern __shared__ __align__(1024) char smem[];
    // layout: ring (STAGES x STAGE_BYTES) | group lists (2 x cap u16) | barriers | misc
    const int list_stride = ((p.cap * 2 + 15) & ~15) / 2;
    uint16_t *lists = reinterpret_cast<uint16_t *>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + Cfg::STAGES * Cfg::STAGE_BYTES + 4 * list_stride);
    // full[4], empty[4], acc_full[2], acc_empty[2], lfull[2], lempty[2]
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + 4), accf0 = smem_u32(bars + 8),
                   acce0 = smem_u32(bars + 10), lfull0 = smem_u32(bars + 12), lempty0 = smem_u32(bars + 14);
    volatile int *nlive = reinterpret_cast<volatile int *>(bars + 16);
    volatile int *abort_flag = nlive + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(const_cast<int *>(nlive + 3));
    volatile int *noff = nlive + 4;              // [2]: where the item's part of the listed tile's groups starts
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);         // the even CTA's producer; bytes of both CTAs' copies
            mbar_init(empty0 + 8 * s, 1);        // one commit per stage, delivered to both CTAs
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(accf0 + 8 * b, 1);
            mbar_init(acce0 + 8 * b, 2 * Cfg::EPI_WARPS);   // (even CTA) the epilogue warps of both CTAs
            mbar_init(lfull0 + 8 * b, 1);
            mbar_init(lempty0 + 8 * b, Cfg::EPI_WARPS + (leader ? 2 : 1));   // producer warp, MMA thread (even CTA), epilogue warps
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(Cfg::TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                          // both CTAs' barriers exist before anything remote touches them
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const int nGroups = (p.nKB + T_GROUP_KB - 1) / T_GROUP_KB;
    bool ok = true;

    // With the wide tile, 12 warps leave 168 registers per thread and an epilogue thread keeps a 128-column row of
    // run sums: the first four warps (producer, MMA, mask, idle) hand registers over to the eight epilogue warps.
    // The instruction sits at the head of each side's own branch so that the code below it is compiled for its register allowance.
    if (warp < 4) {
    if constexpr (NB == 256) asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (warp == 2) {
        // ---------------- mask warp: live groups of the pair's tile (8 row blocks of A, 4 column blocks of B) ----------------
        int it = 0;
        for (int item = pair; item < p.num_items && ok; item += num_pairs, ++it) {
            const PairItem w = pair_item(p, item);
            const int tile = w.tile;
            const int buf = it & 1;
            ok = mbar_wait(lempty0 + 8 * buf, ((it >> 1) & 1) ^ 1, abort_flag);
            if (!ok) break;
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            uint16_t *list = lists + buf * list_stride;
            int pos = 0;
            for (int g0 = 0; g0 < nGroups; g0 += 32) {
                const int g = g0 + lane;
                unsigned live = 0;
                if (g < nGroups) {
                    if ((p.nKB & 3) == 0) {
                        // the group's four pattern bytes of a row block are one aligned word: 8 + NB / 32 independent loads
                        unsigned aw = 0, bw = 0;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int mb = tm * 8 + i, nb = tn * (NB / 32) + i;
                            if (mb < p.a_rows) aw |= __ldg(reinterpret_cast<const unsigned *>(p.a_pat + (size_t)mb * p.nKB) + g);
                            if (i < NB / 32 && nb < p.b_rows)
                                bw |= __ldg(reinterpret_cast<const unsigned *>(p.b_pat + (size_t)nb * p.nKB) + g);
                        }
                        const unsigned j = aw & bw;
                        live = ((j & 0xFFu) ? 1u : 0u) | ((j & 0xFF00u) ? 2u : 0u) | ((j & 0xFF0000u) ? 4u : 0u) |
                               ((j & 0xFF000000u) ? 8u : 0u);
                    } else {
                        unsigned au[T_GROUP_KB] = {0, 0, 0, 0}, bu[T_GROUP_KB] = {0, 0, 0, 0};
#pragma unroll 1
                        for (int i = 0; i < 8; ++i) {       // not unrolled: this warp runs on a small register allowance
                            const int mb = tm * 8 + i, nb = tn * (NB / 32) + i;
#pragma unroll
                            for (int j = 0; j < T_GROUP_KB; ++j) {
                                const int kb = g * T_GROUP_KB + j;
                                if (kb < p.nKB) {
                                    if (mb < p.a_rows) au[j] |= p.a_pat[(size_t)mb * p.nKB + kb];
                                    if (i < NB / 32 && nb < p.b_rows) bu[j] |= p.b_pat[(size_t)nb * p.nKB + kb];
                                }
                            }
                        }
#pragma unroll
                        for (int j = 0; j < T_GROUP_KB; ++j) live |= ((au[j] & bu[j]) != 0u ? 1u : 0u) << j;
                    }
                }
                const unsigned m = __ballot_sync(0xFFFFFFFFu, live != 0u);
                if (live && bounds_ok(pos + __popc(m & ((1u << lane) - 1u)) < p.cap, p.status, 50))   // checked build: site 50
                    list[pos + __popc(m & ((1u << lane) - 1u))] = (uint16_t)(g | (live << 12));
                pos += __popc(m);
            }
            if (lane == 0) {
                // a split tile: this item multiplies the first or the second half of the tile's live groups
                const int lo = w.split && w.half ? pos / 2 : 0, hi = w.split && !w.half ? pos / 2 : pos;
                noff[buf] = lo;
                nlive[buf] = hi - lo;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(lfull0 + 8 * buf);
        }
    } else if (warp == 0) {
        // ---------------- producer: this CTA's halves of the group; bytes are counted in the even CTA ----------------
        if (lane < 4) tma_prefetch_descriptor(&maps.a_hi + lane);
        int slot = 0, it = 0;
        uint32_t phase = 0;
        for (int item = pair; item < p.num_items && ok; item += num_pairs, ++it) {
            const PairItem w = pair_item(p, item);
            const int tile = w.tile;
            const int buf = it & 1;
            ok = mbar_wait(lfull0 + 8 * buf, (it >> 1) & 1, abort_flag);
            if (!ok) break;
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            const uint16_t *list = lists + buf * list_stride + noff[buf];
            const int n = nlive[buf];
            const int row0 = (lane & 2) ? tn * NB + (int)rank * (NB / 2) : tm * P2_TILE_M + (int)rank * 128;
            const uint32_t part_off = lane == 0 ? 0u : lane == 1 ? (uint32_t)P2_A_PART
                                    : lane == 2 ? 2u * P2_A_PART : 2u * P2_A_PART + Cfg::B_PART;
            for (int q = 0; q < n; ++q) {
                ok = mbar_wait(empty0 + 8 * slot, phase ^ 1, abort_flag);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
                const uint32_t full_leader = map_to_cta(full0 + 8 * slot, 0);
                if (leader && lane == 0) mbar_arrive_expect_tx(full0 + 8 * slot, 2u * Cfg::STAGE_BYTES);
                __syncwarp();
                if (lane < 4) {
                    const int k = (int)(list[q] & 0xFFFu) * (T_GROUP_KB * BK);
                    tma_load_2d_pair(smem_u32(smem) + (uint32_t)slot * Cfg::STAGE_BYTES + part_off, &maps.a_hi + lane, k, row0,
                                     full_leader);
                }
                if (++slot == Cfg::STAGES) {
                    slot = 0;
                    phase ^= 1;
                }
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(lempty0 + 8 * buf);
        }
    }
    else if (warp == 1) {
        // ---------------- MMA issue: one thread of the even CTA, for both CTAs ----------------
        if (leader && lane == 0) {
            int slot = 0, it = 0;
            uint32_t phase = 0, chunk = 0;
            bool landed = false;                         // the next group's copies were seen complete by a poll
            const uint32_t ring_lo = umma_desc_lo(smem_u32(smem));
            for (int item = pair; item < p.num_items && ok; item += num_pairs, ++it) {
                const int buf = it & 1;
                ok = mbar_wait(lfull0 + 8 * buf, (it >> 1) & 1, abort_flag);
                if (!ok) break;
                const uint16_t *list = lists + buf * list_stride + noff[buf];
                const int n = nlive[buf];
                for (int c0 = 0; c0 < n && ok; c0 += T_CHUNK, ++chunk) {
                    const uint32_t ab = chunk & 1u;
                    ok = mbar_wait(acce0 + 8 * ab, ((chunk >> 1) & 1u) ^ 1u, abort_flag);   // drained in both CTAs
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d = tmem + ab * (uint32_t)NB;
                    uint32_t accumulate = 0;
                    const int c1 = min(n, c0 + T_CHUNK);
                    for (int q = c0; q < c1; ++q) {
                        if (!landed) ok = mbar_wait(full0 + 8 * slot, phase, abort_flag);  // both CTAs' copies landed
                        if (!ok) break;
                        const uint32_t ah = ring_lo + (uint32_t)slot * (Cfg::STAGE_BYTES >> 4);
                        const int nslot = slot + 1 == Cfg::STAGES ? 0 : slot + 1;
                        landed = umma_group<true, Cfg::IDESC>(d, ah, ah + (P2_A_PART >> 4), ah + 2 * (P2_A_PART >> 4),
                                                  ah + ((2 * P2_A_PART + Cfg::B_PART) >> 4), (unsigned)list[q] >> 12,
                                                  accumulate, full0 + 8 * nslot, nslot ? phase : phase ^ 1u);
                        umma_commit_pair(empty0 + 8 * slot);
                        if (++slot == Cfg::STAGES) {
                            slot = 0;
                            phase ^= 1;
                        }
                    }
                    if (!ok) break;
                    umma_commit_pair(accf0 + 8 * ab);
                }
                if (!ok) break;
                mbar_arrive(lempty0 + 8 * buf);
            }
        }
    }
    } else {
        if constexpr (NB == 256) asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        // ---------------- epilogue: this CTA's 128 rows of the accumulator, one C row per thread ----------------
        const int q = (warp - 4) & 3, half = (warp - 4) >> 2;    // TMEM lanes 32 q .., columns 128 half ..
        float *stage = p.stage_off ? reinterpret_cast<float *>(smem + p.stage_off) + (warp - 4) * T_STAGE_FLOATS : nullptr;
        int it = 0;
        uint32_t chunk = 0;
        for (int item = pair; item < p.num_items && ok; item += num_pairs, ++it) {
            const PairItem w = pair_item(p, item);
            const int tile = w.tile;
            const int buf = it & 1;
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            ok = mbar_wait(lfull0 + 8 * buf, (it >> 1) & 1, abort_flag);
            if (!ok) break;
            const int n = nlive[buf];
            __syncwarp();
            if (lane == 0) mbar_arrive(lempty0 + 8 * buf);
            float acc[TILE_N];
#pragma unroll
            for (int j = 0; j < TILE_N; ++j) acc[j] = 0.0f;
            for (int c0 = 0; c0 < n && ok; c0 += T_CHUNK, ++chunk) {
                const uint32_t ab = chunk & 1u;
                ok = mbar_wait(accf0 + 8 * ab, (chunk >> 1) & 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int cc = 0; cc < TILE_N; cc += 32) {
                    uint32_t r[32];
                    tmem_ld_32(tmem + ((uint32_t)(q * 32) << 16) + ab * (uint32_t)NB + (uint32_t)(half * 128 + cc), r);
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[cc + j] += __uint_as_float(r[j]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(acce0 + 8 * ab, 0));
            }
            if (!ok) break;
            if (!(w.split && n == 0))     // a split tile's C was zeroed beforehand: nothing to add is nothing to do
                store_row_block(acc, stage, p.C, tm * P2_TILE_M + (int)rank * 128 + q * 32, tn * NB + half * 128, p.M, p.N,
                                lane, w.split);
        }
    }

    if (!ok && lane == 0) atomicExch(p.status, (int)ESMM_ERR_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();        // nothing of the other CTA (its barriers, shared memory, tensor memory) is touched after this
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Cfg::TMEM_COLS));
}

}  // namespace esmm

// "B offline" state of the 3xTF32 path (opaque to callers)
struct esmm_tf32x3_b {
    int K, N, Kc;            // Kc: columns kept (a multiple of 8; == K without compaction)
    int device;
    int *d_klist;            // Kc entries, or nullptr when every k is kept
    float *d_bt;             // Bt_hi (N x Kc) then Bt_lo (N x Kc)
    uint8_t *d_b_pat;        // patterns of the kept rows of B: ceil(N / 32) x Kc / 8
};

extern "C" {

void esmm_tf32x3_b_destroy(esmm_tf32x3_b *b)
{
    if (!b) return;
    cudaFree(b->d_klist);
    cudaFree(b->d_bt);
    cudaFree(b->d_b_pat);
    delete b;
}

int esmm_tf32x3_b_create(const float *d_B, int K, int N, int compact, esmm_tf32x3_b **out)
{
    using namespace esmm;
    if (!d_B || !out) return ESMM_ERR_NULL;
    *out = nullptr;
    if (K <= 0 || N <= 0 || (K & 7) || (N & 3)) return ESMM_ERR_SHAPE;
    if (((uintptr_t)d_B) & 15) return ESMM_ERR_ALIGN;
    const int nKB = K / BK, nNB = ceil_div(N, PAT_N);
    esmm_tf32x3_b *b = new esmm_tf32x3_b();
    b->K = K;
    b->N = N;
    b->Kc = K;
    int st = ESMM_OK;
    auto fail = [&](int code) {
        esmm_tf32x3_b_destroy(b);
        return code;
    };
    if (cudaGetDevice(&b->device) != cudaSuccess) return fail(record_cuda_error_text("cudaGetDevice failed"));

    // patterns of the whole of B, on the host too: they say which rows of B hold anything at all
    std::vector<uint8_t> pat((size_t)nNB * nKB);
    uint8_t *d_pat = nullptr;
    if (cudaMalloc(&d_pat, pat.size()) != cudaSuccess) return fail(record_cuda_error_text("cudaMalloc failed (B patterns)"));
    st = esmm_preprocess_b(d_B, K, N, d_pat, nullptr);
    if (st == ESMM_OK && cudaMemcpy(pat.data(), d_pat, pat.size(), cudaMemcpyDeviceToHost) != cudaSuccess)
        st = record_cuda_error_text("cudaMemcpy failed (B patterns)");
    if (st != ESMM_OK) {
        cudaFree(d_pat);
        return fail(st);
    }

    std::vector<int> klist;
    if (compact) {
        std::vector<uint8_t> any(nKB, 0);
        for (int nb = 0; nb < nNB; ++nb)
            for (int kb = 0; kb < nKB; ++kb) any[kb] |= pat[(size_t)nb * nKB + kb];
        for (int k = 0; k < K; ++k)
            if ((any[k >> 3] >> (k & 7)) & 1) klist.push_back(k);
        if (klist.empty()) klist.push_back(-1);              // B is all zero: one group of zero columns
        while (klist.size() % (T_GROUP_KB * BK)) klist.push_back(-1);   // whole fetch groups
        if ((int)klist.size() >= K)
            klist.clear();                                   // nothing to gain: keep the direct path
        else
            b->Kc = (int)klist.size();
    }
    const int Kc = b->Kc, nKBc = Kc / BK;
    if (!klist.empty()) {
        // patterns of the kept rows: bit i of block jb comes from row klist[8 jb + i]
        std::vector<uint8_t> pc((size_t)nNB * nKBc, 0);
        for (int nb = 0; nb < nNB; ++nb)
            for (int j = 0; j < Kc; ++j) {
                const int k = klist[j];
                if (k >= 0 && ((pat[(size_t)nb * nKB + (k >> 3)] >> (k & 7)) & 1)) pc[(size_t)nb * nKBc + (j >> 3)] |= 1u << (j & 7);
            }
        cudaFree(d_pat);
        d_pat = nullptr;
        if (cudaMalloc(&b->d_b_pat, pc.size()) != cudaSuccess ||
            cudaMemcpy(b->d_b_pat, pc.data(), pc.size(), cudaMemcpyHostToDevice) != cudaSuccess ||
            cudaMalloc(&b->d_klist, (size_t)Kc * sizeof(int)) != cudaSuccess ||
            cudaMemcpy(b->d_klist, klist.data(), (size_t)Kc * sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess)
            return fail(record_cuda_error_text("cudaMalloc / cudaMemcpy failed (compacted B patterns)"));
    } else {
        b->d_b_pat = d_pat;
    }

    if (cudaMalloc(&b->d_bt, (size_t)2 * N * Kc * sizeof(float)) != cudaSuccess)
        return fail(record_cuda_error_text("cudaMalloc failed (split B)"));
    dim3 grid((unsigned)ceil_div(N, 32), (unsigned)ceil_div(Kc, 32)), block(32, 8);
    esmm_tf32_split_transpose_kernel<<<grid, block>>>(d_B, K, N, b->d_klist, Kc, b->d_bt, b->d_bt + (size_t)N * Kc);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail(record_cuda_error_text(cudaGetErrorString(e)));
    *out = b;
    return ESMM_OK;
}

int esmm_tf32x3_b_live_k(const esmm_tf32x3_b *b) { return b ? b->Kc : 0; }

size_t esmm_tf32x3_workspace_bytes(int M, int K)
{
    if (M <= 0 || K <= 0) return 0;
    const size_t pat = (esmm_a_pattern_bytes(M, K, 32) + 255) & ~(size_t)255;
    return pat + (size_t)2 * M * K * sizeof(float);
}

int esmm_sgemm_joint_tf32x3(int M, const float *d_A, const esmm_tf32x3_b *b, float *d_C, void *d_workspace,
                            void *stream_)
{
    using namespace esmm;
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!d_A || !b || !d_C || !d_workspace) return ESMM_ERR_NULL;
    const int N = b->N, K = b->K, Kc = b->Kc;
    if (M <= 0) return ESMM_ERR_SHAPE;
    if (((uintptr_t)d_A | (uintptr_t)d_C) & 15) return ESMM_ERR_ALIGN;
    if (((uintptr_t)d_workspace) & 255) return ESMM_ERR_ALIGN;
    const int nKB = Kc / BK, groups = ceil_div(nKB, T_GROUP_KB);
    if (groups > 4095) return ESMM_ERR_TOO_LARGE;   // 12-bit group index in the list entries

    int dev = 0;
    ESMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev != b->device) return record_cuda_error_text("esmm_sgemm_joint_tf32x3: B was prepared on another device");
    // per device, once: SM count and the opt-in to the kernels' dynamic shared memory (not thread-safe by design:
    // like the rest of the library, one host thread per device)
    static int sms_of[64];
    static unsigned char opted[64];
    if (dev < 0 || dev >= 64) return record_cuda_error_text("esmm_sgemm_joint_tf32x3: device ordinal out of range");
    if (!sms_of[dev]) ESMM_CUDA_TRY(cudaDeviceGetAttribute(&sms_of[dev], cudaDevAttrMultiProcessorCount, dev));
    const int sms = sms_of[dev];
    if (!opted[dev]) {
        ESMM_CUDA_TRY(cudaFuncSetAttribute(esmm_joint_sgemm_tf32x3_pair_kernel<128>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
        ESMM_CUDA_TRY(cudaFuncSetAttribute(esmm_joint_sgemm_tf32x3_pair_kernel<256>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
        ESMM_CUDA_TRY(cudaFuncSetAttribute(esmm_joint_sgemm_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           SMEM_LIMIT));
        opted[dev] = 1;
    }

    // Which kernel: the one with the smallest estimated time per SM, in units of one 128 x 128 tile's tensor time.
    // A 256 x 256 tile is two units per SM at the tensor rate; a 256 x 128 tile one unit at 1.19 and a 128 x 128 tile
    // on one CTA one unit at 1.24 (measured at 3072^3, where all three fill their waves alike); a pair kernel's
    // partly filled last wave counts half when its tiles can be split along K.  Small problems therefore take the
    // smaller tiles (1024^2 x 4096: 97 us on 256 x 128 pairs, 105 us on single CTAs, 137 us on 256 x 256 pairs), large
    // ones the 256 x 256 pairs.  ESMM_TF32_PAIR = 0 | 128 | 256 overrides the choice.
    const int pair_env = tuning_get("TF32_PAIR", -1);
    const int pairs_all = std::max(1, sms / 2);
    const bool can_split = groups >= 12 && tuning_get("TF32_SPLIT_LAST", 1) != 0;
    int nb = 0;
    {
        auto pair_waves = [&](int tiles) {
            const int full = tiles / pairs_all, left = tiles % pairs_all;
            if (!left) return (double)full;
            return full + ((full > 0 && 2 * left <= pairs_all && can_split) ? 0.5 : 1.0);
        };
        const double c1 = 1.24 * ceil_div(ceil_div(M, TILE_M) * ceil_div(N, TILE_N), sms);
        const double c128 = 1.19 * pair_waves(ceil_div(M, P2_TILE_M) * ceil_div(N, 128));
        const double c256 = 2.0 * pair_waves(ceil_div(M, P2_TILE_M) * ceil_div(N, 256));
        if (M >= 192) {
            // near-ties go to the larger tile (512 x 11008 x 4096: 0.190 ms on 256 x 256 pairs, 0.202 on 256 x 128)
            nb = (N >= 192 && c256 <= 1.05 * c128 && c256 <= 1.05 * c1) ? 256 : (c128 <= c1 ? 128 : 0);
            if (pair_env == 0 || pair_env == 128 || (pair_env == 256 && N >= 192)) nb = pair_env;
            if (pair_env == 256 && N < 192) nb = 128;
        }
    }

    // workspace (sized for the uncompacted K): A patterns | A_hi | A_lo, all of the kept columns only
    uint8_t *a_pat = static_cast<uint8_t *>(d_workspace);
    float *a_hi = reinterpret_cast<float *>(a_pat + ((esmm_a_pattern_bytes(M, K, 32) + 255) & ~(size_t)255));
    float *a_lo = a_hi + (size_t)M * Kc;

    Tf32Params p;
    memset(&p, 0, sizeof p);
    p.M = M;
    p.N = N;
    p.K = Kc;
    p.nKB = nKB;
    p.cap = groups + 32;
    p.a_rows = ceil_div(M, 32);
    p.b_rows = ceil_div(N, PAT_N);
    p.tiles_m = ceil_div(M, nb ? P2_TILE_M : TILE_M);
    p.tiles_n = ceil_div(N, nb ? nb : TILE_N);
    p.num_tiles = p.tiles_m * p.tiles_n;
    p.num_items = p.num_tiles;
    p.split_first = p.num_tiles;
    p.a_pat = a_pat;
    p.b_pat = b->d_b_pat;
    p.C = d_C;
    p.status = device_status_ptr();
    if (!p.status) return ESMM_ERR_CUDA;

    // The last wave of a pair kernel: `left` tiles for `pairs` pairs.  Where two halves per tile still fit into one
    // wave, those tiles are split along K (their part of C is zeroed by the split pass below).
    const int pairs = std::max(1, std::min(pairs_all, p.num_tiles));
    ZeroJob zj;
    memset(&zj, 0, sizeof zj);
    if (nb) {
        const int left = p.num_tiles % pairs;
        if (left > 0 && p.num_tiles > pairs && 2 * left <= pairs && can_split) {
            p.split_first = p.num_tiles - left;
            p.num_items = p.num_tiles + left;
            zj.C = d_C;
            zj.N = N;
            zj.tiles_m = p.tiles_m;
            zj.tiles_n = p.tiles_n;
            zj.nb = nb;
            zj.first = p.split_first;
            zj.count = left;
        }
    }

    // shared memory of the product kernel, checked before anything is launched
    const size_t ring = nb == 128   ? (size_t)PairCfg<128>::STAGE_BYTES * PairCfg<128>::STAGES
                        : nb == 256 ? (size_t)PairCfg<256>::STAGE_BYTES * PairCfg<256>::STAGES
                                    : (size_t)T_STAGES * T_STAGE_BYTES;
    const int epi_warps = nb == 256 ? PairCfg<256>::EPI_WARPS : 4;
    size_t smem = ring + 2 * ((p.cap * 2 + 15) & ~15) + 16 * 8 + 32;
    if (smem > (size_t)SMEM_LIMIT) return ESMM_ERR_TOO_LARGE;
    const size_t staging = (size_t)epi_warps * T_STAGE_FLOATS * 4;
    if (smem + staging <= (size_t)SMEM_LIMIT && tuning_get("TF32_DIRECT_STORES", 0) == 0) {
        p.stage_off = (int)smem;                               // a multiple of 16
        smem += staging;
    }

    const float *bt_hi = b->d_bt, *bt_lo = b->d_bt + (size_t)N * Kc;
    const CUtensorMapL2promotion l2 = CU_TENSOR_MAP_L2_PROMOTION_L2_128B;
    const CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B;
    const uint32_t box_k = T_GROUP_KB * BK, b_rows_box = nb ? nb / 2 : TILE_N;
    CUtensorMap m_a_hi, m_a_lo, m_b_hi, m_b_lo;
    int st = make_map_2d(&m_a_hi, a_hi, (uint64_t)Kc, (uint64_t)M, box_k, 128, sw, l2);
    if (!st) st = make_map_2d(&m_a_lo, a_lo, (uint64_t)Kc, (uint64_t)M, box_k, 128, sw, l2);
    if (!st) st = make_map_2d(&m_b_hi, bt_hi, (uint64_t)Kc, (uint64_t)N, box_k, b_rows_box, sw, l2);
    if (!st) st = make_map_2d(&m_b_lo, bt_lo, (uint64_t)Kc, (uint64_t)N, box_k, b_rows_box, sw, l2);
    if (st) return st;

    {
        dim3 grid((unsigned)ceil_div(Kc, 512), (unsigned)(ceil_div(M, 32) + 8 * zj.count));
        esmm_tf32_split_pattern_kernel<<<grid, 256, 0, stream>>>(d_A, M, K, b->d_klist, Kc, a_hi, a_lo, a_pat, zj);
        ESMM_CUDA_TRY(cudaGetLastError());
    }
    if (nb) {
        Tf32PairMaps maps;
        maps.a_hi = m_a_hi;
        maps.a_lo = m_a_lo;
        maps.b_hi = m_b_hi;
        maps.b_lo = m_b_lo;
        if (nb == 128)
            esmm_joint_sgemm_tf32x3_pair_kernel<128><<<2 * pairs, PairCfg<128>::THREADS, smem, stream>>>(maps, p);
        else
            esmm_joint_sgemm_tf32x3_pair_kernel<256><<<2 * pairs, PairCfg<256>::THREADS, smem, stream>>>(maps, p);
    } else {
        Tf32Maps maps;
        maps.a_hi = m_a_hi;
        maps.a_lo = m_a_lo;
        maps.b_hi = m_b_hi;
        maps.b_lo = m_b_lo;
        esmm_joint_sgemm_tf32x3_kernel<<<std::min(sms, p.num_tiles), T_THREADS, smem, stream>>>(maps, p);
    }
    ESMM_CUDA_TRY(cudaGetLastError());
    return ESMM_OK;
}

}  // extern "C"
