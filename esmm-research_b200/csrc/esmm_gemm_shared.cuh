// Pieces shared by the two joint-sparse GEMM kernels (row-major A and packed A).
#pragma once

#include <cstdio>
#include <cstdlib>

#include "esmm_common.cuh"

namespace esmm {

constexpr int TILE_M = 128;
constexpr int TILE_N = 128;
constexpr int GROUP_M = 8;         // tile rows per raster group
constexpr int SMEM_LIMIT = 232448; // 227 KB per CTA on sm_100

#ifdef __CUDACC__
// Tiles are walked in groups of `group_m` tile rows (GROUP_M unless the launch says otherwise), column by column
// inside a group, so that the CTAs running at the same time share a compact set of A row panels and B column panels
// in L2.  A pass over a group touches the group's A panels and all of B, and B comes from DRAM again for every group.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int &tm, int &tn, int group_m = GROUP_M)
{
    const int per_group = group_m * tiles_n;
    const int group = tile / per_group;
    const int first_m = group * group_m;
    const int gsize = min(tiles_m - first_m, group_m);
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

#endif  // __CUDACC__

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn()
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
inline int make_map_2d(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer,
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

// 3-D FP32 tensor (d0 fastest, contiguous; strides of d1 and d2 in bytes), box b0 x b1 x b2.
inline int make_map_3d(CUtensorMap *map, const void *base, uint64_t d0, uint64_t d1, uint64_t d2,
                       uint64_t stride1, uint64_t stride2, uint32_t b0, uint32_t b1, uint32_t b2)
{
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return record_cuda_error_text("cuTensorMapEncodeTiled entry point not available");
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1, stride2};
    cuuint32_t box[3] = {b0, b1, b2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char buf[96];
        snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled (3-D) failed with CUresult %d", (int)r);
        return record_cuda_error_text(buf);
    }
    return ESMM_OK;
}

}  // namespace esmm
