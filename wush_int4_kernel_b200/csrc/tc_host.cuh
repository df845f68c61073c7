// Host-side TMA descriptor helper shared by the kernels that stage tiles with
// cp.async.bulk.tensor.  The driver's encoder is reached through the runtime's entry-point
// query (resolved once in wush_init), so the library does not link against libcuda.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace wush {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
extern EncodeTiledFn g_encode_tiled;
int resolve_tensor_map_encoder();

// 2-D row-major tensor (rows x inner elements), box (box_rows x box_inner); rows and columns
// outside the tensor read as zero.
inline int make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t inner,
                       uint64_t rows, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swz)
{
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {inner * (uint64_t)elem_bytes};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    if (!g_encode_tiled) return fail(WUSH_ERR_CUDA, "tensor-map encoder not resolved (wush_init not run?)");
    CUresult r = g_encode_tiled(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(WUSH_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return WUSH_OK;
}

}  // namespace wush
