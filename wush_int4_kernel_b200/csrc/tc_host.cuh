// Host-side TMA descriptor helper shared by the kernels that stage tiles with
// cp.async.bulk.tensor.  The driver's encoder is reached through the runtime's entry-point
// query (resolved once in wush_init), so the library does not link against libcuda.
#pragma once
#include <cuda.h>
#include <stdint.h>

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
    // A decode call re-uses the same few (pointer, shape) combinations step after step; encoding costs a
    // microsecond or two each, which an eager call of a 15 us kernel notices.  Small per-thread cache; a
    // descriptor depends on nothing but these arguments.
    struct Entry { const void* base; uint64_t inner, rows; uint32_t box_inner, box_rows; int dt, elem_bytes, swz; bool valid; CUtensorMap map; };
    static thread_local Entry cache[32] = {};
    uint64_t h = (uint64_t)(uintptr_t)base * 0x9E3779B97F4A7C15ull;
    h ^= (inner * 0xC2B2AE3D27D4EB4Full) ^ (rows * 0x165667B19E3779F9ull) ^ ((uint64_t)box_inner << 40) ^ ((uint64_t)box_rows << 20) ^
         ((uint64_t)dt << 8) ^ (uint64_t)swz;
    Entry& slot = cache[(h >> 32) & 31];
    if (slot.valid && slot.base == base && slot.inner == inner && slot.rows == rows && slot.box_inner == box_inner &&
        slot.box_rows == box_rows && slot.dt == (int)dt && slot.elem_bytes == elem_bytes && slot.swz == (int)swz) {
        *map = slot.map;
        return WUSH_OK;
    }
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {inner * (uint64_t)elem_bytes};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    if (!g_encode_tiled) return fail(WUSH_ERR_CUDA, "tensor-map encoder not resolved (wush_init not run?)");
    CUresult r = g_encode_tiled(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(WUSH_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    slot = Entry{base, inner, rows, box_inner, box_rows, (int)dt, elem_bytes, (int)swz, true, *map};
    return WUSH_OK;
}

}  // namespace wush
