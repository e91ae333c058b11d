// Host helper: encode 2-D tiled TMA descriptors without linking libcuda (the driver entry
// point is looked up through the runtime, so the library still loads on a machine with no
// driver).  Stands in for the reference's create_tma_desc_A (src/fp16.cu:177-219).
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace b200spmm {

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
        if (q != cudaDriverEntryPointSuccess) return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// 2-D row-major tensor [rows][row_bytes / elt] with row pitch `pitch_bytes`; box
// {box_inner elements, box_rows}.  Out-of-range elements read as zero.  Returns false on failure.
inline bool encode_2d(CUtensorMap *map, CUtensorMapDataType type, const void *base, uint64_t inner_elems,
                      uint64_t rows, uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows,
                      CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {inner_elems, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, type, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace b200spmm
