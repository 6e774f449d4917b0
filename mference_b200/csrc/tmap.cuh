// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled) without linking libcuda: the driver entry point
// is looked up at run time, so the library still loads on a machine that has no GPU driver.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace mfb {

// Tiled tensor map of `rank` (<= 3) dimensions.  dims / box in elements, innermost first; strides in bytes for
// dimensions 1 .. rank-1 (multiples of 16).  Returns MFB_OK or MFB_ERR_CUDA with the error text set.
inline int32_t encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t rank, const void* base,
                                 const uint64_t* dims, const uint64_t* strides, const uint32_t* box,
                                 CUtensorMapSwizzle swizzle) {
    typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static encode_fn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
        MFB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &found));
        MFB_REQUIRE(sym != nullptr && found == cudaDriverEntryPointSuccess, MFB_ERR_CUDA,
                    "cuTensorMapEncodeTiled is not available in this driver");
        fn = reinterpret_cast<encode_fn>(sym);
    }
    cuuint64_t gdims[3] = {1, 1, 1}, gstrides[2] = {16, 16};
    cuuint32_t gbox[3] = {1, 1, 1}, estr[3] = {1, 1, 1};
    for (uint32_t i = 0; i < rank; ++i) { gdims[i] = dims[i]; gbox[i] = box[i]; }
    for (uint32_t i = 0; i + 1 < rank; ++i) gstrides[i] = strides[i];
    const CUresult r = fn(map, dtype, rank, const_cast<void*>(base), gdims, gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with code %d", (int)r);
        return MFB_ERR_CUDA;
    }
    return MFB_OK;
}

}  // namespace mfb
