// tma_host.hpp -- host-side construction of 2-D TMA tensor maps (cuTensorMapEncodeTiled through the runtime's driver
// entry point, so the library does not link libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "backend.hpp"

namespace vqb {

inline CUtensorMap make_tensor_map_2d(const float *ptr, unsigned long long inner, unsigned long long rows, unsigned box_inner,
                                      unsigned box_rows, CUtensorMapSwizzle swizzle)
{
    typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                      const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    if (!fn) throw Error(100, "cuTensorMapEncodeTiled is not available from this driver");
    CUtensorMap m;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)inner * sizeof(float)};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw Error(100, "cuTensorMapEncodeTiled failed (" + std::to_string((int)r) + ")");
    return m;
}

} // namespace vqb
