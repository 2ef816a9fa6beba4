// Tensor map over the dense operand B for TMA gather4 loads: B is described as a 2-D fp32 tensor
// (columns innermost, extent N; rows extent K, pitch ldb), and one cp.async.bulk.tensor...tile::gather4
// brings four arbitrary rows of it, `box_cols` columns wide, into consecutive rows of shared memory.
// Columns beyond N are filled with zeros without touching memory.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace cutespmm {

// cuTensorMapEncodeTiled is looked up through the runtime: the library does not link libcuda.
inline cudaError_t make_b_tensor_map(CUtensorMap *out, const float *B, uint64_t N, uint64_t K, uint64_t ldb, uint32_t box_cols,
                                     CUtensorMapSwizzle swizzle)
{
    using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                       const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeTiledFn enc = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    if (!enc) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {N, K};
    const cuuint64_t strides[1] = {ldb * sizeof(float)};
    const cuuint32_t box[2] = {box_cols, 1}, estr[2] = {1, 1};
    if (enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(B), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    return cudaSuccess;
}

}  // namespace cutespmm
