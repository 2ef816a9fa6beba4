// Device side of cutespmm_plan_create_device: packs CSR columns and values that already live on the GPU into the
// interleaved (column, value) pairs the row kernel streams, and checks the column range on the way.  The
// reference preprocesses on the host only (HRPB, data.cu:80-335) and its caller uploads the result; with the
// nonzeros already on the device (a graph built there, the output of another kernel) that round trip is the
// dominant cost of creating a plan.
#include <cuda_runtime.h>

#include <cstdint>

#include "device_plan.hpp"

namespace cutespmm {

namespace {

__global__ void __launch_bounds__(256) pack_pairs_kernel(const uint32_t *__restrict__ cols, const float *__restrict__ vals, uint2 *__restrict__ pairs,
                                                         uint64_t nnz, uint32_t K, uint32_t *__restrict__ bad)
{
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    bool out_of_range = false;
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < nnz + 2; j += stride) {
        if (j < nnz) {
            const uint32_t c = __ldcs(cols + j);
            out_of_range |= c >= K;
            pairs[j] = make_uint2(c, __float_as_uint(__ldcs(vals + j)));
        } else {
            pairs[j] = make_uint2(0u, 0u);  // the slack the tile copies may read behind the last pair
        }
    }
    if (__any_sync(0xffffffffu, out_of_range) && (threadIdx.x & 31) == 0) atomicOr(bad, 1u);
}

}  // namespace

cudaError_t launch_pack_pairs(const uint32_t *cols, const float *vals, void *pairs, uint64_t nnz, uint32_t K, uint32_t *bad, int sm_count,
                              cudaStream_t s)
{
    const uint64_t want = (nnz + 2 + 255) / 256;
    const uint32_t blocks = (uint32_t)(want < (uint64_t)sm_count * 8 ? want : (uint64_t)sm_count * 8);
    pack_pairs_kernel<<<blocks ? blocks : 1, 256, 0, s>>>(cols, vals, static_cast<uint2 *>(pairs), nnz, K, bad);
    return cudaGetLastError();
}

}  // namespace cutespmm
