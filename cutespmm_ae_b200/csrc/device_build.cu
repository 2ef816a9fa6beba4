// Device side of cutespmm_plan_create_device: packs CSR columns and values that already live on the GPU into the
// interleaved (column, value) pairs the row kernel streams, and checks the column range on the way.  The
// reference preprocesses on the host only (HRPB, data.cu:80-335) and its caller uploads the result; with the
// nonzeros already on the device (a graph built there, the output of another kernel) that round trip is the
// dominant cost of creating a plan.
#include <cuda_runtime.h>

#include <cstdint>

#include "device_plan.hpp"
#include "plan.hpp"

namespace cutespmm {

namespace {

constexpr unsigned kFullMask = 0xffffffffu;

// ---- panel analysis: the distinct columns of every 16-row panel, ascending --------------------------------------
// The device counterpart of HRPB's per-panel column census (reference data.cu:116-209, a K-sized flag array per
// thread): one block per panel sorts the panel's column indices in shared memory (bitonic) and compacts the distinct
// ones into acols[row_ptr[first row of the panel] ...] -- a panel has at most as many distinct columns as nonzeros,
// so the panel's own nonzero range is room enough.  Panels with more than kDevPanelMax nonzeros are left out
// (ncols = kPanelTooLarge): they hold a long row and stay with the row kernel.
__global__ void __launch_bounds__(256) panel_columns_kernel(const uint32_t *__restrict__ row_ptr, const uint2 *__restrict__ pairs, uint32_t M,
                                                            uint32_t num_panels, uint32_t *__restrict__ ncols,
                                                            uint32_t *__restrict__ acols)
{
    extern __shared__ uint32_t buf[];  // kDevPanelMax column indices
    __shared__ uint32_t warp_sums[8];
    __shared__ uint32_t running;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (uint32_t q = blockIdx.x; q < num_panels; q += gridDim.x) {
        const uint32_t r0 = q * kPanelRows, r1 = min(M, r0 + kPanelRows);
        const uint32_t j0 = __ldg(row_ptr + r0), n = __ldg(row_ptr + r1) - j0;
        if (n == 0 || n > kDevPanelMax) {
            if (tid == 0) ncols[q] = n == 0 ? 0u : kPanelTooLarge;
            continue;
        }
        uint32_t size = 32;
        while (size < n) size <<= 1;
        for (uint32_t i = tid; i < size; i += blockDim.x) buf[i] = i < n ? __ldg(&pairs[j0 + i].x) : 0xffffffffu;
        if (tid == 0) running = 0;
        __syncthreads();
        for (uint32_t k = 2; k <= size; k <<= 1)
            for (uint32_t j = k >> 1; j > 0; j >>= 1) {
                for (uint32_t i = tid; i < size; i += blockDim.x) {
                    const uint32_t x = i ^ j;
                    if (x > i) {
                        const uint32_t a = buf[i], b = buf[x];
                        if ((a > b) == ((i & k) == 0)) {
                            buf[i] = b;
                            buf[x] = a;
                        }
                    }
                }
                __syncthreads();
            }
        // compact the distinct values, in order: rank = number of distinct values in front
        for (uint32_t base = 0; base < n; base += blockDim.x) {
            const uint32_t i = base + tid;
            const bool first = i < n && (i == 0 || buf[i] != buf[i - 1]);
            const unsigned ballot = __ballot_sync(kFullMask, first);
            if (lane == 0) warp_sums[warp] = __popc(ballot);
            __syncthreads();
            uint32_t off = running;
            for (uint32_t w = 0; w < warp; ++w) off += warp_sums[w];
            if (first) acols[j0 + off + __popc(ballot & ((1u << lane) - 1u))] = buf[i];
            __syncthreads();
            if (tid == 0) {
                uint32_t t = 0;
                for (uint32_t w = 0; w < blockDim.x / 32; ++w) t += warp_sums[w];
                running += t;
            }
            __syncthreads();
        }
        if (tid == 0) ncols[q] = running;
        __syncthreads();
    }
}

// maxcol[q] = largest column index among the nonzeros of 16-row panel q (0 when it has none); one warp per panel
__global__ void __launch_bounds__(256) panel_max_col_kernel(const uint32_t *__restrict__ row_ptr, const uint2 *__restrict__ pairs, uint32_t M,
                                                            uint32_t num_panels, uint32_t *__restrict__ maxcol)
{
    const uint32_t lane = threadIdx.x & 31, warps = gridDim.x * (blockDim.x / 32);
    for (uint32_t q = blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5); q < num_panels; q += warps) {
        const uint32_t r0 = q * kPanelRows, r1 = min(M, r0 + kPanelRows);
        const uint32_t j0 = __ldg(row_ptr + r0), j1 = __ldg(row_ptr + r1);
        uint32_t m = 0;
        for (uint32_t j = j0 + lane; j < j1; j += 32) m = max(m, __ldg(&pairs[j].x));
        for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(kFullMask, m, o));
        if (lane == 0) maxcol[q] = m;
    }
}

// position of (row r, column c) of a 16 x 8 brick in its record, in mma.m16n8k8 A-fragment order (plan.hpp)
__device__ __forceinline__ uint32_t frag_index(uint32_t r, uint32_t c) { return ((r & 7u) * 4u + (c & 3u)) * 4u + (r >> 3) + 2u * (c >> 2); }

// ---- brick records of the panels routed to the tensor-core kernel ----------------------------------------------
// One warp per brick panel: the lanes write the panel's column list (8 per slot) and the record headers, then lane r
// walks row r of the panel in storage order and drops every value into its brick (duplicates of one position add up
// in storage order, as in the host builder).  The records were zeroed beforehand.
__global__ void __launch_bounds__(128) brick_fill_kernel(const uint32_t *__restrict__ row_ptr, const uint2 *__restrict__ pairs, uint32_t M,
                                                         const uint32_t *__restrict__ which, const uint32_t *__restrict__ first_slot,
                                                         const uint32_t *__restrict__ last_slot, uint32_t num_brick_panels,
                                                         const uint32_t *__restrict__ ncols, const uint32_t *__restrict__ acols,
                                                         uint32_t *__restrict__ bcols, uint32_t *__restrict__ brecs)
{
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warps = gridDim.x * (blockDim.x / 32);
    for (uint32_t i = blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5); i < num_brick_panels; i += warps) {
        const uint32_t q = __ldg(which + i), nc = __ldg(ncols + q);
        const uint32_t r0 = q * kPanelRows, j0 = __ldg(row_ptr + r0);
        const uint32_t *ac = acols + j0;
        const uint32_t f = __ldg(first_slot + i), nb = __ldg(last_slot + i) - f, nslots = (nb + 3) / 4 * 4;
        for (uint32_t c = lane; c < nslots * kBrickCols; c += 32) bcols[(size_t)f * kBrickCols + c] = ac[min(c, nc - 1)];
        for (uint32_t b = lane; b < nb; b += 32) {
            uint32_t *rec = brecs + (size_t)(f + b) * kBrickRecWords;
            rec[4] = b + 1 == nb ? 1u : 0u;
            rec[5] = q;
        }
        __syncwarp();
        const uint32_t r = r0 + lane;
        if (lane < kPanelRows && r < M) {
            const uint32_t je = __ldg(row_ptr + r + 1);
            for (uint32_t j = __ldg(row_ptr + r); j < je; ++j) {
                const uint2 pr = __ldg(pairs + j);
                const uint32_t col = pr.x;
                uint32_t lo = 0, hi = nc;  // first position with ac[pos] >= col (the column is in the list)
                while (lo < hi) {
                    const uint32_t mid = (lo + hi) >> 1;
                    if (ac[mid] < col) lo = mid + 1; else hi = mid;
                }
                uint32_t *rec = brecs + (size_t)(f + lo / kBrickCols) * kBrickRecWords;
                const uint32_t bit = lane * kBrickCols + lo % kBrickCols;
                const uint32_t old = atomicOr(&rec[bit >> 5], 1u << (bit & 31));  // rows 4k .. 4k+3 share a word of the map
                float *slot = reinterpret_cast<float *>(rec + kBrickRecHeaderWords + frag_index(lane, lo % kBrickCols));
                const float v = __uint_as_float(pr.y);
                *slot = ((old >> (bit & 31)) & 1u) ? *slot + v : v;
            }
        }
        __syncwarp();
    }
}

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

// pairs[j].value = vals[j]: new values for an unchanged pattern.
__global__ void __launch_bounds__(256) set_values_kernel(uint2 *__restrict__ pairs, const float *__restrict__ vals, uint64_t nnz)
{
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < nnz; j += stride) pairs[j].y = __float_as_uint(__ldcs(vals + j));
}

}  // namespace

cudaError_t launch_set_values(void *pairs, const float *vals, uint64_t nnz, int sm_count, cudaStream_t s)
{
    if (nnz == 0) return cudaSuccess;
    const uint64_t want = (nnz + 255) / 256;
    const uint32_t blocks = (uint32_t)(want < (uint64_t)sm_count * 8 ? want : (uint64_t)sm_count * 8);
    set_values_kernel<<<blocks, 256, 0, s>>>(static_cast<uint2 *>(pairs), vals, nnz);
    return cudaGetLastError();
}

cudaError_t launch_pack_pairs(const uint32_t *cols, const float *vals, void *pairs, uint64_t nnz, uint32_t K, uint32_t *bad, int sm_count,
                              cudaStream_t s)
{
    const uint64_t want = (nnz + 2 + 255) / 256;
    const uint32_t blocks = (uint32_t)(want < (uint64_t)sm_count * 8 ? want : (uint64_t)sm_count * 8);
    pack_pairs_kernel<<<blocks ? blocks : 1, 256, 0, s>>>(cols, vals, static_cast<uint2 *>(pairs), nnz, K, bad);
    return cudaGetLastError();
}

cudaError_t launch_panel_columns(const uint32_t *row_ptr, const void *pairs, uint32_t M, uint32_t num_panels, uint32_t *ncols,
                                 uint32_t *acols, int sm_count, cudaStream_t s)
{
    if (num_panels == 0) return cudaSuccess;
    const uint32_t blocks = num_panels < (uint32_t)sm_count * 16 ? num_panels : (uint32_t)sm_count * 16;
    panel_columns_kernel<<<blocks, 256, kDevPanelMax * sizeof(uint32_t), s>>>(row_ptr, static_cast<const uint2 *>(pairs), M, num_panels,
                                                                              ncols, acols);
    return cudaGetLastError();
}

cudaError_t launch_panel_max_col(const uint32_t *row_ptr, const void *pairs, uint32_t M, uint32_t num_panels, uint32_t *maxcol, int sm_count,
                                 cudaStream_t s)
{
    if (num_panels == 0) return cudaSuccess;
    const uint32_t want = (num_panels + 7) / 8;
    const uint32_t blocks = want < (uint32_t)sm_count * 8 ? want : (uint32_t)sm_count * 8;
    panel_max_col_kernel<<<blocks, 256, 0, s>>>(row_ptr, static_cast<const uint2 *>(pairs), M, num_panels, maxcol);
    return cudaGetLastError();
}

cudaError_t launch_brick_fill(const uint32_t *row_ptr, const void *pairs, uint32_t M, const uint32_t *which,
                              const uint32_t *first_slot, const uint32_t *last_slot, uint32_t num_brick_panels, const uint32_t *ncols,
                              const uint32_t *acols, uint32_t *bcols, uint32_t *brecs, int sm_count, cudaStream_t s)
{
    if (num_brick_panels == 0) return cudaSuccess;
    const uint32_t want = (num_brick_panels + 3) / 4;
    const uint32_t blocks = want < (uint32_t)sm_count * 16 ? want : (uint32_t)sm_count * 16;
    brick_fill_kernel<<<blocks, 128, 0, s>>>(row_ptr, static_cast<const uint2 *>(pairs), M, which, first_slot, last_slot, num_brick_panels,
                                             ncols, acols, bcols, brecs);
    return cudaGetLastError();
}

}  // namespace cutespmm
