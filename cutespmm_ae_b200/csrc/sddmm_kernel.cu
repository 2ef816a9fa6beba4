// SDDMM over the sparsity pattern of a plan: for every stored nonzero (r, c) of A
//
//        out[j] = (scale ? A[r][c] : 1) * sum_n X[r][n] * Y[c][n]
//
// the "edge feature" operator that accompanies SpMM in a graph layer (the reference tree carries it as
// TC-GNN's forward_ef, TC-GNN_ATC23/TCGNN_conv/TCGNN.cpp:265, and its own kernels do not have it), and
// the gradient of SpMM with respect to the values of A (dA = SDDMM(dC, B)).  Like the row kernel it is
// bound by gathering one row of Y per nonzero: a warp owns a row of A, keeps its 128-column slice of
// X[r] in registers, and handles four nonzeros at a time, eight lanes per nonzero, so that a row of Y
// is four 128-byte requests and a dot product needs three shuffles.  Long rows are taken chunk by
// chunk from the plan's work list (no partial sums are needed: every nonzero has its own output).
#include <cuda_runtime.h>

#include <cstdint>

#include "device_plan.hpp"
#include "plan.hpp"

namespace cutespmm {

namespace {

constexpr int kWarps = 8;
constexpr unsigned kFull = 0xffffffffu;

// One pass over columns [c0, c0 + 128) of X and Y for the nonzeros [j0, j1) of `row`.
// first: this is the first pass (write the result); otherwise add to what the earlier passes wrote.
__device__ __forceinline__ void sddmm_span(const SddmmArgs &a, uint32_t row, uint32_t j0, uint32_t j1, uint32_t c0, bool first, int lane)
{
    const int sub = lane & 7, grp = lane >> 3;  // eight lanes per nonzero, four nonzeros per step
    const uint2 *pairs = reinterpret_cast<const uint2 *>(a.pairs);
    float4 x[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t c = c0 + (uint32_t)(sub + 8 * i) * 4;
        x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < a.N) {
            const float *px = a.X + (uint64_t)row * a.ldx + c;
            if (a.vec4 && c + 4 <= a.N) x[i] = __ldg(reinterpret_cast<const float4 *>(px));
            else {
                x[i].x = __ldg(px);
                if (c + 1 < a.N) x[i].y = __ldg(px + 1);
                if (c + 2 < a.N) x[i].z = __ldg(px + 2);
                if (c + 3 < a.N) x[i].w = __ldg(px + 3);
            }
        }
    }
    for (uint32_t j = j0; j < j1; j += 4) {
        const uint32_t mine = j + grp;
        const bool act = mine < j1;
        uint2 pr = make_uint2(0u, 0u);
        if (act) pr = __ldg(pairs + mine);  // the eight lanes of a group read one address
        float s = 0.f;
        if (act) {
            const float *py = a.Y + (uint64_t)pr.x * a.ldy + c0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t c = (uint32_t)(sub + 8 * i) * 4;
                if (c0 + c < a.N) {
                    float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (a.vec4 && c0 + c + 4 <= a.N) y = __ldg(reinterpret_cast<const float4 *>(py + c));
                    else {
                        y.x = __ldg(py + c);
                        if (c0 + c + 1 < a.N) y.y = __ldg(py + c + 1);
                        if (c0 + c + 2 < a.N) y.z = __ldg(py + c + 2);
                        if (c0 + c + 3 < a.N) y.w = __ldg(py + c + 3);
                    }
                    s = fmaf(x[i].x, y.x, s);
                    s = fmaf(x[i].y, y.y, s);
                    s = fmaf(x[i].z, y.z, s);
                    s = fmaf(x[i].w, y.w, s);
                }
            }
        }
        s += __shfl_xor_sync(kFull, s, 4);
        s += __shfl_xor_sync(kFull, s, 2);
        s += __shfl_xor_sync(kFull, s, 1);
        if (act && sub == 0) {
            if (a.scale) s *= __uint_as_float(pr.y);
            a.out[mine] = first ? s : a.out[mine] + s;
        }
    }
}

__global__ void __launch_bounds__(kWarps * 32) sddmm_kernel(SddmmArgs a)
{
    const int lane = threadIdx.x & 31;
    const uint32_t gw = blockIdx.x * kWarps + (threadIdx.x >> 5), nw = gridDim.x * kWarps;
    for (uint32_t c0 = 0; c0 < a.N; c0 += 128) {
        // chunks of long rows (row, j0, j1, slot): the largest items first
        for (uint32_t c = gw; c < a.num_chunks; c += nw) {
            const uint4 ck = __ldg(reinterpret_cast<const uint4 *>(a.chunks) + c);
            sddmm_span(a, ck.x, ck.y, ck.z, c0, c0 == 0, lane);
        }
        // every other row: a warp takes the rows of the tiles in turn
        for (uint32_t t = blockIdx.x; t < a.num_tiles; t += gridDim.x) {
            const uint4 d = __ldg(reinterpret_cast<const uint4 *>(a.tiles) + t);  // row_begin, row_end, pair_begin, pair_end
            for (uint32_t r = d.x + (threadIdx.x >> 5); r < d.y; r += kWarps) {
                const uint32_t j0 = __ldg(a.row_ptr + r), j1 = __ldg(a.row_ptr + r + 1);
                if (j1 > j0) sddmm_span(a, r, j0, j1, c0, c0 == 0, lane);
            }
        }
    }
}

}  // namespace

cudaError_t launch_sddmm(const SddmmArgs &a, int sm_count, cudaStream_t s)
{
    if (a.num_tiles == 0 && a.num_chunks == 0) return cudaSuccess;
    uint32_t blocks = a.num_tiles > (a.num_chunks + kWarps - 1) / kWarps ? a.num_tiles : (a.num_chunks + kWarps - 1) / kWarps;
    const uint32_t cap = (uint32_t)sm_count * 8;
    if (blocks > cap) blocks = cap;
    sddmm_kernel<<<blocks, kWarps * 32, 0, s>>>(a);
    return cudaGetLastError();
}

}  // namespace cutespmm
