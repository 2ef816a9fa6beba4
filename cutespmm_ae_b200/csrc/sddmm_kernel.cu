// SDDMM over the sparsity pattern of a plan: for every stored nonzero (r, c) of A
//
//        out[j] = (scale ? A[r][c] : 1) * sum_n X[r][n] * Y[c][n]
//
// the "edge feature" operator that accompanies SpMM in a graph layer (the reference tree carries it as
// TC-GNN's forward_ef, TC-GNN_ATC23/TCGNN_conv/TCGNN.cpp:265, and its own kernels do not have it), and
// the gradient of SpMM with respect to the values of A (dA = SDDMM(dC, B)).  Like the row kernel it is
// bound by gathering one row of Y per nonzero, and it is built on the same skeleton: the block's tiles
// arrive in shared memory by TMA, warps claim rows as they go, chunks of long rows are dealt over the
// blocks first.  A warp keeps the 128-column span of X[r] in registers and handles eight nonzeros per
// step -- eight lanes per nonzero, so a row of Y is four 128-byte requests and a dot product needs
// three shuffles; two such groups of four are in flight.  Every nonzero has its own output, so nothing
// is summed across work items.
#include <cuda_runtime.h>

#include <cstdint>

#include "device_plan.hpp"
#include "plan.hpp"
#include "tile_stage.cuh"

namespace cutespmm {

namespace {

constexpr unsigned kFull = 0xffffffffu;
constexpr int kSteps = 2;  // groups of four nonzeros in flight per warp

// The lane's part of the 128-column span that starts at column c0 of a row: float4 number sub, sub+8, sub+16, sub+24.
template <bool FAST>
__device__ __forceinline__ void load_span(float4 (&v)[4], const float *row, uint32_t c0, uint32_t N, bool vec4, int sub)
{
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t c = c0 + (uint32_t)(sub + 8 * i) * 4;
        if (FAST) {
            v[i] = __ldg(reinterpret_cast<const float4 *>(row + c));
        } else {
            v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < N) {
                if (vec4 && c + 4 <= N) v[i] = __ldg(reinterpret_cast<const float4 *>(row + c));
                else {
                    v[i].x = __ldg(row + c);
                    if (c + 1 < N) v[i].y = __ldg(row + c + 1);
                    if (c + 2 < N) v[i].z = __ldg(row + c + 2);
                    if (c + 3 < N) v[i].w = __ldg(row + c + 3);
                }
            }
        }
    }
}

__device__ __forceinline__ float dot_span(const float4 (&x)[4], const float4 (&y)[4])
{
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        s = fmaf(x[i].x, y[i].x, s);
        s = fmaf(x[i].y, y[i].y, s);
        s = fmaf(x[i].z, y[i].z, s);
        s = fmaf(x[i].w, y[i].w, s);
    }
    return s;
}

// STEPS groups of four nonzeros, starting at nonzero k of the item: the span c0 of X[row] (in x) against the same span
// of the rows of Y they name.  first: write; otherwise add to the earlier spans' sums.
template <bool FAST, int STEPS, class PairAt>
__device__ __forceinline__ void sddmm_step(const SddmmArgs &a, const float4 (&x)[4], PairAt pair_at, uint32_t k, uint32_t cnt, float *out,
                                           uint32_t c0, bool first, int lane)
{
    const int sub = lane & 7, grp = lane >> 3;
    uint2 pr[STEPS];
    float4 y[STEPS][4];
#pragma unroll
    for (int u = 0; u < STEPS; ++u) {
        const uint32_t mine = k + u * 4 + grp;
        pr[u] = pair_at(min(mine, cnt - 1));  // positions past the end repeat the last pair (a cache hit) and are not stored
        load_span<FAST>(y[u], a.Y + (uint64_t)pr[u].x * a.ldy, c0, a.N, a.vec4 != 0, sub);
    }
#pragma unroll
    for (int u = 0; u < STEPS; ++u) {
        float s = dot_span(x, y[u]);
        s += __shfl_xor_sync(kFull, s, 4);
        s += __shfl_xor_sync(kFull, s, 2);
        s += __shfl_xor_sync(kFull, s, 1);
        const uint32_t mine = k + u * 4 + grp;
        if (mine < cnt && sub == 0) {
            if (a.scale) s *= __uint_as_float(pr[u].y);
            out[mine] = first ? s : out[mine] + s;
        }
    }
}

// Nonzeros [0, cnt) of one row (or chunk) whose pairs are pair_at(k) and whose outputs are out[k]: kSteps groups of four
// in flight while more than four nonzeros are left, one group for a tail of one to four.
template <bool FAST, class PairAt>
__device__ __forceinline__ void sddmm_items(const SddmmArgs &a, const float4 (&x)[4], PairAt pair_at, uint32_t cnt, float *out,
                                            uint32_t c0, bool first, int lane)
{
    uint32_t k = 0;
    for (; k + 4 < cnt; k += 4 * kSteps) sddmm_step<FAST, kSteps>(a, x, pair_at, k, cnt, out, c0, first, lane);
    if (k < cnt) sddmm_step<FAST, 1>(a, x, pair_at, k, cnt, out, c0, first, lane);
}

template <bool FAST>
__global__ void __launch_bounds__(kTileWarps * 32, 3) sddmm_kernel(SddmmArgs a)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane & 7;
    const uint2 *pairs = reinterpret_cast<const uint2 *>(a.pairs);
    __shared__ TileRing ring;
    const TileSource src{reinterpret_cast<const uint4 *>(a.tiles), a.row_ptr, pairs, a.num_tiles};
    tile_ring_start(ring, src);

    // chunks of long rows first (the tiles are on their way): chunk c goes to block c mod gridDim.x.  The pairs of a
    // chunk come 32 at a time with one coalesced load, the next 32 while these are in use.
    {
        const uint4 *chunks = reinterpret_cast<const uint4 *>(a.chunks);
        for (uint32_t c = warp * gridDim.x + blockIdx.x; c < a.num_chunks; c += gridDim.x * kTileWarps) {
            const uint4 ck = __ldg(chunks + c);  // row, j0, j1, slot
            for (uint32_t c0 = 0; c0 < a.N; c0 += 128) {
                float4 x[4];
                load_span<FAST>(x, a.X + (uint64_t)ck.x * a.ldx, c0, a.N, a.vec4 != 0, sub);
                uint2 nxt = make_uint2(0u, 0u);
                if (ck.y + lane < ck.z) nxt = __ldg(pairs + ck.y + lane);
                for (uint32_t j = ck.y; j < ck.z; j += 32) {
                    const uint2 cur = nxt;
                    if (j + 32 + lane < ck.z) nxt = __ldg(pairs + j + 32 + lane);
                    auto pair_at = [&](uint32_t k) { return make_uint2(__shfl_sync(kFull, cur.x, (int)k), __shfl_sync(kFull, cur.y, (int)k)); };
                    sddmm_items<FAST>(a, x, pair_at, min(32u, ck.z - j), a.out + j, c0, c0 == 0, lane);
                }
            }
        }
    }

    for (uint32_t i = 0;; ++i) {
        const uint64_t t = blockIdx.x + (uint64_t)i * gridDim.x;
        if (t >= a.num_tiles) break;
        const int s = i % kTileStages;
        if (!tile_wait(ring, i)) {
            if (lane == 0) atomicExch(a.status, 1u);  // the copy never landed: report, do not hang
            break;
        }
        const TileStage &st = ring.stage[s];
        const uint4 d = st.desc;
        const uint32_t rb = d.x & ~3u, jb = d.z & ~1u;
        for (;;) {
            const uint32_t r = tile_claim_rows(ring, s, 1u, lane) + d.x;
            if (r >= d.y) break;
            const uint32_t j0 = st.row_ptr[r - rb], j1 = st.row_ptr[r - rb + 1];
            if (j1 == j0) continue;
            const uint2 *row_pairs = st.pairs + (j0 - jb);
            auto pair_at = [&](uint32_t k) { return row_pairs[k]; };  // the lanes of a group read one address
            for (uint32_t c0 = 0; c0 < a.N; c0 += 128) {
                float4 x[4];
                load_span<FAST>(x, a.X + (uint64_t)r * a.ldx, c0, a.N, a.vec4 != 0, sub);
                sddmm_items<FAST>(a, x, pair_at, j1 - j0, a.out + j0, c0, c0 == 0, lane);
            }
        }
        tile_release(ring, src, i, t, lane);
    }
}

}  // namespace

cudaError_t launch_sddmm(const SddmmArgs &a, int sm_count, cudaStream_t s)
{
    if (a.num_tiles == 0 && a.num_chunks == 0) return cudaSuccess;
    const uint32_t chunk_blocks = (a.num_chunks + kTileWarps - 1) / kTileWarps;
    uint32_t blocks = a.num_tiles > chunk_blocks ? a.num_tiles : chunk_blocks;
    const uint32_t cap = (uint32_t)sm_count * 3;  // one resident wave
    if (blocks > cap) blocks = cap;
    if (a.vec4 && a.N % 128 == 0) sddmm_kernel<true><<<blocks, kTileWarps * 32, 0, s>>>(a);
    else sddmm_kernel<false><<<blocks, kTileWarps * 32, 0, s>>>(a);
    return cudaGetLastError();
}

}  // namespace cutespmm
