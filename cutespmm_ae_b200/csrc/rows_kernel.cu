// CUDA-core row-gather kernel: the path for rows whose 16x8 bricks are too empty to pay for a
// tensor-core contraction (power-law graphs, uniform random matrices), and the executor of long
// rows cut into chunks.
//
// In the reference every row panel goes through the brick kernel (kernel.cu:119-288), zero-filled
// bricks included; its tile splitter (inc/splitter.hpp:34-124) that would send light tiles to CUDA
// cores is never called.  Here a warp owns one row at a time: the lanes span the columns of B
// (one float4 each at N = 128, so a row of B is one coalesced 512-byte request), the row's
// (column, value) pairs are fetched 32 at a time with one coalesced 8-byte load per lane and handed
// round with shuffles, and the products are accumulated in fp32 registers in storage order.  The
// eight warps of a block take interleaved rows of one scheduling tile, so rows that share columns
// (stencils, block structure) meet in L1.  C rows are written once with streaming stores; nothing
// is read-modify-written and no atomics are used: a long row is cut into chunks whose partial sums
// go to a scratch matrix and are added, in order, by a second small kernel.
#include <cuda_runtime.h>

#include <cstdint>

#include "device_plan.hpp"
#include "plan.hpp"
#include "ptx.cuh"

namespace cutespmm {

namespace {

// Two tunings of the row kernel, chosen per launch (measured on R-MAT graphs and the 512x512 stencil at N = 128):
//   DEEP = false  4 rows of B in flight per warp, 6 blocks (48 warps) per SM: more warps hide the gather latency
//                 better than more loads per warp when rows are short and the grid is several waves of tiles long;
//   DEEP = true   8 rows in flight, 4 blocks per SM: fewer dependent steps per row, better for long rows and when
//                 the whole job is a single wave of tiles and the time is a handful of latencies.
template <bool DEEP> struct Tuning {
    static constexpr int kUnroll = DEEP ? 8 : 4;
    static constexpr int kMinBlocks = DEEP ? 4 : 6;
};
constexpr int kWarps = 8;
constexpr int kStages = 3;  // tiles in flight per block (TMA bulk copies into shared memory)

// One staged tile: its descriptor, the slice of row pointers and the slice of (column, value) pairs,
// each fetched by one bulk copy that starts on a 16-byte boundary at or before the first needed
// element (hence the slack of 3 words / 1 pair in front and behind).
struct __align__(16) TileStage {
    uint4 desc;                               // row_begin, row_end, pair_begin, pair_end
    uint32_t row_ptr[kMaxTileRows + 8];
    uint2 pairs[kMaxTilePairs + 2];
};
constexpr unsigned kFull = 0xffffffffu;

template <int VEC> struct Vec;
template <> struct Vec<4> { using T = float4; };
template <> struct Vec<2> { using T = float2; };
template <> struct Vec<1> { using T = float; };

__device__ __forceinline__ float4 ldg_b(const float4 *p) { return __ldg(p); }
__device__ __forceinline__ float2 ldg_b(const float2 *p) { return __ldg(p); }
__device__ __forceinline__ float ldg_b(const float *p) { return __ldg(p); }

__device__ __forceinline__ void fma_vec(float4 &a, float v, const float4 &b)
{
    a.x = fmaf(v, b.x, a.x); a.y = fmaf(v, b.y, a.y); a.z = fmaf(v, b.z, a.z); a.w = fmaf(v, b.w, a.w);
}
__device__ __forceinline__ void fma_vec(float2 &a, float v, const float2 &b)
{
    a.x = fmaf(v, b.x, a.x); a.y = fmaf(v, b.y, a.y);
}
__device__ __forceinline__ void fma_vec(float &a, float v, const float &b) { a = fmaf(v, b, a); }

__device__ __forceinline__ void zero_vec(float4 &a) { a = make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ void zero_vec(float2 &a) { a = make_float2(0.f, 0.f); }
__device__ __forceinline__ void zero_vec(float &a) { a = 0.f; }

__device__ __forceinline__ void store_stream(float4 *p, const float4 &v) { __stcs(p, v); }
__device__ __forceinline__ void store_stream(float2 *p, const float2 &v) { __stcs(p, v); }
__device__ __forceinline__ void store_stream(float *p, const float &v) { __stcs(p, v); }

// acc[ch] += sum over nonzeros [j0, j1) of val * B[col][lane's columns].  `bl` points at this lane's
// first column of row 0 of B; ok[ch] says whether the lane's ch-th column group exists (ragged N).
template <int VEC, int CH, bool FULL>
__device__ __forceinline__ void accumulate(typename Vec<VEC>::T (&acc)[CH], const uint2 *__restrict__ pairs,
                                           uint32_t j0, uint32_t j1, const float *__restrict__ bl, uint64_t ldb,
                                           const bool (&ok)[CH], int lane)
{
    using V = typename Vec<VEC>::T;
    constexpr int U = (CH == 1) ? 4 : 2;  // nonzeros in flight per step (8 was measured: no gain, spills)
    for (uint32_t j = j0; j < j1; j += 32) {
        const uint32_t n = min(32u, j1 - j);
        uint2 pr = make_uint2(0u, 0u);
        if ((uint32_t)lane < n) pr = __ldcs(pairs + j + lane);
        uint32_t k = 0;
        for (; k + U <= n; k += U) {
            float v[U];
            V b[U][CH];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t c = __shfl_sync(kFull, pr.x, k + u);
                v[u] = __uint_as_float(__shfl_sync(kFull, pr.y, k + u));
                const float *row = bl + (uint64_t)c * ldb;
#pragma unroll
                for (int ch = 0; ch < CH; ++ch) {
                    if (FULL || ok[ch]) b[u][ch] = ldg_b(reinterpret_cast<const V *>(row + ch * 32 * VEC));
                    else zero_vec(b[u][ch]);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int ch = 0; ch < CH; ++ch) fma_vec(acc[ch], v[u], b[u][ch]);
        }
        for (; k < n; ++k) {
            const uint32_t c = __shfl_sync(kFull, pr.x, k);
            const float v = __uint_as_float(__shfl_sync(kFull, pr.y, k));
            const float *row = bl + (uint64_t)c * ldb;
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) {
                if (FULL || ok[ch]) {
                    const V b = ldg_b(reinterpret_cast<const V *>(row + ch * 32 * VEC));
                    fma_vec(acc[ch], v, b);
                }
            }
        }
    }
}

// acc[ch] += sum of val * B[col][lane's columns] over `cnt` staged (column, value) pairs, UU rows of B in flight.
// TAIL: cnt may be smaller than UU; the surplus positions load the row of the last pair again (an L1 hit) and
// are left out of the sum.
template <int VEC, int CH, bool FULL, int UU, bool TAIL>
__device__ __forceinline__ void row_group(typename Vec<VEC>::T (&acc)[CH], const uint2 *pairs_smem, uint32_t cnt, const float *__restrict__ bl,
                                          uint32_t ldb32, const bool (&ok)[CH])
{
    using V = typename Vec<VEC>::T;
    float v[UU];
    V b[UU][CH];
#pragma unroll
    for (int u = 0; u < UU; ++u) {
        const uint2 pr = pairs_smem[TAIL ? min((uint32_t)u, cnt - 1) : (uint32_t)u];  // all lanes read one address: broadcast
        v[u] = __uint_as_float(pr.y);
        const float *row = bl + (uint64_t)pr.x * ldb32;
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
            if (FULL || ok[ch]) b[u][ch] = ldg_b(reinterpret_cast<const V *>(row + ch * 32 * VEC));
            else zero_vec(b[u][ch]);
        }
    }
#pragma unroll
    for (int u = 0; u < UU; ++u)
        if (!TAIL || (uint32_t)u < cnt) {
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) fma_vec(acc[ch], v[u], b[u][ch]);
        }
}

template <int VEC, int CH, bool FULL, bool DEEP>
__global__ void __launch_bounds__(kWarps * 32, Tuning<DEEP>::kMinBlocks) spmm_rows_kernel(RowsArgs a)
{
    using V = typename Vec<VEC>::T;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const uint32_t col0 = blockIdx.y * (32 * VEC * CH) + lane * VEC;  // this lane's first column
    bool ok[CH];
#pragma unroll
    for (int ch = 0; ch < CH; ++ch) ok[ch] = FULL || (col0 + ch * 32 * VEC < a.N);
    const float *bl = a.B + col0;
    const uint32_t ldb32 = (uint32_t)a.ldb;  // < 2^32 (checked by the caller): one 32x32->64 multiply per address
    const uint2 *pairs = reinterpret_cast<const uint2 *>(a.pairs);

    // chunks of long rows first: they are the largest single work items
    {
        const uint32_t gw = blockIdx.x * kWarps + warp, nw = gridDim.x * kWarps;
        for (uint32_t c = gw; c < a.num_chunks; c += nw) {
            const uint4 ck = __ldg(reinterpret_cast<const uint4 *>(a.chunks) + c);  // row, j0, j1, slot
            V acc[CH];
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) zero_vec(acc[ch]);
            accumulate<VEC, CH, FULL>(acc, pairs, ck.y, ck.z, bl, a.ldb, ok, lane);
            float *out = a.scratch + (uint64_t)ck.w * a.ld_scratch + col0;
#pragma unroll
            for (int ch = 0; ch < CH; ++ch)
                if (FULL || ok[ch]) *reinterpret_cast<V *>(out + ch * 32 * VEC) = acc[ch];
        }
    }

    // ---- tiles: descriptor, row pointers and pairs arrive in shared memory by TMA, kStages deep ----
    __shared__ TileStage stage[kStages];
    __shared__ __align__(8) uint64_t full_bar[kStages];
    __shared__ uint32_t next_row[kStages];  // rows of the staged tile already claimed by a warp
    __shared__ uint32_t warps_done[kStages];

    const uint4 *tiles = reinterpret_cast<const uint4 *>(a.tiles);
    auto issue = [&](uint32_t t, int s) {  // one thread: fetch tile t into stage s
        const uint4 d = __ldg(tiles + t);
        const uint32_t rb = d.x & ~3u, re = (d.y + 1 + 3) & ~3u;  // row pointers [rb, re) cover d.x .. d.y
        const uint32_t jb = d.z & ~1u, je = (d.w + 1) & ~1u;      // pairs [jb, je) cover d.z .. d.w-1
        const uint32_t bytes = 16u + (re - rb) * 4u + (je - jb) * 8u;
        ptx::mbar_expect_tx(&full_bar[s], bytes);
        ptx::bulk_g2s(&stage[s].desc, tiles + t, 16u, &full_bar[s]);
        ptx::bulk_g2s(stage[s].row_ptr, a.row_ptr + rb, (re - rb) * 4u, &full_bar[s]);
        if (je > jb) ptx::bulk_g2s(stage[s].pairs, pairs + jb, (je - jb) * 8u, &full_bar[s]);
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            next_row[s] = 0;
            warps_done[s] = 0;
        }
        ptx::fence_mbar_init();
        for (int s = 0; s < kStages; ++s) {
            const uint64_t t = blockIdx.x + (uint64_t)s * gridDim.x;
            if (t < a.num_tiles) issue((uint32_t)t, s);
        }
    }
    __syncthreads();

    for (uint32_t i = 0;; ++i) {
        const uint64_t t = blockIdx.x + (uint64_t)i * gridDim.x;
        if (t >= a.num_tiles) break;
        const int s = i % kStages;
        if (!ptx::mbar_wait(&full_bar[s], (i / kStages) & 1u)) {
            if (lane == 0) atomicExch(a.status, 1u);  // the copy never landed: report, do not hang
            break;
        }
        const uint4 d = stage[s].desc;
        const uint32_t rb = d.x & ~3u, jb = d.z & ~1u;
        for (;;) {
            uint32_t r = 0;
            if (lane == 0) r = atomicAdd(&next_row[s], 1u);
            r = __shfl_sync(kFull, r, 0) + d.x;
            if (r >= d.y) break;
            const uint32_t j0 = stage[s].row_ptr[r - rb], j1 = stage[s].row_ptr[r - rb + 1];
            V acc[CH];
#pragma unroll
            for (int ch = 0; ch < CH; ++ch) zero_vec(acc[ch]);
            constexpr int U = (CH == 1) ? Tuning<DEEP>::kUnroll : Tuning<DEEP>::kUnroll / 2;  // rows of B in flight per warp and step
            uint32_t j = j0 - jb, jend = j1 - jb;  // positions in the staged pair slice
            for (; j + U <= jend; j += U) row_group<VEC, CH, FULL, U, false>(acc, stage[s].pairs + j, U, bl, ldb32, ok);
            // what is left of the row (fewer than U nonzeros) goes as one more group, so that its loads are in flight
            // together instead of one after the other: positions past the end repeat the row's last pair and are not added
            if (const uint32_t rem = jend - j) {
                if (rem > U / 2) row_group<VEC, CH, FULL, U, true>(acc, stage[s].pairs + j, rem, bl, ldb32, ok);
                else row_group<VEC, CH, FULL, U / 2, true>(acc, stage[s].pairs + j, rem, bl, ldb32, ok);
            }
            const uint32_t r_out = a.row_map ? __ldg(a.row_map + r) : r;  // a reordered plan writes the row to its place in the caller's C
            float *out = a.C + (uint64_t)r_out * a.ldc + col0;
#pragma unroll
            for (int ch = 0; ch < CH; ++ch)
                if (FULL || ok[ch]) store_stream(reinterpret_cast<V *>(out + ch * 32 * VEC), acc[ch]);
        }
        // this warp is finished with stage s; the last warp to say so refills it
        __syncwarp();
        if (lane == 0) {
            __threadfence_block();
            if (atomicAdd(&warps_done[s], 1u) == kWarps - 1) {
                __threadfence_block();
                warps_done[s] = 0;
                next_row[s] = 0;
                const uint64_t t2 = t + (uint64_t)kStages * gridDim.x;
                if (t2 < a.num_tiles) {
                    ptx::fence_async_smem();
                    issue((uint32_t)t2, s);
                }
            }
        }
    }
}

// C[row] = scratch[slot0] + scratch[slot0+1] + ... (in slot order: deterministic).
__global__ void __launch_bounds__(128) spmm_fixup_kernel(const uint4 *__restrict__ long_rows, uint32_t num_long_rows,
                                                         const float *__restrict__ scratch, uint64_t ld_scratch,
                                                         float *__restrict__ C, uint64_t ldc, uint32_t N)
{
    for (uint32_t i = blockIdx.x; i < num_long_rows; i += gridDim.x) {
        const uint4 lr = __ldg(long_rows + i);  // row, slot0, slot1
        for (uint32_t n = threadIdx.x; n < N; n += blockDim.x) {
            float s = 0.f;
            for (uint32_t k = lr.y; k < lr.z; ++k) s += scratch[(uint64_t)k * ld_scratch + n];
            __stcs(C + (uint64_t)lr.x * ldc + n, s);
        }
    }
}

// ---- narrow products (N <= 64) -----------------------------------------------------------------------------------
// With 32 or 64 columns a row of B is 128 or 256 bytes: a whole warp per nonzero would leave most lanes idle or move
// four bytes per lane.  Here the warp still owns a row of A, but G of its nonzeros are in flight per load instruction:
// the lanes form G groups of 32/G, a group holds one nonzero, a lane one float4 of that nonzero's row of B.  Each
// group accumulates its own partial sum; the groups are added with shuffles when the row ends (the order of the sum
// differs from the row kernel's: group g adds nonzeros g, g+G, ... first).  Work items are the same tiles and chunks;
// rows are taken in turn by the warps of a block, pairs and row pointers come straight from global memory (rows are
// short here, the tile staging of the wide kernel does not pay).
template <int G>
__global__ void __launch_bounds__(kWarps * 32, 6) spmm_rows_narrow_kernel(RowsArgs a)
{
    constexpr int L = 32 / G;   // lanes per nonzero
    constexpr int U = 4;        // loads in flight per lane
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int grp = lane / L, sub = lane % L;
    const uint32_t col = sub * 4;
    const bool has_col = col < a.N;
    const uint2 *pairs = reinterpret_cast<const uint2 *>(a.pairs);
    const float *bl = a.B + col;
    const uint32_t ldb32 = (uint32_t)a.ldb;
    auto run = [&](uint32_t j0, uint32_t j1, float *out) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t j = j0 + grp; j < j1; j += G * U) {
            float v[U];
            float4 b[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t jj = j + u * G;
                v[u] = 0.f;
                b[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (jj < j1) {
                    const uint2 pr = __ldg(pairs + jj);  // the lanes of a group read one address
                    v[u] = __uint_as_float(pr.y);
                    if (has_col) b[u] = __ldg(reinterpret_cast<const float4 *>(bl + (uint64_t)pr.x * ldb32));
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (j + u * G < j1) fma_vec(acc, v[u], b[u]);
        }
#pragma unroll
        for (int off = L; off < 32; off <<= 1) {
            acc.x += __shfl_xor_sync(kFull, acc.x, off);
            acc.y += __shfl_xor_sync(kFull, acc.y, off);
            acc.z += __shfl_xor_sync(kFull, acc.z, off);
            acc.w += __shfl_xor_sync(kFull, acc.w, off);
        }
        if (grp == 0 && has_col) *reinterpret_cast<float4 *>(out + col) = acc;
    };
    // chunks of long rows first
    {
        const uint32_t gw = blockIdx.x * kWarps + warp, nw = gridDim.x * kWarps;
        for (uint32_t c = gw; c < a.num_chunks; c += nw) {
            const uint4 ck = __ldg(reinterpret_cast<const uint4 *>(a.chunks) + c);  // row, j0, j1, slot
            run(ck.y, ck.z, a.scratch + (uint64_t)ck.w * a.ld_scratch);
        }
    }
    const uint4 *tiles = reinterpret_cast<const uint4 *>(a.tiles);
    for (uint32_t t = blockIdx.x; t < a.num_tiles; t += gridDim.x) {
        const uint4 d = __ldg(tiles + t);
        for (uint32_t r = d.x + warp; r < d.y; r += kWarps) {
            const uint32_t j0 = __ldg(a.row_ptr + r), j1 = __ldg(a.row_ptr + r + 1);
            const uint32_t r_out = a.row_map ? __ldg(a.row_map + r) : r;
            run(j0, j1, a.C + (uint64_t)r_out * a.ldc);
        }
    }
}

template <int G> cudaError_t launch_rows_narrow_t(const RowsArgs &a, int sm_count, cudaStream_t s)
{
    const uint64_t want = (uint64_t)sm_count * 6;
    uint64_t work = a.num_tiles > (a.num_chunks + kWarps - 1) / kWarps ? a.num_tiles : (a.num_chunks + kWarps - 1) / kWarps;
    uint32_t gx = (uint32_t)(work < want ? work : want);
    if (gx == 0) gx = 1;
    spmm_rows_narrow_kernel<G><<<gx, kWarps * 32, 0, s>>>(a);
    return cudaGetLastError();
}

template <int VEC, int CH, bool FULL, bool DEEP>
cudaError_t launch_rows_t(const RowsArgs &a, uint32_t slabs, int sm_count, cudaStream_t s)
{
    static int blocks_per_sm = 0;  // same for every device of one model; queried once
    if (blocks_per_sm == 0) {
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, spmm_rows_kernel<VEC, CH, FULL, DEEP>, kWarps * 32, 0);
        if (e != cudaSuccess) return e;
        blocks_per_sm = n > 0 ? n : 1;
    }
    const uint64_t want = (uint64_t)sm_count * blocks_per_sm;
    uint64_t work = a.num_tiles > (a.num_chunks + kWarps - 1) / kWarps ? a.num_tiles : (a.num_chunks + kWarps - 1) / kWarps;
    uint32_t gx = (uint32_t)(work < want ? work : want);
    if (slabs > 1) gx = (gx + slabs - 1) / slabs;  // keep the whole grid about one resident wave
    if (gx == 0) gx = 1;
    spmm_rows_kernel<VEC, CH, FULL, DEEP><<<dim3(gx, slabs), kWarps * 32, 0, s>>>(a);
    return cudaGetLastError();
}

}  // namespace

int rows_kernel_count(const RowsArgs &a) { return (a.num_tiles || a.num_chunks) ? 1 : 0; }

// Picks the widest vector the pointers, leading dimensions and N allow.
cudaError_t launch_rows(const RowsArgs &a, int sm_count, cudaStream_t s)
{
    if (a.num_tiles == 0 && a.num_chunks == 0) return cudaSuccess;
    const uintptr_t pb = reinterpret_cast<uintptr_t>(a.B), pc = reinterpret_cast<uintptr_t>(a.C),
                    ps = reinterpret_cast<uintptr_t>(a.scratch);
    const bool v4 = !((pb | pc | ps) & 15) && !((a.ldb | a.ldc | a.ld_scratch | a.N) & 3);
    const bool v2 = !((pb | pc | ps) & 7) && !((a.ldb | a.ldc | a.ld_scratch | a.N) & 1);
    const uint32_t N = a.N;
    if (v4 && N <= 64) {  // narrow products: several nonzeros of a row in flight per load instruction
        if (N <= 16) return launch_rows_narrow_t<8>(a, sm_count, s);
        if (N <= 32) return launch_rows_narrow_t<4>(a, sm_count, s);
        return launch_rows_narrow_t<2>(a, sm_count, s);
    }
    // deep: at most one resident wave of tiles, or long rows (measured on shards of R-MAT 2^24: 300 nonzeros per row
    // 2.19 vs 2.38 ms, 21 per row 1.88 vs 1.93 ms in favour of deep; 15 per row (R-MAT 2^20) 0.645 vs 0.611 ms and
    // 3.4 per row 1.50 vs 1.48 ms in favour of shallow)
    const bool deep = (uint64_t)a.num_tiles <= (uint64_t)sm_count * 6 || a.avg_row_nnz >= 20;
#define CUTESPMM_GO(VEC, CH)                                                                   \
    do {                                                                                       \
        const uint32_t w = 32 * VEC * CH, slabs = (N + w - 1) / w;                             \
        if (deep)                                                                              \
            return (N % w == 0) ? launch_rows_t<VEC, CH, true, true>(a, slabs, sm_count, s)    \
                                : launch_rows_t<VEC, CH, false, true>(a, slabs, sm_count, s);  \
        return (N % w == 0) ? launch_rows_t<VEC, CH, true, false>(a, slabs, sm_count, s)       \
                            : launch_rows_t<VEC, CH, false, false>(a, slabs, sm_count, s);     \
    } while (0)
    if (v4 && N > 64) {
        if (N >= 256) CUTESPMM_GO(4, 2);
        CUTESPMM_GO(4, 1);
    }
    if (v2 && N > 32) {
        if (N >= 128) CUTESPMM_GO(2, 2);
        CUTESPMM_GO(2, 1);
    }
    if (N >= 64) CUTESPMM_GO(1, 2);
    CUTESPMM_GO(1, 1);
#undef CUTESPMM_GO
}

cudaError_t launch_fixup(const RowsArgs &a, cudaStream_t s)
{
    if (a.num_long_rows == 0) return cudaSuccess;
    const uint32_t g = a.num_long_rows < 4096 ? a.num_long_rows : 4096;
    spmm_fixup_kernel<<<g, 128, 0, s>>>(reinterpret_cast<const uint4 *>(a.long_rows), a.num_long_rows, a.scratch,
                                        a.ld_scratch, a.C, a.ldc, a.N);
    return cudaGetLastError();
}

}  // namespace cutespmm
