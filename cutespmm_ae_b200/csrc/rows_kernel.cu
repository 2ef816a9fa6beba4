// CUDA-core row-gather kernel: the path for rows whose 16x8 bricks are too empty to pay for a
// tensor-core contraction (power-law graphs, uniform random matrices), and the executor of long
// rows cut into chunks.
//
// In the reference every row panel goes through the brick kernel (kernel.cu:119-288), zero-filled
// bricks included; its tile splitter (inc/splitter.hpp:34-124) that would send light tiles to CUDA
// cores is never called.  Here a warp owns one row at a time: the lanes span the columns of B
// (one float4 each at N = 128, so a row of B is one coalesced 512-byte request), the row's
// (column, value) pairs are read from the block's staged tile in shared memory (tile_stage.cuh; one
// broadcast read per nonzero), and the products are accumulated in fp32 registers in storage order.
// For narrow products (N <= 64) a warp splits into groups of N/4 lanes and owns that many rows at
// once.  The eight warps of a block claim the rows of one scheduling tile as they go, so rows that
// share columns (stencils, block structure) meet in L1.  C rows are written once with streaming
// stores; nothing is read-modify-written: a long row is cut into chunks whose partial sums go to a
// scratch matrix and are added, in slot order, by whichever warp finishes the row's last chunk (one
// counter per long row), in the same launch.
#include <cuda_runtime.h>

#include <cstdint>

#include "device_plan.hpp"
#include "plan.hpp"
#include "ptx.cuh"
#include "tile_stage.cuh"

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
constexpr int kWarps = kTileWarps;
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

__device__ __forceinline__ void add_vec(float4 &a, const float4 &b) { a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
__device__ __forceinline__ void add_vec(float2 &a, const float2 &b) { a.x += b.x; a.y += b.y; }
__device__ __forceinline__ void add_vec(float &a, const float &b) { a += b; }

__device__ __forceinline__ void zero_vec(float4 &a) { a = make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ void zero_vec(float2 &a) { a = make_float2(0.f, 0.f); }
__device__ __forceinline__ void zero_vec(float &a) { a = 0.f; }

__device__ __forceinline__ void store_stream(float4 *p, const float4 &v) { __stcs(p, v); }
__device__ __forceinline__ void store_stream(float2 *p, const float2 &v) { __stcs(p, v); }
__device__ __forceinline__ void store_stream(float *p, const float &v) { __stcs(p, v); }

// acc[ch] += sum over nonzeros [j0, j1) of val * B[col][lane's columns].  `bl` points at this lane's
// first column of row 0 of B; ok[ch] says whether the lane's ch-th column group exists (ragged N).
template <int VEC, int CH, bool FULL, bool DEEP>
__device__ __forceinline__ void accumulate(typename Vec<VEC>::T (&acc)[CH], const uint2 *__restrict__ pairs,
                                           uint32_t j0, uint32_t j1, const float *__restrict__ bl, uint64_t ldb,
                                           const bool (&ok)[CH], int lane)
{
    using V = typename Vec<VEC>::T;
    // nonzeros in flight per step.  With float4 lanes in the 40-register tuning 8 was measured: no gain, spills; the
    // deep tuning and narrow lanes have the registers, and a deeper step shortens the chain of a latency-bound job
    constexpr int U = DEEP ? 8 / CH : ((CH == 1) ? (VEC == 4 ? 4 : 8) : 2);
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

// The same sum for a group of L = 32/G lanes that walks a chunk on its own (G > 1).  The group fetches L pairs with one
// coalesced load (lane i the i-th), the next L while these are in use, and hands them round with shuffles among its
// own lanes (`gmask`), so the groups of a warp may run different lengths.
template <int VEC, int CH, bool FULL, int U, int L>
__device__ __forceinline__ void accumulate_group(typename Vec<VEC>::T (&acc)[CH], const uint2 *__restrict__ pairs, uint32_t j0, uint32_t j1,
                                                 const float *__restrict__ bl, uint32_t ldb32, const bool (&ok)[CH], int sub, unsigned gmask)
{
    using V = typename Vec<VEC>::T;
    constexpr int UU = U < L ? U : L;  // rows of B in flight per step
    uint2 nxt = make_uint2(0u, 0u);
    if (j0 + sub < j1) nxt = __ldg(pairs + j0 + sub);
    for (uint32_t j = j0; j < j1; j += L) {
        const uint2 pr = nxt;
        if (j + L + sub < j1) nxt = __ldg(pairs + j + L + sub);
        const uint32_t n = min((uint32_t)L, j1 - j);
        for (uint32_t k = 0; k < n; k += UU) {
            float v[UU];
            V b[UU][CH];
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                const int src = (int)min(k + u, n - 1);  // positions past the end repeat the last pair and are not added
                const uint32_t c = __shfl_sync(gmask, pr.x, src, L);
                v[u] = __uint_as_float(__shfl_sync(gmask, pr.y, src, L));
                const float *row = bl + (uint64_t)c * ldb32;
#pragma unroll
                for (int ch = 0; ch < CH; ++ch) {
                    if (FULL || ok[ch]) b[u][ch] = ldg_b(reinterpret_cast<const V *>(row + ch * 32 * VEC));
                    else zero_vec(b[u][ch]);
                }
            }
#pragma unroll
            for (int u = 0; u < UU; ++u)
                if (k + u < n) {
#pragma unroll
                    for (int ch = 0; ch < CH; ++ch) fma_vec(acc[ch], v[u], b[u][ch]);
                }
        }
    }
}

// What the chunk part of the kernel needs.  The pointers bl / scratch / C already point at this lane's first column.
struct ChunkArgs {
    const uint2 *pairs;
    const uint4 *chunks;     // {row, j0, j1, slot}
    const uint4 *long_rows;  // {row of C, slot0, slot1, -}
    const uint32_t *chunk_owner;
    uint32_t *arrivals;
    const float *bl;
    float *scratch, *C;
    uint64_t ldb, ld_scratch, ldc;
    uint32_t num_chunks, N, col0;
};

// A chunk's partial sum goes to its slot of the scratch matrix; the warp (or group) that completes a row's last
// outstanding chunk adds the slots in slot order -- so the sum does not depend on who that was -- and writes the row
// of C.  Nobody waits for anybody: whoever is not last just moves on.
template <int VEC, int CH, bool FULL, bool DEEP, int G>
__device__ __forceinline__ void run_chunks(const ChunkArgs &a)
{
    using V = typename Vec<VEC>::T;
    constexpr int L = 32 / G;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int grp = G == 1 ? 0 : lane / L, sub = G == 1 ? lane : lane % L;
    bool ok[CH];
#pragma unroll
    for (int ch = 0; ch < CH; ++ch) ok[ch] = FULL || (a.col0 + ch * 32 * VEC < a.N);
    // chunk (group) c goes to block c mod gridDim.x: spread over the SMs, and the warps of a block that got none
    // start on the block's tile at once (rows of a tile are claimed as they go, so they take over the others' share)
    const uint32_t gw = warp * gridDim.x + blockIdx.x, nw = gridDim.x * kWarps;
    for (uint64_t cw = gw; cw * G < a.num_chunks; cw += nw) {
        const uint64_t c = cw * G + grp;
        const bool have = c < a.num_chunks;
        uint4 ck = make_uint4(0u, 0u, 0u, 0u);
        if (have) ck = __ldg(a.chunks + c);
        // which long row the chunk belongs to.  The narrow kernels (small N: latency-bound jobs) ask now and use the
        // answer after the gathers; the wide ones ask when they need it and keep the registers for the gathers.
        uint32_t owner = 0;
        uint4 lr = make_uint4(0u, 0u, 0u, 0u);  // row of C, slot0, slot1
        if (G > 1 && have && sub == 0) {
            owner = __ldg(a.chunk_owner + ck.w);
            lr = __ldg(a.long_rows + owner);
        }
        V acc[CH];
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) zero_vec(acc[ch]);
        if constexpr (G == 1) accumulate<VEC, CH, FULL, DEEP>(acc, a.pairs, ck.y, ck.z, a.bl, a.ldb, ok, lane);
        else accumulate_group<VEC, CH, FULL, Tuning<DEEP>::kUnroll, L>(acc, a.pairs, ck.y, ck.z, a.bl, (uint32_t)a.ldb, ok, sub, (L == 32 ? kFull : ((1u << L) - 1u)) << (grp * L));
        if (have) {
            float *out = a.scratch + (uint64_t)ck.w * a.ld_scratch;
#pragma unroll
            for (int ch = 0; ch < CH; ++ch)
                if (FULL || ok[ch]) __stcg(reinterpret_cast<V *>(out + ch * 32 * VEC), acc[ch]);
        }
        __threadfence();  // this lane's part of the slot is visible device-wide before the arrival is counted
        __syncwarp();
        uint32_t lr_row = 0, slot0 = 0, slot1 = 0;
        if (have && sub == 0) {
            if (G == 1) {
                owner = __ldg(a.chunk_owner + ck.w);
                lr = __ldg(a.long_rows + owner);
            }
            uint32_t *cnt = a.arrivals + (uint64_t)owner * gridDim.y + blockIdx.y;
            if (atomicAdd(cnt, 1u) == lr.z - lr.y - 1) {  // every chunk of this row and column slab has arrived
                *cnt = 0;                                  // ready for the next launch
                __threadfence();
                lr_row = lr.x; slot0 = lr.y; slot1 = lr.z;
            }
        }
        constexpr int R = (VEC * CH >= 8) ? 4 : 8;  // slots in flight
        if constexpr (G == 1) {
            lr_row = __shfl_sync(kFull, lr_row, 0);
            slot0 = __shfl_sync(kFull, slot0, 0);
            slot1 = __shfl_sync(kFull, slot1, 0);
            if (slot1 > slot0) {
#pragma unroll
                for (int ch = 0; ch < CH; ++ch) zero_vec(acc[ch]);
#pragma unroll R
                for (uint32_t k = slot0; k < slot1; ++k) {
#pragma unroll
                    for (int ch = 0; ch < CH; ++ch)
                        if (FULL || ok[ch]) add_vec(acc[ch], __ldcg(reinterpret_cast<const V *>(a.scratch + (uint64_t)k * a.ld_scratch + ch * 32 * VEC)));
                }
                float *crow = a.C + (uint64_t)lr_row * a.ldc;
#pragma unroll
                for (int ch = 0; ch < CH; ++ch)
                    if (FULL || ok[ch]) store_stream(reinterpret_cast<V *>(crow + ch * 32 * VEC), acc[ch]);
            }
        } else {
            // The whole warp adds the slots of every row one of its groups completed: group h takes slots h, h+G, ...
            // in order, then the groups' sums are added pairwise (a fixed tree: the result depends on nothing but G).
            __syncwarp();
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const uint32_t s0 = __shfl_sync(kFull, slot0, g * L), s1 = __shfl_sync(kFull, slot1, g * L);
                const uint32_t row = __shfl_sync(kFull, lr_row, g * L);
                if (s1 > s0) {  // the same for every lane of the warp
                    zero_vec(acc[0]);
#pragma unroll R
                    for (uint32_t k = s0 + grp; k < s1; k += G)
                        if (FULL || ok[0]) add_vec(acc[0], __ldcg(reinterpret_cast<const V *>(a.scratch + (uint64_t)k * a.ld_scratch)));
#pragma unroll
                    for (int off = L; off < 32; off <<= 1) {
                        acc[0].x += __shfl_xor_sync(kFull, acc[0].x, off);
                        acc[0].y += __shfl_xor_sync(kFull, acc[0].y, off);
                        acc[0].z += __shfl_xor_sync(kFull, acc[0].z, off);
                        acc[0].w += __shfl_xor_sync(kFull, acc[0].w, off);
                    }
                    if (grp == 0 && (FULL || ok[0])) store_stream(reinterpret_cast<V *>(a.C + (uint64_t)row * a.ldc), acc[0]);
                }
            }
        }
        if constexpr (G > 1) __syncwarp();
    }
}

// G = rows of A (or chunks) a warp works on at the same time.  G = 1: the 32 lanes span 32*VEC*CH columns of B.
// G = 2, 4, 8 (narrow products, N <= 64, float4 lanes): the warp is G groups of 32/G lanes, a group spans the whole
// row of B and owns a row of A of its own, so a warp keeps G times as many gathers in flight and no lane idles.
template <int VEC, int CH, bool FULL, bool DEEP, int G>
__global__ void __launch_bounds__(kWarps * 32, Tuning<DEEP>::kMinBlocks) spmm_rows_kernel(RowsArgs a)
{
    using V = typename Vec<VEC>::T;
    static_assert(G == 1 || (VEC == 4 && CH == 1), "row groups are for float4 lanes and one column group");
    constexpr int L = 32 / G;  // lanes of a group
    const int lane = threadIdx.x & 31;
    const int grp = G == 1 ? 0 : lane / L, sub = G == 1 ? lane : lane % L;
    const uint32_t col0 = blockIdx.y * (32 * VEC * CH) + sub * VEC;  // this lane's first column
    bool ok[CH];
#pragma unroll
    for (int ch = 0; ch < CH; ++ch) ok[ch] = FULL || (col0 + ch * 32 * VEC < a.N);
    const float *bl = a.B + col0;
    const uint32_t ldb32 = (uint32_t)a.ldb;  // < 2^32 (checked by the caller): one 32x32->64 multiply per address
    const uint2 *pairs = reinterpret_cast<const uint2 *>(a.pairs);

    // ---- tiles: descriptor, row pointers and pairs arrive in shared memory by TMA, kTileStages deep ----
    __shared__ TileRing ring;
    const TileSource src{reinterpret_cast<const uint4 *>(a.tiles), a.row_ptr, pairs, a.num_tiles};
    tile_ring_start(ring, src);

    // Chunks of long rows first (the first tiles are on their way meanwhile): they are the largest single work items.
    if (a.num_chunks)
        run_chunks<VEC, CH, FULL, DEEP, G>(ChunkArgs{pairs, reinterpret_cast<const uint4 *>(a.chunks), reinterpret_cast<const uint4 *>(a.long_rows),
                                                     a.chunk_owner, a.arrivals, bl, a.scratch + col0, a.C + col0, a.ldb, a.ld_scratch, a.ldc,
                                                     a.num_chunks, a.N, col0});

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
            uint32_t r = tile_claim_rows(ring, s, (uint32_t)G, lane) + d.x;
            if (r >= d.y) break;
            r += grp;  // the group's own row
            if (G == 1 || r < d.y) {
                const uint32_t j0 = st.row_ptr[r - rb], j1 = st.row_ptr[r - rb + 1];
                V acc[CH];
#pragma unroll
                for (int ch = 0; ch < CH; ++ch) zero_vec(acc[ch]);
                constexpr int U = (CH == 1) ? Tuning<DEEP>::kUnroll : Tuning<DEEP>::kUnroll / 2;  // rows of B in flight per group and step
                uint32_t j = j0 - jb, jend = j1 - jb;  // positions in the staged pair slice
                for (; j + U <= jend; j += U) row_group<VEC, CH, FULL, U, false>(acc, st.pairs + j, U, bl, ldb32, ok);
                // what is left of the row (fewer than U nonzeros) goes as one more group, so that its loads are in flight
                // together instead of one after the other: positions past the end repeat the row's last pair and are not added
                if (const uint32_t rem = jend - j) {
                    if (rem > U / 2) row_group<VEC, CH, FULL, U, true>(acc, st.pairs + j, rem, bl, ldb32, ok);
                    else row_group<VEC, CH, FULL, U / 2, true>(acc, st.pairs + j, rem, bl, ldb32, ok);
                }
                const uint32_t r_out = a.row_map ? __ldg(a.row_map + r) : r;  // a reordered plan writes the row to its place in the caller's C
                float *out = a.C + (uint64_t)r_out * a.ldc + col0;
#pragma unroll
                for (int ch = 0; ch < CH; ++ch)
                    if (FULL || ok[ch]) store_stream(reinterpret_cast<V *>(out + ch * 32 * VEC), acc[ch]);
            }
            if constexpr (G > 1) __syncwarp();
        }
        tile_release(ring, src, i, t, lane);  // the last warp to leave the stage refills it
    }
}

template <int VEC, int CH, bool FULL, bool DEEP, int G = 1>
cudaError_t launch_rows_t(const RowsArgs &a, uint32_t slabs, int sm_count, cudaStream_t s)
{
    static int blocks_per_sm = 0;  // same for every device of one model; queried once
    if (blocks_per_sm == 0) {
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, spmm_rows_kernel<VEC, CH, FULL, DEEP, G>, kWarps * 32, 0);
        if (e != cudaSuccess) return e;
        blocks_per_sm = n > 0 ? n : 1;
    }
    const uint64_t want = (uint64_t)sm_count * blocks_per_sm;
    const uint64_t chunk_blocks = ((uint64_t)a.num_chunks + kWarps * G - 1) / (kWarps * G);
    uint64_t work = a.num_tiles > chunk_blocks ? a.num_tiles : chunk_blocks;
    uint32_t gx = (uint32_t)(work < want ? work : want);
    if (slabs > 1) gx = (gx + slabs - 1) / slabs;  // keep the whole grid about one resident wave
    if (gx == 0) gx = 1;
    spmm_rows_kernel<VEC, CH, FULL, DEEP, G><<<dim3(gx, slabs), kWarps * 32, 0, s>>>(a);
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
    if (v4 && N <= 64) {  // narrow products: G rows of A per warp, a group of 32/G float4 lanes spans the row of B
#define CUTESPMM_GROUPS(G)                                                                              \
    do {                                                                                                \
        if (deep) return (N == 128 / G) ? launch_rows_t<4, 1, true, true, G>(a, 1, sm_count, s)         \
                                        : launch_rows_t<4, 1, false, true, G>(a, 1, sm_count, s);       \
        return (N == 128 / G) ? launch_rows_t<4, 1, true, false, G>(a, 1, sm_count, s)                  \
                              : launch_rows_t<4, 1, false, false, G>(a, 1, sm_count, s);                \
    } while (0)
        if (N <= 16) CUTESPMM_GROUPS(8);
        if (N <= 32) CUTESPMM_GROUPS(4);
        CUTESPMM_GROUPS(2);
#undef CUTESPMM_GROUPS
    }
    if (v4) {
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

}  // namespace cutespmm
