// The staging ring the row-walking kernels share (the product's row kernel and SDDMM): a block's scheduling tiles --
// descriptor, slice of row pointers, slice of (column, value) pairs -- arrive in shared memory by TMA bulk copies,
// kTileStages tiles deep; the warps of the block claim rows of the staged tile as they go, and the last warp to leave a
// stage refills it.  No block-wide barrier after the start; every wait is bounded.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "plan.hpp"
#include "ptx.cuh"

namespace cutespmm {

constexpr int kTileWarps = 8;   // warps of a block that walks tiles
constexpr int kTileStages = 3;  // tiles in flight per block

// One staged tile.  Each of the three parts is fetched by one bulk copy that starts on a 16-byte boundary at or before
// the first needed element (hence the slack of 3 words / 1 pair in front and behind).
struct __align__(16) TileStage {
    uint4 desc;                               // row_begin, row_end, pair_begin, pair_end
    uint32_t row_ptr[kMaxTileRows + 8];
    uint2 pairs[kMaxTilePairs + 2];
};

struct TileRing {
    TileStage stage[kTileStages];
    alignas(8) uint64_t full_bar[kTileStages];
    uint32_t next_row[kTileStages];    // rows of the staged tile already claimed
    uint32_t warps_done[kTileStages];  // warps that have left the stage
};

// What a block needs to know about the plan to fetch its tiles.
struct TileSource {
    const uint4 *tiles;
    const uint32_t *row_ptr;
    const uint2 *pairs;
    uint32_t num_tiles;
};

// One thread: fetch tile t into stage s.
__device__ __forceinline__ void tile_issue(TileRing &ring, const TileSource &src, uint32_t t, int s)
{
    const uint4 d = __ldg(src.tiles + t);
    const uint32_t rb = d.x & ~3u, re = (d.y + 1 + 3) & ~3u;  // row pointers [rb, re) cover d.x .. d.y
    const uint32_t jb = d.z & ~1u, je = (d.w + 1) & ~1u;      // pairs [jb, je) cover d.z .. d.w-1
    const uint32_t bytes = 16u + (re - rb) * 4u + (je - jb) * 8u;
    ptx::mbar_expect_tx(&ring.full_bar[s], bytes);
    ptx::bulk_g2s(&ring.stage[s].desc, src.tiles + t, 16u, &ring.full_bar[s]);
    ptx::bulk_g2s(ring.stage[s].row_ptr, src.row_ptr + rb, (re - rb) * 4u, &ring.full_bar[s]);
    if (je > jb) ptx::bulk_g2s(ring.stage[s].pairs, src.pairs + jb, (je - jb) * 8u, &ring.full_bar[s]);
}

// Whole block: set the ring up and ask for the block's first tiles (tile i of block b is b + i * gridDim.x).
// Ends with a block-wide barrier.
__device__ __forceinline__ void tile_ring_start(TileRing &ring, const TileSource &src)
{
    if (threadIdx.x == 0) {
        for (int s = 0; s < kTileStages; ++s) {
            ptx::mbar_init(&ring.full_bar[s], 1);
            ring.next_row[s] = 0;
            ring.warps_done[s] = 0;
        }
        ptx::fence_mbar_init();
        for (int s = 0; s < kTileStages; ++s) {
            const uint64_t t = blockIdx.x + (uint64_t)s * gridDim.x;
            if (t < src.num_tiles) tile_issue(ring, src, (uint32_t)t, s);
        }
    }
    __syncthreads();
}

// Bounded wait for the block's i-th tile.  false = the copy never landed.
__device__ __forceinline__ bool tile_wait(TileRing &ring, uint32_t i)
{
    return ptx::mbar_wait(&ring.full_bar[i % kTileStages], (i / kTileStages) & 1u);
}

// Whole warp: claim `count` consecutive rows of the staged tile; returns the offset of the first inside the tile.
__device__ __forceinline__ uint32_t tile_claim_rows(TileRing &ring, int s, uint32_t count, int lane)
{
    uint32_t r = 0;
    if (lane == 0) r = atomicAdd(&ring.next_row[s], count);
    return __shfl_sync(0xffffffffu, r, 0);
}

// Whole warp: this warp is finished with the block's i-th tile (tile index t); the last warp to say so refills the stage.
__device__ __forceinline__ void tile_release(TileRing &ring, const TileSource &src, uint32_t i, uint64_t t, int lane)
{
    const int s = i % kTileStages;
    __syncwarp();
    if (lane == 0) {
        __threadfence_block();
        if (atomicAdd(&ring.warps_done[s], 1u) == kTileWarps - 1) {
            __threadfence_block();
            ring.warps_done[s] = 0;
            ring.next_row[s] = 0;
            const uint64_t t2 = t + (uint64_t)kTileStages * gridDim.x;
            if (t2 < src.num_tiles) {
                ptx::fence_async_smem();
                tile_issue(ring, src, (uint32_t)t2, s);
            }
        }
    }
}

}  // namespace cutespmm
