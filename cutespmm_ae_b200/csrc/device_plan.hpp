// Kernel argument blocks and launcher prototypes shared by the C ABI and the kernel files.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace cutespmm {

// Opts a kernel in to more than 48 KB of dynamic shared memory.  The attribute belongs to the (function, device)
// pair, so it is set once per device ordinal: a process that drives several GPUs configures each of them.
// (The kernel is a template argument, not a function argument: the table below must be one per kernel, and two
// instantiations of a kernel template share a function-pointer type.)
template <auto Kernel> cudaError_t allow_dynamic_smem(int bytes)
{
    constexpr int kMaxDevices = 64;
    static bool done[kMaxDevices] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < kMaxDevices && done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess && dev >= 0 && dev < kMaxDevices) done[dev] = true;
    return e;
}

// Arguments of the row-gather kernel.
struct RowsArgs {
    const uint32_t *row_ptr;   // M+1 offsets into pairs
    const void *pairs;         // nnz x {col, fp32 bits}
    const void *tiles;         // num_tiles x {row_begin, row_end, pair_begin, pair_end}
    const void *chunks;        // num_chunks x {row, j0, j1, slot}
    const void *long_rows;     // the whole list of long rows {row of C, slot0, slot1, -}, indexed by chunk_owner
    const uint32_t *chunk_owner;  // per scratch slot: index of the long row the chunk belongs to
    uint32_t *arrivals;        // per long row and column slab: chunks finished so far (zero between launches)
    uint32_t num_tiles, num_chunks, split_nnz;
    uint32_t avg_row_nnz;      // nonzeros per row of the whole matrix (picks the kernel's tuning)
    const float *B;            // K x N window, leading dimension ldb
    float *C;                  // M x N window, leading dimension ldc
    float *scratch;            // partial sums, leading dimension ld_scratch
    uint64_t ldb, ldc, ld_scratch;
    uint32_t N;
    uint32_t *status;          // device status word: set to 1 when a bounded wait gives up
    const uint32_t *row_map;   // reordered plan: row r of the work lists is row row_map[r] of C (nullptr: identity)
};

cudaError_t launch_rows(const RowsArgs &a, int sm_count, cudaStream_t s);
int rows_kernel_count(const RowsArgs &a);

// Arguments of the SDDMM kernel (sddmm_kernel.cu): out[j] = (scale ? value of nonzero j : 1) * <X[row of j], Y[column of j]>.
struct SddmmArgs {
    const uint32_t *row_ptr;
    const void *pairs, *tiles, *chunks;  // the plan's nonzeros and its row-kernel work list over every row
    uint32_t num_tiles, num_chunks;
    const float *X, *Y;                  // M x N and K x N, row-major
    uint64_t ldx, ldy;
    float *out;                          // one value per nonzero, in the plan's storage order
    uint32_t N;
    uint32_t scale;                      // 1: multiply by the stored value of A
    uint32_t vec4;                       // 1: X, Y and their leading dimensions allow 16-byte loads
    uint32_t *status;                    // device status word: set to 1 when a bounded wait gives up
};
cudaError_t launch_sddmm(const SddmmArgs &a, int sm_count, cudaStream_t s);

// Arguments of the tensor-core brick kernel.
constexpr int kBrickWarps = 15;  // warps per block; each is an independent pipeline over its own brick range
struct BrickArgs {
    const uint32_t *cols;         // 8 columns per brick slot (+ readable slack of a few groups behind the end)
    const uint32_t *recs;         // brick records (map, flags, panel, values in fragment order): slot k at word k * kBrickRecWords
    const uint32_t *panel_first;  // per brick panel: slot of its first brick (a multiple of 4)
    const uint32_t *panel_last;   // per brick panel: one past the slot of its last brick
    uint32_t num_bricks, num_panels;
    uint32_t M, K;
    const float *B;
    float *C;
    uint64_t ldb, ldc;
    uint32_t N;
    uint32_t round_b;             // 1: round B to tf32 to nearest, 0: truncate
    uint32_t *status;             // device status word: set to 2 when a bounded wait gives up
    const uint32_t *row_map;      // reordered plan: row r of a panel is row row_map[r] of C (nullptr: identity)
};

cudaError_t launch_brick(const BrickArgs &a, int sm_count, cudaStream_t s);
bool brick_supports(uint32_t N, uint64_t ldb, uint64_t ldc, const void *B, const void *C);

// Arguments of the tcgen05 slab kernel (128-row panels).
struct SlabArgs {
    const uint32_t *cols;         // 8 columns per step slot (+ readable slack)
    const uint32_t *recs;         // step records
    const uint32_t *rec_off;      // per step slot (+1) record offsets in 16-byte units (+ slack)
    const uint32_t *panel_first;  // per slab panel: slot of its first step (a multiple of 4)
    const uint32_t *panel_last;   // per slab panel: one past the slot of its last step
    const uint32_t *panel_ids;    // per slab panel: its 128-row panel index
    uint32_t num_panels;
    uint32_t M, K;
    const float *B;
    float *C;
    uint64_t ldb, ldc;
    uint32_t N;                   // a multiple of 128
    uint32_t *status;             // device status word: set to 3 when a bounded wait gives up
};
cudaError_t launch_slab(const SlabArgs &a, int sm_count, cudaStream_t s);
bool slab_supports(uint32_t N, uint64_t ldb, uint64_t ldc, const void *B, const void *C);

// pairs[j] = (cols[j], bits of vals[j]) for j < nnz, two zero pairs behind; *bad |= 1 when a column is >= K
cudaError_t launch_pack_pairs(const uint32_t *cols, const float *vals, void *pairs, uint64_t nnz, uint32_t K, uint32_t *bad, int sm_count,
                              cudaStream_t s);
// Device side of the panel analysis and of the brick packing (device_build.cu).  kDevPanelMax: nonzeros of a panel the
// shared-memory sort takes (32 KB of column indices); 16 rows of at most kMaxSplitNnz nonzeros fit, so every panel
// left out holds a long row and runs on the row kernel whatever its density.
constexpr uint32_t kDevPanelMax = 8192;
cudaError_t launch_set_values(void *pairs, const float *vals, uint64_t nnz, int sm_count, cudaStream_t s);
cudaError_t launch_panel_columns(const uint32_t *row_ptr, const void *pairs, uint32_t M, uint32_t num_panels, uint32_t *ncols,
                                 uint32_t *acols, int sm_count, cudaStream_t s);
cudaError_t launch_panel_max_col(const uint32_t *row_ptr, const void *pairs, uint32_t M, uint32_t num_panels, uint32_t *maxcol, int sm_count,
                                 cudaStream_t s);
cudaError_t launch_brick_fill(const uint32_t *row_ptr, const void *pairs, uint32_t M, const uint32_t *which,
                              const uint32_t *first_slot, const uint32_t *last_slot, uint32_t num_brick_panels, const uint32_t *ncols,
                              const uint32_t *acols, uint32_t *bcols, uint32_t *brecs, int sm_count, cudaStream_t s);


}  // namespace cutespmm
