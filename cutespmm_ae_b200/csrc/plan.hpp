// Internal definition of a plan: the device-resident form of A plus the work lists of the two
// kernel families.  Host code only (no CUDA types) so the builder can be compiled and tested on a
// machine without a GPU.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/cutespmm.h"

namespace cutespmm {

constexpr uint32_t kPanelRows = 16;   // row-panel height; HRPB's TM (inc.h:18-20)
constexpr uint32_t kBlockCols = 16;   // active-column block width; HRPB's TK (inc.h:21-23)
constexpr uint32_t kBrickCols = 8;    // one tensor-core brick is 16 rows x 8 active columns (mma m16n8k8)
constexpr uint32_t kRowCost = 4;      // scheduling cost of a row besides its nonzeros (pointer loads, C store)
constexpr uint32_t kDefaultSplitNnz = 256;
constexpr uint32_t kDefaultTileCost = 512;
constexpr uint32_t kMaxTileRows = 256;   // rows of one scheduling tile (bounds the staged row-pointer slice)
constexpr uint32_t kMaxTilePairs = 640;  // nonzeros of one scheduling tile (bounds the staged pair slice)
// Adaptive sizing of the row kernel's work items (when the caller leaves split_nnz and tile_nnz at 0):
constexpr uint32_t kResidentTiles = 560;          // tiles aimed at for a small job: one wave of the kernel's deep tuning (148 SMs x 4 blocks) less 5 %
constexpr uint32_t kMinAdaptiveTileCost = 96;     // smallest tile it makes (8 warps x 12 cost units)
constexpr uint32_t kMaxAdaptiveTileCost = 1024;   // largest: beyond it the job is not small, tiles go back to the default cost
constexpr uint32_t kAdaptiveSplitDivisor = 8192;  // rows are cut from job cost / this nonzeros on: 256 from 2.1 M cost units
constexpr uint32_t kMinAdaptiveSplitNnz = 128;    // ... but never from fewer than this
constexpr uint32_t kMinChunkNnz = 32;             // smallest piece of a cut row
constexpr uint32_t kMaxSplitNnz = 384;   // a row must fit a tile together with a part-filled one
constexpr uint32_t kScratchCols = 512;  // widest N one launch handles; wider products run in column windows

// One nonzero as the row kernel reads it: column index and fp32 bit pattern side by side (8 bytes,
// one coalesced 64-bit load per lane).
struct Pair {
    uint32_t col;
    uint32_t val_bits;
};

// A scheduling tile of the row kernel: rows [row_begin, row_end) whose nonzeros are pairs
// [pair_begin, pair_end); at most kMaxTileRows rows and kMaxTilePairs nonzeros, no long row inside.
struct Tile {
    uint32_t row_begin, row_end, pair_begin, pair_end;
};

constexpr uint32_t kMinBrickPanels = 4440;  // path auto: fewer dense panels than two per warp of a full brick grid go to the row kernel
constexpr uint32_t kPanelTooLarge = 0xffffffffu;  // column count of a panel the device builder did not analyse

// A chunk of a long row: nonzeros [j0, j1) of `row`; its partial result is row `slot` of the scratch.
struct Chunk {
    uint32_t row, j0, j1, slot;
};
// A long row: C[row] = sum of scratch rows [slot0, slot1), added in that order.
struct LongRow {
    uint32_t row, slot0, slot1, pad;
};

// The brick kernel reads one flat stream of bricks (16 rows x 8 active columns each), panel after
// panel.  Brick k owns columns brick_cols[8k .. 8k+8) and the record that starts at 16-byte unit
// brick_rec_off[k] of brick_recs:
//     words 0-3   occupancy map, bit (r*8 + c) set when A[row r of the panel][column c of the brick] is stored
//     word  4     bit 0: last brick of its panel
//     word  5     panel index (rows 16*panel .. 16*panel+15)
//     words 6-7   0
//     words 8-135 the whole 16 x 8 brick (fp32, unrounded), zeros included, in the order the MMA wants it: word
//                 8 + 4*lane + i is A-fragment register i of that lane (brick_frag_index below), so a lane expands
//                 nothing: it loads its four values with one 128-bit read
// Every slot has a record of kBrickRecWords words (empty slots: zeros), brick k at word k * kBrickRecWords.
// (A packed record -- map plus the stored values only, expanded by popcounts as the reference does,
// kernel.cu:20-27 -- is a quarter of the size but was measured 5-11 % slower: the expansion is 50 dependent
// instructions per brick in a kernel that is bound by instruction latency, not by bytes.)
constexpr uint32_t kBrickRecHeaderWords = 8;
constexpr uint32_t kBrickRecWords = kBrickRecHeaderWords + 128;
// mma.m16n8k8 row-major A fragment: lane (g = lane / 4, t = lane % 4) holds a0 = A[g][t], a1 = A[g+8][t],
// a2 = A[g][t+4], a3 = A[g+8][t+4].  Position of element (row r, column c) of a brick in the dense record.
constexpr uint32_t brick_frag_index(uint32_t r, uint32_t c) { return ((r & 7u) * 4u + (c & 3u)) * 4u + (r >> 3) + 2u * (c >> 2); }
constexpr uint32_t kSlabRows = 128;      // rows of a slab panel (the M of one tcgen05.mma)
constexpr uint32_t kSlabMaxVals = 192;   // values one step record may hold (bounds the shared-memory stage)
constexpr uint32_t kSlabMaxRows = 32;    // rows one step record may list (one builder lane each)
constexpr uint32_t kSlabRecHeaderWords = 8;
constexpr uint32_t kSlabRecMaxWords = kSlabRecHeaderWords + kSlabMaxRows + kSlabMaxVals;

struct HostPlan {
    uint64_t M = 0, K = 0, nnz = 0;
    cutespmm_options_t opts{};
    bool device_built = false;  // the nonzeros were packed on the device; the host holds row pointers and work lists only
    bool values_on_device = false;  // cutespmm_plan_set_values replaced the values on the device: the host copy in `pairs` is stale
    bool adaptive_tiling = false;  // the caller left split_nnz and tile_nnz at 0: small jobs get smaller tiles and chunks

    // ---- row reordering (CUTESPMM_REORDER_CLUSTER_ROWS): row r of everything below is row row_map[r] of the caller's
    // matrix, and the kernels write its result to that row of C; empty = identity ----
    std::vector<uint32_t> row_map;

    // ---- row kernel ----
    std::vector<uint32_t> row_ptr;       // M+1, offsets into pairs
    std::vector<Pair> pairs;             // nnz
    std::vector<Tile> tiles;
    std::vector<uint8_t> row_path;       // per panel: 0 = rows kernel, 1 = brick kernel
    std::vector<Chunk> chunks;
    std::vector<LongRow> long_rows;

    // ---- panel analysis (HRPB-compatible view) ----
    std::vector<uint32_t> blocked_row_ptr;  // num_panels+1
    std::vector<uint32_t> active_cols;      // per panel ascending distinct columns, zero-padded to x16

    // largest column index of every 16-row panel (0 for an empty panel): which rows of B a block of rows needs, for
    // the host-buffer call that lets rows of C leave while later rows of B still arrive
    std::vector<uint32_t> panel_max_col;

    // ---- row kernel over every row (used when a product's N does not fit the brick kernel) ----
    std::vector<Tile> tiles_all;
    std::vector<Chunk> chunks_all;
    std::vector<LongRow> long_rows_all;

    // ---- brick kernel ----
    std::vector<uint32_t> brick_cols;     // 8 per brick (a short last brick repeats its last column)
    std::vector<uint32_t> brick_recs;     // records, see above
    std::vector<uint32_t> brick_rec_off;  // per brick slot (+1) the record offset in 16-byte units
    // Brick slots: every panel's bricks are followed by empty slots up to a multiple of 4, so a
    // panel starts on a group-of-4 boundary of brick_cols / brick_rec_off.
    std::vector<uint32_t> panel_first_brick;  // per brick panel: slot of its first brick (multiple of 4)
    std::vector<uint32_t> panel_last_brick;   // per brick panel: one past the slot of its last brick
    uint64_t num_bricks = 0;
    uint64_t brick_panels = 0;
    std::vector<uint32_t> brick_panel_ids;    // device-built plans: the panel index of every brick panel, ascending
    uint64_t brick_slots = 0;                 // slots of the brick stream (bricks plus the empty slots that pad panels to groups of 4)

    // ---- slab kernel (tcgen05): 128-row panels, one record per step of 8 active columns ----
    // Step t owns columns slab_cols[8t .. 8t+8) and the record at 16-byte unit slab_rec_off[t] of slab_recs:
    //     word 0      number of rows with a nonzero in this step | (last step of its panel) << 16
    //     word 1      128-row panel index
    //     word 2      number of values stored (<= kSlabMaxVals), word 3: 0
    //     words 4-7   128-bit map of the rows that have an entry
    //     words 8..   one entry per such row, in row order: row in panel | 8-bit column mask << 8 | index of its first value << 16
    //                 (padded to a multiple of 4 entries), then the values in (row, column) order, padded to x4
    // A step with more than kSlabMaxRows rows or kSlabMaxVals values is stored as several steps over the same 8 columns.
    // Every panel's steps are followed by empty slots up to a multiple of 4 (group-aligned metadata).
    std::vector<uint32_t> slab_cols, slab_recs, slab_rec_off;
    std::vector<uint32_t> slab_first, slab_last;  // per 128-row panel with nonzeros: slot range of its steps
    std::vector<uint32_t> slab_ids;               // ... and its panel index (rows 128*id .. 128*id+127)
    std::vector<uint8_t> slab_path;               // per 128-row panel: 1 = executed by the slab kernel
    uint64_t slab_steps = 0, slab_panels = 0;

    uint64_t num_panels() const { return (M + kPanelRows - 1) / kPanelRows; }
};

// Validates the CSR input and fills every host-side member of `p`.  Returns a cutespmm_status_t;
// on failure `err` holds the message.
int build_host_plan(HostPlan &p, uint64_t M, uint64_t K, const uint64_t *rowPtr, const uint32_t *cols,
                    const float *vals, const cutespmm_options_t *opts, std::string &err);

// The row-kernel part of a plan from the row pointers alone (tiles, chunks of long rows, fix-up list): what a plan
// needs on the host when the nonzeros themselves stay on the device.  p.pairs stays empty and p.device_built is
// set: the HRPB views and the host-side decode are not available for such a plan.
int build_rows_plan_from_row_ptr(HostPlan &p, uint64_t M, uint64_t K, std::vector<uint32_t> &&row_ptr,
                                 const cutespmm_options_t *opts, std::string &err);

// Second half of a device-built plan: with the per-panel distinct-column counts (nullptr: row kernel only) chooses
// each panel's kernel, lays out the brick slots and cuts the work lists.
void finish_device_plan(HostPlan &p, const std::vector<uint32_t> *panel_ncols);
void choose_panel_paths(HostPlan &p, const std::vector<uint32_t> &panel_ncols);

// Rebuilds CSR from the packed arrays (rows-kernel part from pairs, brick part from maps + values).
void decode_host_plan(const HostPlan &p, uint64_t *rowPtr, uint32_t *cols, float *vals);

int partition_rows(uint64_t M, const uint64_t *rowPtr, uint32_t nparts, uint32_t align_rows, uint32_t row_cost,
                   uint64_t *bounds, std::string &err);

}  // namespace cutespmm
