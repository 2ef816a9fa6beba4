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
constexpr uint32_t kDefaultSplitNnz = 1024;
constexpr uint32_t kDefaultTileCost = 1024;
constexpr uint32_t kMaxTileRows = 512;
constexpr uint32_t kScratchCols = 512;  // widest N one launch handles; wider products run in column windows

// One nonzero as the row kernel reads it: column index and fp32 bit pattern side by side (8 bytes,
// one coalesced 64-bit load per lane).
struct Pair {
    uint32_t col;
    uint32_t val_bits;
};

// A chunk of a long row: nonzeros [j0, j1) of `row`; its partial result is row `slot` of the scratch.
struct Chunk {
    uint32_t row, j0, j1, slot;
};
// A long row: C[row] = sum of scratch rows [slot0, slot1), added in that order.
struct LongRow {
    uint32_t row, slot0, slot1, pad;
};

// Work item of the brick kernel: one 16-row panel (or a piece of one).
struct PanelItem {
    uint32_t panel;       // panel index: rows [16*panel, 16*panel+16)
    uint32_t col_begin;   // first entry of this item in brick_cols[]
    uint32_t num_cols;    // active columns of the item (multiple of 8, padded entries repeat a valid column)
    uint32_t val_begin;   // first fp32 of this item in brick_vals[]
    uint32_t map_begin;   // first bitmap (one 128-bit map per brick) in brick_maps[]
    uint32_t flags;       // bit 0: result goes to scratch slot `slot` instead of C
    uint32_t slot;
    uint32_t pad;
};

struct HostPlan {
    uint64_t M = 0, K = 0, nnz = 0;
    cutespmm_options_t opts{};

    // ---- row kernel ----
    std::vector<uint32_t> row_ptr;       // M+1, offsets into pairs
    std::vector<Pair> pairs;             // nnz
    std::vector<uint32_t> tile_rows;     // T+1 row boundaries of the scheduling tiles
    std::vector<uint8_t> row_path;       // per panel: 0 = rows kernel, 1 = brick kernel
    std::vector<Chunk> chunks;
    std::vector<LongRow> long_rows;

    // ---- panel analysis (HRPB-compatible view) ----
    std::vector<uint32_t> blocked_row_ptr;  // num_panels+1
    std::vector<uint32_t> active_cols;      // per panel ascending distinct columns, zero-padded to x16

    // ---- brick kernel ----
    std::vector<PanelItem> panel_items;
    std::vector<uint32_t> brick_cols;   // active columns per item (padded to x8)
    std::vector<uint32_t> brick_maps;   // 4 words per brick, bit (r*8 + c) of the 128-bit map = A[r][c] present
    std::vector<float> brick_vals;      // values in bit order, each brick padded to a multiple of 4 floats
    uint64_t num_bricks = 0;
    uint64_t brick_panels = 0;

    uint64_t num_panels() const { return (M + kPanelRows - 1) / kPanelRows; }
};

// Validates the CSR input and fills every host-side member of `p`.  Returns a cutespmm_status_t;
// on failure `err` holds the message.
int build_host_plan(HostPlan &p, uint64_t M, uint64_t K, const uint64_t *rowPtr, const uint32_t *cols,
                    const float *vals, const cutespmm_options_t *opts, std::string &err);

// Rebuilds CSR from the packed arrays (rows-kernel part from pairs, brick part from maps + values).
void decode_host_plan(const HostPlan &p, uint64_t *rowPtr, uint32_t *cols, float *vals);

int partition_rows(uint64_t M, const uint64_t *rowPtr, uint32_t nparts, uint32_t align_rows, uint32_t row_cost,
                   uint64_t *bounds, std::string &err);

}  // namespace cutespmm
