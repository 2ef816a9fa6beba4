// Packs the panels routed to the tensor-core kernel into bricks: per panel its ascending active
// columns (padded to a multiple of 8), per 16x8 brick a 128-bit occupancy map and the values in
// map order.  The role of the block/brick writer in the reference (data.cu:212-296), with a
// different layout: one brick spans 8 active columns (the K extent of mma.m16n8k8), maps and values
// live in separate arrays so both can be fetched with 16-byte aligned bulk copies, and there are
// no per-block headers chaining to the next block.
#include "plan.hpp"

#include <algorithm>
#include <cstring>

namespace cutespmm {

constexpr uint32_t kMaxItemCols = 1024;  // active columns one work item covers; wider panels are cut

void build_brick_part(HostPlan &p, const std::vector<uint32_t> &panel_ncols)
{
    p.panel_items.clear();
    p.brick_cols.clear();
    p.brick_maps.clear();
    p.brick_vals.clear();
    p.num_bricks = 0;
    p.brick_panels = 0;
    const uint64_t P = p.num_panels();
    // offsets of each panel's active columns inside active_cols (zero-padded to x16 per panel)
    uint64_t acol_off = 0;
    std::vector<uint32_t> local;  // column -> local index, via binary search on the sorted list
    for (uint64_t q = 0; q < P; ++q) {
        const uint32_t nc = panel_ncols[q];
        const uint64_t my_off = acol_off;
        acol_off += (uint64_t)((nc + kBlockCols - 1) / kBlockCols) * kBlockCols;
        if (!p.row_path[q]) continue;
        ++p.brick_panels;
        const uint32_t *acols = &p.active_cols[my_off];
        const uint64_t r0 = q * kPanelRows, r1 = std::min<uint64_t>(p.M, r0 + kPanelRows);
        const uint32_t npieces = (nc + kMaxItemCols - 1) / kMaxItemCols;
        uint32_t slot_base = 0;
        if (npieces > 1) {
            // rows of the scratch for this panel: [row in panel][piece]; one fix-up entry per row
            slot_base = (uint32_t)p.chunks.size();
            for (uint32_t r = 0; r < kPanelRows; ++r) {
                for (uint32_t k = 0; k < npieces; ++k)
                    p.chunks.push_back(Chunk{(uint32_t)(r0 + r), 0, 0, (uint32_t)p.chunks.size()});  // slot placeholder, no nonzeros
                if (r0 + r < p.M)
                    p.long_rows.push_back(LongRow{(uint32_t)(r0 + r), slot_base + r * npieces, slot_base + (r + 1) * npieces, 0});
            }
        }
        for (uint32_t piece = 0; piece < npieces; ++piece) {
            const uint32_t c0 = piece * kMaxItemCols, c1 = std::min(nc, c0 + kMaxItemCols);
            const uint32_t ncp = (c1 - c0 + kBrickCols - 1) / kBrickCols * kBrickCols;
            PanelItem it{};
            it.panel = (uint32_t)q;
            it.col_begin = (uint32_t)p.brick_cols.size();
            it.num_cols = ncp;
            it.val_begin = (uint32_t)p.brick_vals.size();
            it.map_begin = (uint32_t)(p.brick_maps.size() / 4);
            it.flags = npieces > 1 ? 1u : 0u;
            it.slot = slot_base + piece;
            it.pad = npieces;  // stride between consecutive rows' slots
            for (uint32_t c = c0; c < c0 + ncp; ++c) p.brick_cols.push_back(acols[std::min(c, c1 - 1)]);
            const uint32_t nbricks = ncp / kBrickCols;
            // dense image of this piece, brick by brick
            std::vector<float> img((size_t)nbricks * 128, 0.0f);
            std::vector<uint8_t> present((size_t)nbricks * 128, 0);
            for (uint64_t r = r0; r < r1; ++r) {
                for (uint32_t j = p.row_ptr[r]; j < p.row_ptr[r + 1]; ++j) {
                    const uint32_t col = p.pairs[j].col;
                    const uint32_t lc = (uint32_t)(std::lower_bound(acols, acols + nc, col) - acols);
                    if (lc < c0 || lc >= c1) continue;
                    const uint32_t b = (lc - c0) / kBrickCols, cc = (lc - c0) % kBrickCols;
                    float v;
                    std::memcpy(&v, &p.pairs[j].val_bits, 4);
                    const size_t at = (size_t)b * 128 + (r - r0) * kBrickCols + cc;
                    img[at] += v;  // duplicates of one (row, column) merge here
                    present[at] = 1;
                }
            }
            for (uint32_t b = 0; b < nbricks; ++b) {
                uint32_t map[4] = {0, 0, 0, 0};
                uint32_t cnt = 0;
                for (uint32_t bit = 0; bit < 128; ++bit) {
                    if (!present[(size_t)b * 128 + bit]) continue;
                    map[bit >> 5] |= 1u << (bit & 31);
                    p.brick_vals.push_back(img[(size_t)b * 128 + bit]);
                    ++cnt;
                }
                while (cnt % 4) { p.brick_vals.push_back(0.0f); ++cnt; }
                p.brick_maps.insert(p.brick_maps.end(), map, map + 4);
                ++p.num_bricks;
            }
            p.panel_items.push_back(it);
        }
    }
}

}  // namespace cutespmm
