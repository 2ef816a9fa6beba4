// Packs the panels routed to the tensor-core kernel into the flat brick stream described in
// plan.hpp.  The role of the block/brick writer in the reference (data.cu:212-296) with a different
// layout: a brick spans 8 active columns (the K extent of mma.m16n8k8 / one tcgen05 K step), every
// record is self-describing (map, panel, end-of-panel flag), has a fixed size and starts on a 16-byte
// boundary so one TMA bulk copy fetches it, holds the brick's values already in MMA fragment order,
// and the column list is a separate array the producer lanes read coalesced.  Values are stored
// unrounded (the kernel rounds to tf32 like the reference's cvt.rna, kernel.cu:28-29), so the
// format is lossless.
#include "plan.hpp"

#include <algorithm>
#include <cstring>

namespace cutespmm {

// Which panels go to the brick kernel and which slots of the brick stream each of them owns: every offset follows
// from the per-panel column counts because records have a fixed size.  Fills panel_first_brick / panel_last_brick /
// num_bricks / brick_panels, returns the number of slots and lists the panels (ascending) in `which`.
uint64_t layout_brick_slots(HostPlan &p, const std::vector<uint32_t> &panel_ncols, std::vector<uint32_t> &which)
{
    p.panel_first_brick.clear();
    p.panel_last_brick.clear();
    p.num_bricks = 0;
    p.brick_panels = 0;
    which.clear();
    const uint64_t P = p.num_panels();
    for (uint64_t q = 0; q < P; ++q)
        if (p.row_path[q] == 1 && panel_ncols[q] != 0) which.push_back((uint32_t)q);
    p.brick_panels = which.size();
    p.panel_first_brick.resize(which.size());
    p.panel_last_brick.resize(which.size());
    uint64_t slots = 0;
    for (size_t i = 0; i < which.size(); ++i) {
        const uint32_t nbricks = (panel_ncols[which[i]] + kBrickCols - 1) / kBrickCols;
        p.panel_first_brick[i] = (uint32_t)slots;  // a multiple of 4
        p.panel_last_brick[i] = (uint32_t)(slots + nbricks);
        p.num_bricks += nbricks;
        slots += (nbricks + 3) / 4 * 4;  // groups of 4 slots start on a panel boundary; the surplus slots stay empty
    }
    p.brick_slots = slots;
    return slots;
}

void build_brick_part(HostPlan &p, const std::vector<uint32_t> &panel_ncols)
{
    p.brick_cols.clear();
    p.brick_recs.clear();
    p.brick_rec_off.clear();
    const uint64_t P = p.num_panels();
    std::vector<uint64_t> acol_off(P + 1, 0);
    for (uint64_t q = 0; q < P; ++q)
        acol_off[q + 1] = acol_off[q] + (uint64_t)((panel_ncols[q] + kBlockCols - 1) / kBlockCols) * kBlockCols;
    std::vector<uint32_t> which;  // panels routed to the brick kernel, ascending
    const uint64_t slots = layout_brick_slots(p, panel_ncols, which);
    p.brick_panel_ids = which;
    p.brick_cols.assign(slots * kBrickCols, 0u);
    p.brick_recs.assign(slots * kBrickRecWords, 0u);  // empty slots: zero records
    p.brick_rec_off.resize(slots + 1);
    for (uint64_t k = 0; k <= slots; ++k) p.brick_rec_off[k] = (uint32_t)(k * (kBrickRecWords / 4));
    // pass 2: every panel writes its own slots
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t i = 0; i < (int64_t)which.size(); ++i) {
        const uint64_t q = which[i];
        const uint32_t nc = panel_ncols[q];
        const uint32_t *acols = &p.active_cols[acol_off[q]];
        const uint64_t r0 = q * kPanelRows, r1 = std::min<uint64_t>(p.M, r0 + kPanelRows);
        const uint32_t first = p.panel_first_brick[i], nbricks = p.panel_last_brick[i] - first;
        const uint32_t nslots = (nbricks + 3) / 4 * 4;
        for (uint32_t c = 0; c < nslots * kBrickCols; ++c) p.brick_cols[(size_t)first * kBrickCols + c] = acols[std::min(c, nc - 1)];
        for (uint32_t b = 0; b < nbricks; ++b) {
            uint32_t *rec = &p.brick_recs[(size_t)(first + b) * kBrickRecWords];
            rec[4] = b + 1 == nbricks ? 1u : 0u;
            rec[5] = (uint32_t)q;
        }
        for (uint64_t r = r0; r < r1; ++r) {
            const uint32_t *cursor = acols;
            for (uint32_t j = p.row_ptr[r]; j < p.row_ptr[r + 1]; ++j) {
                const uint32_t col = p.pairs[j].col;  // ascending inside the row
                cursor = std::lower_bound(cursor, acols + nc, col);
                const uint32_t lc = (uint32_t)(cursor - acols);
                uint32_t *rec = &p.brick_recs[(size_t)(first + lc / kBrickCols) * kBrickRecWords];
                const uint32_t bit = (uint32_t)(r - r0) * kBrickCols + lc % kBrickCols;
                float v, acc;
                std::memcpy(&v, &p.pairs[j].val_bits, 4);
                uint32_t *slot = &rec[kBrickRecHeaderWords + brick_frag_index(bit / kBrickCols, bit % kBrickCols)];
                std::memcpy(&acc, slot, 4);
                acc = (rec[bit >> 5] >> (bit & 31)) & 1u ? acc + v : v;  // duplicates of one (row, column) merge here
                std::memcpy(slot, &acc, 4);
                rec[bit >> 5] |= 1u << (bit & 31);
            }
        }
    }
}

}  // namespace cutespmm
