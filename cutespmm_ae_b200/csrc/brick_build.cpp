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

void build_brick_part(HostPlan &p, const std::vector<uint32_t> &panel_ncols)
{
    p.brick_cols.clear();
    p.brick_recs.clear();
    p.brick_rec_off.clear();
    p.panel_first_brick.clear();
    p.panel_last_brick.clear();
    p.num_bricks = 0;
    p.brick_panels = 0;
    const uint64_t P = p.num_panels();
    uint64_t acol_off = 0;
    std::vector<float> img;
    std::vector<uint8_t> present;
    for (uint64_t q = 0; q < P; ++q) {
        const uint32_t nc = panel_ncols[q];
        const uint64_t my_off = acol_off;
        acol_off += (uint64_t)((nc + kBlockCols - 1) / kBlockCols) * kBlockCols;
        if (p.row_path[q] != 1 || nc == 0) continue;
        ++p.brick_panels;
        p.panel_first_brick.push_back((uint32_t)p.brick_rec_off.size());  // slot index, a multiple of 4
        const uint32_t *acols = &p.active_cols[my_off];
        const uint64_t r0 = q * kPanelRows, r1 = std::min<uint64_t>(p.M, r0 + kPanelRows);
        const uint32_t nbricks = (nc + kBrickCols - 1) / kBrickCols;
        const uint32_t nslots = (nbricks + 3) / 4 * 4;  // the panel's brick slots: groups of 4 start on a panel boundary
        for (uint32_t c = 0; c < nslots * kBrickCols; ++c) p.brick_cols.push_back(acols[std::min(c, nc - 1)]);
        img.assign((size_t)nbricks * 128, 0.0f);
        present.assign((size_t)nbricks * 128, 0);
        for (uint64_t r = r0; r < r1; ++r) {
            const uint32_t *cursor = acols;
            for (uint32_t j = p.row_ptr[r]; j < p.row_ptr[r + 1]; ++j) {
                const uint32_t col = p.pairs[j].col;  // ascending inside the row
                cursor = std::lower_bound(cursor, acols + nc, col);
                const uint32_t lc = (uint32_t)(cursor - acols);
                float v;
                std::memcpy(&v, &p.pairs[j].val_bits, 4);
                const size_t at = (size_t)(lc / kBrickCols) * 128 + (r - r0) * kBrickCols + lc % kBrickCols;
                img[at] += v;  // duplicates of one (row, column) merge here
                present[at] = 1;
            }
        }
        for (uint32_t b = 0; b < nbricks; ++b) {
            p.brick_rec_off.push_back((uint32_t)(p.brick_recs.size() / 4));
            uint32_t head[kBrickRecHeaderWords] = {0, 0, 0, 0, b + 1 == nbricks ? 1u : 0u, (uint32_t)q, 0, 0};
            for (uint32_t bit = 0; bit < 128; ++bit)
                if (present[(size_t)b * 128 + bit]) head[bit >> 5] |= 1u << (bit & 31);
            p.brick_recs.insert(p.brick_recs.end(), head, head + kBrickRecHeaderWords);
            const size_t base = p.brick_recs.size();
            p.brick_recs.resize(base + 128, 0u);
            for (uint32_t bit = 0; bit < 128; ++bit)
                if (present[(size_t)b * 128 + bit])
                    std::memcpy(&p.brick_recs[base + brick_frag_index(bit / kBrickCols, bit % kBrickCols)], &img[(size_t)b * 128 + bit], 4);
            ++p.num_bricks;
        }
        for (uint32_t b = nbricks; b < nslots; ++b) {  // empty slots
            p.brick_rec_off.push_back((uint32_t)(p.brick_recs.size() / 4));
            p.brick_recs.resize(p.brick_recs.size() + kBrickRecWords, 0u);
        }
        p.panel_last_brick.push_back((uint32_t)(p.brick_rec_off.size() - (nslots - nbricks)));
    }
    p.brick_rec_off.push_back((uint32_t)(p.brick_recs.size() / 4));
}

}  // namespace cutespmm
