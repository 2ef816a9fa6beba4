// Packs 128-row panels for the tcgen05 slab kernel: per panel its ascending active columns in steps
// of 8, per step a record listing the rows that have a nonzero there (row, 8-bit column mask, value
// offset) and the values.  Same idea as the reference's active-column blocks (data.cu:188-296) at
// the granularity of the Blackwell tensor core: one step is one tcgen05.mma of 128 x N x 8.
#include "plan.hpp"

#include <algorithm>
#include <cstring>

namespace cutespmm {

namespace {
struct Ent {
    uint32_t step, row, col;  // step of the panel, row in panel, column in step
    float val;
};
}  // namespace

void build_slab_part(HostPlan &p)
{
    p.slab_cols.clear(); p.slab_recs.clear(); p.slab_rec_off.clear();
    p.slab_first.clear(); p.slab_last.clear(); p.slab_ids.clear();
    p.slab_steps = 0; p.slab_panels = 0;
    const uint64_t SP = (p.M + kSlabRows - 1) / kSlabRows;
    std::vector<uint32_t> acols;
    std::vector<Ent> ents, sorted;
    std::vector<uint32_t> count;
    for (uint64_t q = 0; q < SP; ++q) {
        if (!p.slab_path[q]) continue;
        const uint64_t r0 = q * kSlabRows, r1 = std::min<uint64_t>(p.M, r0 + kSlabRows);
        const uint32_t j0 = p.row_ptr[r0], j1 = p.row_ptr[r1];
        if (j0 == j1) continue;
        acols.resize(j1 - j0);
        for (uint32_t j = j0; j < j1; ++j) acols[j - j0] = p.pairs[j].col;
        std::sort(acols.begin(), acols.end());
        acols.erase(std::unique(acols.begin(), acols.end()), acols.end());
        const uint32_t nc = (uint32_t)acols.size(), nsteps = (nc + 7) / 8;
        // entries in (row, column) order; equal (row, column) pairs merge
        ents.clear();
        for (uint64_t r = r0; r < r1; ++r) {
            const uint32_t *cursor = acols.data();
            for (uint32_t j = p.row_ptr[r]; j < p.row_ptr[r + 1]; ++j) {
                cursor = std::lower_bound(cursor, static_cast<const uint32_t *>(acols.data() + nc), p.pairs[j].col);
                const uint32_t lc = (uint32_t)(cursor - acols.data());
                float v;
                std::memcpy(&v, &p.pairs[j].val_bits, 4);
                if (!ents.empty() && ents.back().row == r - r0 && ents.back().step == lc / 8 && ents.back().col == lc % 8)
                    ents.back().val += v;
                else
                    ents.push_back(Ent{lc / 8, (uint32_t)(r - r0), lc % 8, v});
            }
        }
        // stable counting sort by step keeps (row, column) order inside a step
        count.assign(nsteps + 1, 0);
        for (const Ent &e : ents) ++count[e.step + 1];
        for (uint32_t t = 0; t < nsteps; ++t) count[t + 1] += count[t];
        sorted.resize(ents.size());
        {
            std::vector<uint32_t> pos(count.begin(), count.end() - 1);
            for (const Ent &e : ents) sorted[pos[e.step]++] = e;
        }
        ++p.slab_panels;
        p.slab_first.push_back((uint32_t)p.slab_rec_off.size());
        p.slab_ids.push_back((uint32_t)q);
        const size_t first_rec_of_panel = p.slab_rec_off.size();
        for (uint32_t t = 0; t < nsteps; ++t) {
            uint32_t a = count[t];
            const uint32_t b = count[t + 1];
            while (a < b) {  // one record per <= kSlabMaxRows rows and <= kSlabMaxVals values, cut at a row boundary
                uint32_t e = a, nv = 0, nr = 0;
                while (e < b) {
                    uint32_t f = e;
                    while (f < b && sorted[f].row == sorted[e].row) ++f;
                    if (nv + (f - e) > kSlabMaxVals || nr == kSlabMaxRows) break;
                    nv += f - e;
                    ++nr;
                    e = f;
                }
                // header + entries
                std::vector<uint32_t> entries;
                std::vector<uint32_t> vals;
                for (uint32_t i = a; i < e;) {
                    uint32_t f = i, mask = 0;
                    const uint32_t off = (uint32_t)vals.size();
                    while (f < e && sorted[f].row == sorted[i].row) {
                        mask |= 1u << sorted[f].col;
                        uint32_t vb;
                        std::memcpy(&vb, &sorted[f].val, 4);
                        vals.push_back(vb);
                        ++f;
                    }
                    entries.push_back(sorted[i].row | (mask << 8) | (off << 16));
                    i = f;
                }
                p.slab_rec_off.push_back((uint32_t)(p.slab_recs.size() / 4));
                const uint32_t cnt = (uint32_t)entries.size();
                p.slab_recs.push_back(cnt);  // "last step" flag is set below, once the panel's last record is known
                p.slab_recs.push_back((uint32_t)q);
                p.slab_recs.push_back((uint32_t)vals.size());
                p.slab_recs.push_back(0u);
                uint32_t rowmap[4] = {0, 0, 0, 0};
                for (uint32_t en : entries) rowmap[(en & 0xffu) >> 5] |= 1u << (en & 31u);
                p.slab_recs.insert(p.slab_recs.end(), rowmap, rowmap + 4);
                while (entries.size() % 4) entries.push_back(0u);
                while (vals.size() % 4) vals.push_back(0u);
                p.slab_recs.insert(p.slab_recs.end(), entries.begin(), entries.end());
                p.slab_recs.insert(p.slab_recs.end(), vals.begin(), vals.end());
                for (uint32_t c = 0; c < 8; ++c) p.slab_cols.push_back(acols[std::min(t * 8 + c, nc - 1)]);
                ++p.slab_steps;
                a = e;
            }
        }
        // flag the panel's last record, then pad the slot range to a multiple of 4
        p.slab_recs[(size_t)p.slab_rec_off.back() * 4] |= 1u << 16;
        p.slab_last.push_back((uint32_t)p.slab_rec_off.size());
        while ((p.slab_rec_off.size() - first_rec_of_panel) % 4 || p.slab_rec_off.size() % 4) {
            p.slab_rec_off.push_back((uint32_t)(p.slab_recs.size() / 4));
            for (uint32_t c = 0; c < 8; ++c) p.slab_cols.push_back(acols[nc - 1]);
        }
    }
    p.slab_rec_off.push_back((uint32_t)(p.slab_recs.size() / 4));
}

}  // namespace cutespmm
