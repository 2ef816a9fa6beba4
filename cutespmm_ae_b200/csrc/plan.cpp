// Host preprocessing: CSR -> device-ready arrays and nnz-balanced work lists.
//
// Takes the place of HRPB::DATASTRUCT (reference data.cu:94-335) and of SPMM_TC::partition
// (reference spmm.cu:691-822).  Differences that matter to a caller:
//   * memory is proportional to the input (the reference allocates (M/16)*(K/16)+1 offsets,
//     data.cu:91, and three K*64-word scratch arrays, data.cu:95-98);
//   * correct for any number of OpenMP threads (the reference indexes per-thread scratch by the
//     thread id it asked for, data.cu:105-113);
//   * rows need not be sorted; every nonzero is kept;
//   * the work list is balanced by nonzeros and does not depend on a per-GPU occupancy table
//     (spmm.cu:290-690 has no entry for a 148-SM part).
#include "plan.hpp"

#include <algorithm>
#include <cstring>
#include <numeric>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace cutespmm {

void build_brick_part(HostPlan &p, const std::vector<uint32_t> &panel_ncols);  // brick_build.cpp
uint64_t layout_brick_slots(HostPlan &p, const std::vector<uint32_t> &panel_ncols, std::vector<uint32_t> &which);
void build_slab_part(HostPlan &p);                                             // slab_build.cpp

// Returns whether the caller left both scheduling sizes (split_nnz, tile_nnz) to the library.
static bool fill_default_options(cutespmm_options_t &o, const cutespmm_options_t *in)
{
    std::memset(&o, 0, sizeof(o));
    if (in) {
        const size_t n = std::min<size_t>(in->struct_size ? in->struct_size : sizeof(o), sizeof(o));
        std::memcpy(&o, in, n);
    }
    o.struct_size = sizeof(o);
    const bool sizes_left_open = o.split_nnz == 0 && o.tile_nnz == 0;
    if (o.split_nnz == 0) o.split_nnz = kDefaultSplitNnz;
    if (o.split_nnz > kMaxSplitNnz) o.split_nnz = kMaxSplitNnz;
    if (o.tile_nnz == 0) o.tile_nnz = kDefaultTileCost;
    if (o.brick_density <= 0.0f) o.brick_density = 0.125f;
    if (o.min_brick_panels == 0) o.min_brick_panels = kMinBrickPanels;
    return sizes_left_open;
}

// Distinct columns of every 16-row panel, ascending: the HRPB view (data.cu:116-149 counts them,
// data.cu:188-209 sorts them).  Fills blocked_row_ptr / active_cols and returns the per-panel counts.
static std::vector<uint32_t> analyze_panels(HostPlan &p)
{
    const uint64_t P = p.num_panels();
    std::vector<uint32_t> ncols(P, 0);
    // pass 1: count distinct columns per panel
    std::vector<uint64_t> col_off(P + 1, 0);
#pragma omp parallel
    {
        std::vector<uint32_t> buf;
#pragma omp for schedule(dynamic, 256)
        for (int64_t q = 0; q < (int64_t)P; ++q) {
            const uint64_t r0 = (uint64_t)q * kPanelRows, r1 = std::min<uint64_t>(p.M, r0 + kPanelRows);
            const uint32_t j0 = p.row_ptr[r0], j1 = p.row_ptr[r1];
            buf.resize(j1 - j0);
            for (uint32_t j = j0; j < j1; ++j) buf[j - j0] = p.pairs[j].col;
            std::sort(buf.begin(), buf.end());
            ncols[q] = (uint32_t)(std::unique(buf.begin(), buf.end()) - buf.begin());
        }
    }
    p.panel_max_col.assign(P, 0u);
    p.blocked_row_ptr.assign(P + 1, 0);
    for (uint64_t q = 0; q < P; ++q) {
        const uint32_t nb = (ncols[q] + kBlockCols - 1) / kBlockCols;
        p.blocked_row_ptr[q + 1] = p.blocked_row_ptr[q] + nb;
        col_off[q + 1] = col_off[q] + (uint64_t)nb * kBlockCols;
    }
    p.active_cols.assign(col_off[P], 0u);
    // pass 2: write them
#pragma omp parallel
    {
        std::vector<uint32_t> buf;
#pragma omp for schedule(dynamic, 256)
        for (int64_t q = 0; q < (int64_t)P; ++q) {
            const uint64_t r0 = (uint64_t)q * kPanelRows, r1 = std::min<uint64_t>(p.M, r0 + kPanelRows);
            const uint32_t j0 = p.row_ptr[r0], j1 = p.row_ptr[r1];
            buf.resize(j1 - j0);
            for (uint32_t j = j0; j < j1; ++j) buf[j - j0] = p.pairs[j].col;
            std::sort(buf.begin(), buf.end());
            const size_t n = std::unique(buf.begin(), buf.end()) - buf.begin();
            std::copy(buf.begin(), buf.begin() + n, p.active_cols.begin() + col_off[q]);
            if (n) p.panel_max_col[q] = buf[n - 1];
        }
    }
    return ncols;
}

// Cuts the rows that the row kernel executes into tiles of about equal cost (nonzeros + kRowCost per
// row).  A tile is a run of consecutive rows inside one stretch of row-kernel panels, bounded so that
// its row pointers and pairs fit the kernel's shared-memory stage.  A long row ends the running
// tile and is not part of any: its nonzeros are executed as chunks.
static void build_tiles(const HostPlan &p, bool all_rows, std::vector<Tile> &tiles, std::vector<Chunk> &chunks,
                        std::vector<LongRow> &long_rows)
{
    const uint64_t P = p.num_panels();
    uint32_t split = p.opts.split_nnz;
    uint64_t target = p.opts.tile_nnz;
    bool latency_bound = false;
    if (p.adaptive_tiling) {
        // The default sizes (tiles of cost 512, chunks of 256 nonzeros) keep the per-item overhead small when the grid is
        // many waves long.  A small job is a handful of memory latencies long, and then the longest chain of dependent
        // gathers of one warp IS the run time: a 256-nonzero chunk is 64 steps of four loads, about 30 us, when the
        // rest of a 200 000-nonzero matrix is done in 10.  So the work is cut finer the smaller the job: tiles so that
        // one resident wave of blocks holds them all, rows cut from a shorter length on (not below 128: a piece costs
        // about eight latencies of its own -- descriptor, pairs, arrival count, the sum -- so shorter rows are quicker
        // whole), and a cut row into pieces of about sqrt(length / 2) nonzeros: the chain is a piece's gathers followed
        // by the sum of the pieces, the sum runs a few slots per step, and that length makes the two about equal.
        uint64_t total = 0;
        for (uint64_t q = 0; q < P; ++q) {
            if (!all_rows && p.row_path[q]) continue;
            const uint64_t r0 = q * kPanelRows, r1 = std::min<uint64_t>(p.M, r0 + kPanelRows);
            total += (p.row_ptr[r1] - p.row_ptr[r0]) + (r1 - r0) * kRowCost;
        }
        if (total / kResidentTiles <= kMaxAdaptiveTileCost) target = std::max<uint64_t>(kMinAdaptiveTileCost, total / kResidentTiles);
        if (total / kAdaptiveSplitDivisor < split) {
            latency_bound = true;
            split = (uint32_t)std::max<uint64_t>(kMinAdaptiveSplitNnz, total / kAdaptiveSplitDivisor);
        }
    }
    auto piece_of = [&](uint32_t len) {  // nonzeros per chunk of a row of `len` nonzeros that is being cut
        if (!latency_bound) return split;
        uint32_t s = 1;
        while ((uint64_t)s * s * 2 < len) ++s;  // ceil(sqrt(len / 2)): a latency-bound job has fewer than 2.1 M nonzeros, about 1 000 steps at most
        return std::min(split, std::max(kMinChunkNnz, s));
    };
    tiles.clear();
    chunks.clear();
    long_rows.clear();
    std::vector<Tile> row_tiles;
    uint64_t q = 0;
    while (q < P) {
        if (!all_rows && p.row_path[q]) { ++q; continue; }
        uint64_t q1 = q;
        while (q1 < P && (all_rows || !p.row_path[q1])) ++q1;
        const uint64_t r_end = std::min<uint64_t>(p.M, q1 * kPanelRows);
        uint64_t r = q * kPanelRows;
        uint64_t begin = r, cost = 0;
        auto close = [&](uint64_t end) {
            if (end > begin) row_tiles.push_back(Tile{(uint32_t)begin, (uint32_t)end, p.row_ptr[begin], p.row_ptr[end]});
            cost = 0;
        };
        for (; r < r_end; ++r) {
            const uint32_t len = p.row_ptr[r + 1] - p.row_ptr[r];
            if (len > split) {
                close(r);
                begin = r + 1;
                LongRow lr{p.row_map.empty() ? (uint32_t)r : p.row_map[r], (uint32_t)chunks.size(), 0, 0};  // the row of C the sum goes to
                const uint32_t piece = piece_of(len);
                for (uint32_t j = p.row_ptr[r]; j < p.row_ptr[r + 1]; j += piece)
                    chunks.push_back(Chunk{(uint32_t)r, j, std::min<uint32_t>(j + piece, p.row_ptr[r + 1]),
                                           (uint32_t)chunks.size()});
                lr.slot1 = (uint32_t)chunks.size();
                long_rows.push_back(lr);
                continue;
            }
            if (p.row_ptr[r + 1] - p.row_ptr[begin] > kMaxTilePairs || r - begin >= kMaxTileRows) {
                close(r);
                begin = r;
            }
            cost += len + kRowCost;
            if (cost >= target) {
                close(r + 1);
                begin = r + 1;
            }
        }
        close(r_end);
        q = q1;
    }
    tiles = std::move(row_tiles);
}

static void apply_row_order(HostPlan &p, std::vector<uint32_t> &&order);

// CUTESPMM_REORDER_CLUSTER_ROWS: reorders the rows of the plan so that rows with similar column sets are neighbours.
// Rows are sorted by their first kClusterKeyCols column indices (columns are ascending inside a row), a row with
// fewer columns before its extensions, ties by original position (stable, so an already good order survives); empty
// rows go last.  The role of the "find the most similar row" step the reference sketches (inc/CSR.hpp:612-679, an
// O(rows^2) search) at the cost of one sort.  Rewrites row_ptr / pairs in the new order and records row_map.
static void cluster_rows(HostPlan &p)
{
    constexpr uint32_t kClusterKeyCols = 8;
    const uint64_t M = p.M;
    if (M < 2) return;
    std::vector<uint32_t> order(M);
    std::iota(order.begin(), order.end(), 0u);
    const std::vector<uint32_t> &rp = p.row_ptr;
    const std::vector<Pair> &pr = p.pairs;
    auto less = [&](uint32_t a, uint32_t b) {
        const uint32_t la = rp[a + 1] - rp[a], lb = rp[b + 1] - rp[b];
        if ((la == 0) != (lb == 0)) return lb == 0;  // empty rows last
        const uint32_t n = std::min(std::min(la, lb), kClusterKeyCols);
        for (uint32_t i = 0; i < n; ++i) {
            const uint32_t ca = pr[rp[a] + i].col, cb = pr[rp[b] + i].col;
            if (ca != cb) return ca < cb;
        }
        if (n < kClusterKeyCols && la != lb) return la < lb;
        return a < b;
    };
    std::stable_sort(order.begin(), order.end(), less);
    apply_row_order(p, std::move(order));
}

// Applies a row order (order[new position] = original row) to row_ptr / pairs and records it as row_map.
static void apply_row_order(HostPlan &p, std::vector<uint32_t> &&order)
{
    const uint64_t M = p.M;
    bool identity = true;
    for (uint64_t r = 0; r < M && identity; ++r) identity = order[r] == r;
    if (identity) return;
    const std::vector<uint32_t> &rp = p.row_ptr;
    std::vector<uint32_t> new_rp(M + 1, 0);
    for (uint64_t r = 0; r < M; ++r) new_rp[r + 1] = new_rp[r] + (rp[order[r] + 1] - rp[order[r]]);
    std::vector<Pair> new_pairs(p.nnz);
#pragma omp parallel for schedule(dynamic, 4096)
    for (int64_t r = 0; r < (int64_t)M; ++r)
        std::copy(p.pairs.begin() + rp[order[r]], p.pairs.begin() + rp[order[r] + 1], new_pairs.begin() + new_rp[r]);
    p.row_ptr = std::move(new_rp);
    p.pairs = std::move(new_pairs);
    p.row_map = std::move(order);
}

// CUTESPMM_REORDER_SIMILAR_ROWS: grows every 16-row panel greedily.  A panel starts from the first unplaced row;
// then, fifteen times, the unplaced row with the most columns already in the panel's column set joins it.  Ties go to
// the row whose shared columns are shared with the most rows of the panel (the sum over its columns of how many panel
// rows have the column: this is what makes a panel grow as a compact patch instead of a chain), then to the row that
// brings the fewest new columns, then to the lowest index.  Both scores are kept up to date through the
// column-to-rows index: every row that has a column of the row just placed gains one.  The first score is
// the pairwise similarity the reference defines (row_simlarity, inc/CSR.hpp:612-662) used the way its
// find_most_similar (inc/CSR.hpp:664-679) would be, without the all-pairs search.  Columns named by more than
// kMaxFanout rows are left out of the index (a hub column makes every row look similar and costs the most to follow).
static void group_similar_rows(HostPlan &p)
{
    constexpr uint32_t kMaxFanout = 96;
    const uint64_t M = p.M, K = p.K;
    if (M <= kPanelRows || p.nnz == 0) return;
    const std::vector<uint32_t> &rp = p.row_ptr;
    const std::vector<Pair> &pr = p.pairs;
    // column -> rows index (CSC pattern) over the columns of modest fan-out
    std::vector<uint32_t> cdeg(K, 0u);
    for (const Pair &e : pr) ++cdeg[e.col];
    std::vector<uint64_t> cptr(K + 1, 0);
    for (uint64_t c = 0; c < K; ++c) cptr[c + 1] = cptr[c] + (cdeg[c] <= kMaxFanout ? cdeg[c] : 0);
    std::vector<uint32_t> crow(cptr[K]);
    {
        std::vector<uint64_t> cur(cptr.begin(), cptr.end() - 1);
        for (uint64_t r = 0; r < M; ++r)
            for (uint32_t j = rp[r]; j < rp[r + 1]; ++j)
                if (cdeg[pr[j].col] <= kMaxFanout) crow[cur[pr[j].col]++] = (uint32_t)r;
    }
    std::vector<uint8_t> placed(M, 0);
    std::vector<uint32_t> in_set(K, 0u);  // panel stamp of the panel whose column set holds the column
    std::vector<uint32_t> score(M, 0u), weight(M, 0u), touched, order;
    order.reserve(M);
    uint64_t next_seed = 0;
    uint32_t stamp = 0;
    auto add_row = [&](uint32_t r) {
        placed[r] = 1;
        order.push_back(r);
        for (uint32_t j = rp[r]; j < rp[r + 1]; ++j) {
            const uint32_t c = pr[j].col;
            const bool fresh = in_set[c] != stamp;
            in_set[c] = stamp;
            for (uint64_t i = cptr[c]; i < cptr[c + 1]; ++i) {
                const uint32_t q = crow[i];
                if (placed[q]) continue;
                if (weight[q]++ == 0) touched.push_back(q);
                if (fresh) ++score[q];
            }
        }
    };
    while (order.size() < M) {
        while (placed[next_seed]) ++next_seed;
        ++stamp;
        touched.clear();
        add_row((uint32_t)next_seed);
        for (uint32_t i = 1; i < kPanelRows && order.size() < M; ++i) {
            uint32_t best = 0xffffffffu, best_score = 0, best_weight = 0, best_new = 0;
            size_t keep = 0;
            for (size_t t = 0; t < touched.size(); ++t) {
                const uint32_t q = touched[t];
                if (placed[q]) continue;
                touched[keep++] = q;
                const uint32_t sc = score[q], wt = weight[q], fresh = (rp[q + 1] - rp[q]) - std::min(sc, rp[q + 1] - rp[q]);
                const bool better = sc != best_score ? sc > best_score
                                    : wt != best_weight ? wt > best_weight
                                    : fresh != best_new ? fresh < best_new
                                                        : q < best;
                if (best == 0xffffffffu || better) {
                    best = q; best_score = sc; best_weight = wt; best_new = fresh;
                }
            }
            touched.resize(keep);
            if (best == 0xffffffffu) {  // nothing shares a column with the panel: take the next unplaced row
                while (next_seed < M && placed[next_seed]) ++next_seed;
                if (next_seed >= M) break;
                best = (uint32_t)next_seed;
            }
            add_row(best);
        }
        for (uint32_t q : touched) score[q] = weight[q] = 0;
    }
    apply_row_order(p, std::move(order));
}

// Which kernel executes each 16-row panel (row_path: 0 = row kernel, 1 = brick kernel), from the panel's nonzero
// count, its number of distinct columns and its longest row.  A panel whose column count is kPanelTooLarge was not
// analysed (the device builder skips panels beyond its shared-memory sort) and stays with the row kernel.
void choose_panel_paths(HostPlan &p, const std::vector<uint32_t> &panel_ncols)
{
    const uint64_t P = p.num_panels();
    p.row_path.assign(P, 0);
    if (p.opts.path == CUTESPMM_PATH_ROWS) return;
#pragma omp parallel for schedule(static)
    for (int64_t q = 0; q < (int64_t)P; ++q) {
        const uint64_t r0 = (uint64_t)q * kPanelRows, r1 = std::min<uint64_t>(p.M, r0 + kPanelRows);
        const uint32_t n = p.row_ptr[r1] - p.row_ptr[r0];
        if (n == 0 || panel_ncols[q] == kPanelTooLarge) continue;  // empty panels: the row kernel writes their zeros
        if (p.opts.path == CUTESPMM_PATH_BRICK) { p.row_path[q] = 1; continue; }
        if (p.opts.path == CUTESPMM_PATH_SLAB) continue;  // decided per 128-row panel by the caller
        // AUTO: fill of the panel's 16 x (8*ceil(ncols/8)) dense image
        const uint32_t padded = (panel_ncols[q] + kBrickCols - 1) / kBrickCols * kBrickCols;
        const float fill = (float)n / (float)(kPanelRows * padded);
        bool long_row = false;
        for (uint64_t r = r0; r < r1; ++r) long_row |= (p.row_ptr[r + 1] - p.row_ptr[r]) > p.opts.split_nnz;
        p.row_path[q] = (fill >= p.opts.brick_density && !long_row) ? 1 : 0;
    }
    if (p.opts.path == CUTESPMM_PATH_AUTO) {
        // The brick kernel is a grid of independent per-warp pipelines, one panel at a time each: below about two
        // panels per warp of a full grid (148 SMs x 15 warps) most of them idle while the others walk their panel
        // brick by brick, and a second launch for the remaining rows costs more than it saves.  Measured on the 43
        // matrices the reference ships (10 k - 80 k rows): the row kernel alone is 1.3 - 1.4x faster than the mixed
        // plan there, while the two synthetic brick workloads (12 000 and 16 384 panels) stay on bricks.
        uint64_t bricks = 0;
        for (uint64_t q = 0; q < P; ++q) bricks += p.row_path[q] == 1;
        if (bricks < p.opts.min_brick_panels) std::fill(p.row_path.begin(), p.row_path.end(), (uint8_t)0);
    }
}

int build_rows_plan_from_row_ptr(HostPlan &p, uint64_t M, uint64_t K, std::vector<uint32_t> &&row_ptr,
                                 const cutespmm_options_t *opts, std::string &err)
{
    if (M >= (1ull << 32) - kPanelRows || K >= (1ull << 32)) { err = "M and K must be below 2^32"; return CUTESPMM_EUNSUPPORTED; }
    if (row_ptr.size() != M + 1) { err = "rowPtr must have M+1 entries"; return CUTESPMM_EINVAL; }
    if (row_ptr[0] != 0) { err = "rowPtr[0] must be 0"; return CUTESPMM_EINVAL; }
    if (opts && opts->path == CUTESPMM_PATH_SLAB) {
        err = "the slab path is built by the host builder only (cutespmm_plan_create)";
        return CUTESPMM_EUNSUPPORTED;
    }
    if (opts && opts->path > CUTESPMM_PATH_SLAB) { err = "unknown path"; return CUTESPMM_EINVAL; }
    p.adaptive_tiling = fill_default_options(p.opts, opts);
    if (p.opts.reorder) { err = "row reordering is done by the host builder only (cutespmm_plan_create)"; return CUTESPMM_EUNSUPPORTED; }
    int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : bad)
    for (int64_t r = 0; r < (int64_t)M; ++r) bad |= row_ptr[r + 1] < row_ptr[r];
    if (bad) { err = "rowPtr is not non-decreasing"; return CUTESPMM_EINVAL; }
    p.M = M; p.K = K; p.nnz = row_ptr[M];
    p.row_ptr = std::move(row_ptr);
    p.device_built = true;
    p.row_path.assign(p.num_panels(), 0);
    p.slab_path.assign((M + kSlabRows - 1) / kSlabRows, 0);
    return CUTESPMM_OK;
}

void finish_device_plan(HostPlan &p, const std::vector<uint32_t> *panel_ncols)
{
    if (panel_ncols) {
        choose_panel_paths(p, *panel_ncols);
        // the HRPB view blockedRowPtr follows from the counts -- unless a panel was left out of the analysis
        bool complete = true;
        p.blocked_row_ptr.assign(p.num_panels() + 1, 0);
        for (uint64_t q = 0; q < p.num_panels(); ++q) {
            complete &= (*panel_ncols)[q] != kPanelTooLarge;
            p.blocked_row_ptr[q + 1] = p.blocked_row_ptr[q] + (complete ? ((*panel_ncols)[q] + kBlockCols - 1) / kBlockCols : 0);
        }
        if (!complete) p.blocked_row_ptr.clear();
        std::vector<uint32_t> which;
        layout_brick_slots(p, *panel_ncols, which);
        p.brick_panel_ids = std::move(which);
    }
    build_tiles(p, false, p.tiles, p.chunks, p.long_rows);
    if (p.brick_panels) build_tiles(p, true, p.tiles_all, p.chunks_all, p.long_rows_all);
}

int build_host_plan(HostPlan &p, uint64_t M, uint64_t K, const uint64_t *rowPtr, const uint32_t *cols,
                    const float *vals, const cutespmm_options_t *opts, std::string &err)
{
    if (!rowPtr) { err = "rowPtr is NULL"; return CUTESPMM_EINVAL; }
    if (M >= (1ull << 32) - kPanelRows || K >= (1ull << 32)) { err = "M and K must be below 2^32"; return CUTESPMM_EUNSUPPORTED; }
    if (rowPtr[0] != 0) { err = "rowPtr[0] must be 0"; return CUTESPMM_EINVAL; }
    const uint64_t nnz = rowPtr[M];
    if (nnz >= (1ull << 32)) { err = "more than 2^32-1 nonzeros in one plan: shard the rows"; return CUTESPMM_EUNSUPPORTED; }
    if (nnz && (!cols || !vals)) { err = "cols/vals is NULL"; return CUTESPMM_EINVAL; }
    if (opts && opts->path > CUTESPMM_PATH_SLAB) { err = "unknown path"; return CUTESPMM_EINVAL; }
    p.adaptive_tiling = fill_default_options(p.opts, opts);
    if (p.opts.reorder > CUTESPMM_REORDER_SIMILAR_ROWS) { err = "unknown reorder option"; return CUTESPMM_EINVAL; }
    if (p.opts.path == CUTESPMM_PATH_SLAB && p.opts.reorder) {
        err = "row reordering is available on the row and brick kernels (path auto, rows or brick)";
        return CUTESPMM_EUNSUPPORTED;
    }
    if (p.opts.path == CUTESPMM_PATH_SLAB && (p.opts.flags & CUTESPMM_FLAG_ROUND_B_NEAREST)) {
        err = "the slab path cannot round B to nearest: the copy engine places B in the tensor core's operand layout and no thread touches it";
        return CUTESPMM_EUNSUPPORTED;
    }
    p.M = M; p.K = K; p.nnz = nnz;

    // validation + 32-bit row pointers
    int bad = 0;
    p.row_ptr.resize(M + 1);
#pragma omp parallel for schedule(static) reduction(| : bad)
    for (int64_t r = 0; r <= (int64_t)M; ++r) {
        if (r < (int64_t)M && rowPtr[r + 1] < rowPtr[r]) bad |= 1;
        if (rowPtr[r] > nnz) bad |= 1;
        p.row_ptr[r] = (uint32_t)rowPtr[r];
    }
    if (bad & 1) { err = "rowPtr is not non-decreasing"; return CUTESPMM_EINVAL; }

    // pairs, sorted by column inside each row (stable: equal columns keep input order)
    p.pairs.resize(nnz);
#pragma omp parallel for schedule(dynamic, 1024) reduction(| : bad)
    for (int64_t r = 0; r < (int64_t)M; ++r) {
        const uint64_t j0 = rowPtr[r], j1 = rowPtr[r + 1];
        bool sorted = true;
        for (uint64_t j = j0; j < j1; ++j) {
            uint32_t vb;
            std::memcpy(&vb, &vals[j], 4);
            p.pairs[j] = Pair{cols[j], vb};
            if (cols[j] >= K) bad |= 2;
            if (j > j0 && cols[j] < cols[j - 1]) sorted = false;
        }
        if (!sorted)
            std::stable_sort(p.pairs.begin() + j0, p.pairs.begin() + j1,
                             [](const Pair &a, const Pair &b) { return a.col < b.col; });
    }
    if (bad & 2) { err = "column index out of range (>= K)"; return CUTESPMM_EINVAL; }

    if (p.opts.reorder == CUTESPMM_REORDER_CLUSTER_ROWS) cluster_rows(p);
    if (p.opts.reorder == CUTESPMM_REORDER_SIMILAR_ROWS) group_similar_rows(p);

    const std::vector<uint32_t> panel_ncols = analyze_panels(p);

    choose_panel_paths(p, panel_ncols);
    // 128-row panels for the slab (tcgen05) kernel; their 16-row panels are marked 2
    const uint64_t SP = (p.M + kSlabRows - 1) / kSlabRows;
    p.slab_path.assign(SP, 0);
    if (p.opts.path == CUTESPMM_PATH_SLAB) {
        for (uint64_t q = 0; q < SP; ++q) {
            const uint64_t r0 = q * kSlabRows, r1 = std::min<uint64_t>(p.M, r0 + kSlabRows);
            if (p.row_ptr[r1] == p.row_ptr[r0]) continue;
            p.slab_path[q] = 1;
            for (uint64_t pq = r0 / kPanelRows; pq < (r1 + kPanelRows - 1) / kPanelRows; ++pq) p.row_path[pq] = 2;
        }
    }
    build_tiles(p, false, p.tiles, p.chunks, p.long_rows);
    build_brick_part(p, panel_ncols);
    build_slab_part(p);
    if (p.brick_panels || p.slab_panels) build_tiles(p, true, p.tiles_all, p.chunks_all, p.long_rows_all);
    return CUTESPMM_OK;
}

void decode_host_plan(const HostPlan &p, uint64_t *rowPtr, uint32_t *cols, float *vals)
{
    // The pairs array holds every nonzero (both kernels' rows); the brick arrays are a second
    // encoding of the brick panels.  Decode each part from the encoding its kernel reads.
    const uint64_t P = p.num_panels();
    std::vector<std::vector<std::pair<uint32_t, float>>> rows(p.M);
    for (uint64_t q = 0; q < P; ++q) {
        if (p.row_path[q]) continue;
        const uint64_t r0 = q * kPanelRows, r1 = std::min<uint64_t>(p.M, r0 + kPanelRows);
        for (uint64_t r = r0; r < r1; ++r)
            for (uint32_t j = p.row_ptr[r]; j < p.row_ptr[r + 1]; ++j) {
                float v;
                std::memcpy(&v, &p.pairs[j].val_bits, 4);
                rows[r].push_back({p.pairs[j].col, v});
            }
    }
    for (uint64_t i = 0; i < p.panel_first_brick.size(); ++i)
    for (uint64_t k = p.panel_first_brick[i]; k < p.panel_last_brick[i]; ++k) {  // the panel's bricks (not its empty slots)
        const uint32_t *rec = &p.brick_recs[(size_t)p.brick_rec_off[k] * 4];
        const uint32_t panel = rec[5];
        for (uint32_t bit = 0; bit < 128; ++bit) {
            if (!((rec[bit >> 5] >> (bit & 31)) & 1u)) continue;
            float v;
            std::memcpy(&v, &rec[kBrickRecHeaderWords + brick_frag_index(bit / kBrickCols, bit % kBrickCols)], 4);
            rows[(size_t)panel * kPanelRows + bit / kBrickCols].push_back({p.brick_cols[k * kBrickCols + bit % kBrickCols], v});
        }
    }
    for (uint64_t t = 0; t + 1 < p.slab_rec_off.size(); ++t) {
        if (p.slab_rec_off[t + 1] == p.slab_rec_off[t]) continue;  // empty slot
        const uint32_t *rec = &p.slab_recs[(size_t)p.slab_rec_off[t] * 4];
        const uint32_t cnt = rec[0] & 0xffffu, panel = rec[1];
        const uint32_t *entries = rec + kSlabRecHeaderWords;
        const uint32_t *vals = entries + (cnt + 3) / 4 * 4;
        for (uint32_t e = 0; e < cnt; ++e) {
            const uint32_t row = entries[e] & 0xffu, mask = (entries[e] >> 8) & 0xffu;
            uint32_t k = entries[e] >> 16;
            for (uint32_t c = 0; c < 8; ++c) {
                if (!((mask >> c) & 1u)) continue;
                float v;
                std::memcpy(&v, &vals[k++], 4);
                rows[(size_t)panel * kSlabRows + row].push_back({p.slab_cols[t * 8 + c], v});
            }
        }
    }
    if (!p.row_map.empty()) {  // back to the caller's row order
        std::vector<std::vector<std::pair<uint32_t, float>>> orig(p.M);
        for (uint64_t r = 0; r < p.M; ++r) orig[p.row_map[r]] = std::move(rows[r]);
        rows = std::move(orig);
    }
    uint64_t off = 0;
    for (uint64_t r = 0; r < p.M; ++r) {
        rowPtr[r] = off;
        std::stable_sort(rows[r].begin(), rows[r].end(),
                         [](const auto &a, const auto &b) { return a.first < b.first; });
        for (auto &e : rows[r]) {
            cols[off] = e.first;
            vals[off] = e.second;
            ++off;
        }
    }
    rowPtr[p.M] = off;
}

int partition_rows(uint64_t M, const uint64_t *rowPtr, uint32_t nparts, uint32_t align_rows, uint32_t row_cost,
                   uint64_t *bounds, std::string &err)
{
    if (!rowPtr || !bounds || nparts == 0) { err = "bad argument"; return CUTESPMM_EINVAL; }
    if (align_rows == 0) align_rows = 1;
    const uint64_t total = (rowPtr[M] - rowPtr[0]) + (uint64_t)row_cost * M;
    bounds[0] = 0;
    uint64_t r = 0;
    for (uint32_t k = 1; k < nparts; ++k) {
        // smallest aligned r with cost(rows [0, r)) >= k/nparts of the total
        const long double want = (long double)total * k / nparts;
        uint64_t lo = r, hi = M;
        while (lo < hi) {
            const uint64_t mid = lo + (hi - lo) / 2;
            const long double c = (long double)(rowPtr[mid] - rowPtr[0]) + (long double)row_cost * mid;
            if (c < want) lo = mid + 1; else hi = mid;
        }
        // round to the nearer multiple of align_rows, staying monotone and inside [0, M]
        uint64_t down = lo / align_rows * align_rows, up = std::min<uint64_t>(M, down + align_rows);
        auto cost_at = [&](uint64_t x) { return (long double)(rowPtr[x] - rowPtr[0]) + (long double)row_cost * x; };
        uint64_t pick = (want - cost_at(down) <= cost_at(up) - want) ? down : up;
        if (pick < r) pick = r;
        bounds[k] = r = pick;
    }
    bounds[nparts] = M;
    return CUTESPMM_OK;
}

}  // namespace cutespmm
