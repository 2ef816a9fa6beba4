// The extern "C" surface declared in include/cutespmm.h: plan life cycle, execution, sharding.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "device_plan.hpp"
#include "nvtx.hpp"
#include "plan.hpp"
#include "plan_object.hpp"

using namespace cutespmm;

namespace {
thread_local std::string g_last_error;
}
namespace cutespmm {
void set_last_error(const std::string &msg) { g_last_error = msg; }
int fail_status(int status, const std::string &msg)
{
    g_last_error = msg;
    return status;
}
int fail_cuda_status(cudaError_t e, const char *what)
{
    g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
    return e == cudaErrorMemoryAllocation ? CUTESPMM_ENOMEM : CUTESPMM_ECUDA;
}
}
namespace {

int fail(int status, const std::string &msg) { return fail_status(status, msg); }
int fail_cuda(cudaError_t e, const char *what) { return fail_cuda_status(e, what); }

template <class T> cudaError_t upload(const std::vector<T> &h, void **d, uint64_t &bytes)
{
    *d = nullptr;
    if (h.empty()) return cudaSuccess;
    cudaError_t e = cudaMalloc(d, h.size() * sizeof(T));
    if (e != cudaSuccess) return e;
    bytes += h.size() * sizeof(T);
    return cudaMemcpy(*d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
}
}  // namespace

extern "C" {

const char *cutespmm_status_string(int status)
{
    switch (status) {
        case CUTESPMM_OK: return "success";
        case CUTESPMM_EINVAL: return "invalid argument";
        case CUTESPMM_ENOMEM: return "out of memory";
        case CUTESPMM_ECUDA: return "CUDA error";
        case CUTESPMM_EUNSUPPORTED: return "unsupported";
        case CUTESPMM_EIO: return "I/O error";
        case CUTESPMM_ETIMEOUT: return "device-side wait timed out";
        case CUTESPMM_ECOMM: return "communication library error";
        default: return "unknown status";
    }
}
const char *cutespmm_last_error(void) { return g_last_error.c_str(); }
int cutespmm_version(void) { return 100; }

static int build_common(cutespmm_plan_t **out, uint64_t M, uint64_t K, const uint64_t *rowPtr, const uint32_t *cols,
                        const float *vals, const cutespmm_options_t *opts)
{
    if (!out) return fail(CUTESPMM_EINVAL, "plan is NULL");
    *out = nullptr;
    cutespmm_plan *p = new (std::nothrow) cutespmm_plan();
    if (!p) return fail(CUTESPMM_ENOMEM, "host allocation failed");
    std::string err;
    int st;
    try {
        st = build_host_plan(p->host, M, K, rowPtr, cols, vals, opts, err);
    } catch (const std::bad_alloc &) {
        st = CUTESPMM_ENOMEM;
        err = "host allocation failed while building the plan";
    }
    if (st != CUTESPMM_OK) {
        delete p;
        return fail(st, err);
    }
    *out = p;
    return CUTESPMM_OK;
}

int cutespmm_plan_build_host(cutespmm_plan_t **plan, uint64_t M, uint64_t K, const uint64_t *rowPtr,
                             const uint32_t *cols, const float *vals, const cutespmm_options_t *opts)
{
    return build_common(plan, M, K, rowPtr, cols, vals, opts);
}

// The current device, checked to be one this library runs on.
static int usable_device(int *dev, int *sm_count)
{
    cudaError_t e = cudaGetDevice(dev);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice (libcutespmm needs a CUDA device; there is no CPU path)");
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, *dev);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetDeviceProperties");
    if (prop.major < 10)
        return fail(CUTESPMM_EUNSUPPORTED, "this library is built for sm_100a (B200) only; found compute capability " +
                                               std::to_string(prop.major) + "." + std::to_string(prop.minor));
    *sm_count = prop.multiProcessorCount;
    return CUTESPMM_OK;
}

// What the row kernel needs to finish long rows inside the launch: per scratch slot the long row it belongs to (for
// both work lists), one arrival counter per long row and column slab (zero between launches), and the scratch matrix.
static cudaError_t reserve_long_row_state(cutespmm_plan *p, uint64_t &by, const char **what)
{
    const HostPlan &h = p->host;
    auto owners = [](const std::vector<Chunk> &chunks, const std::vector<LongRow> &rows) {
        std::vector<uint32_t> v(chunks.size(), 0u);
        for (size_t i = 0; i < rows.size(); ++i)
            for (uint32_t k = rows[i].slot0; k < rows[i].slot1; ++k) v[k] = (uint32_t)i;
        return v;
    };
    cudaError_t e;
    *what = "chunk owners";
    if ((e = upload(owners(h.chunks, h.long_rows), &p->d_chunk_owner, by)) != cudaSuccess) return e;
    if ((e = upload(owners(h.chunks_all, h.long_rows_all), &p->d_chunk_owner_all, by)) != cudaSuccess) return e;
    const uint64_t counters = (uint64_t)std::max(h.long_rows.size(), h.long_rows_all.size()) * (kScratchCols / 32) * sizeof(uint32_t);
    if (counters) {
        *what = "arrival counters";
        if ((e = cudaMalloc(&p->d_arrivals, counters)) != cudaSuccess || (e = cudaMemset(p->d_arrivals, 0, counters)) != cudaSuccess) return e;
        by += counters;
    }
    const uint64_t scratch = (uint64_t)std::max(h.chunks.size(), h.chunks_all.size()) * kScratchCols * sizeof(float);
    if (scratch) {
        *what = "scratch";
        if ((e = cudaMalloc(&p->d_scratch, scratch)) != cudaSuccess) return e;
        by += scratch;
    }
    return cudaSuccess;
}

// Uploads every array of a complete host-side plan to the current device and reserves scratch and status word.
static int upload_plan(cutespmm_plan *p, int dev, int sm_count)
{
    HostPlan &h = p->host;
    p->device = dev;
    p->sm_count = sm_count;
    p->on_device = true;
    uint64_t &by = p->device_bytes;
    cudaError_t e;
#define UP(vec, ptr) \
    if ((e = upload(vec, &ptr, by)) != cudaSuccess) return fail_cuda(e, "uploading " #vec);
    {   // bulk copies of a tile start/end on 16-byte boundaries: keep readable slack behind both arrays
        std::vector<uint32_t> rp(h.row_ptr);
        rp.resize(rp.size() + 8, rp.back());
        std::vector<Pair> pr(h.pairs);
        pr.resize(pr.size() + 2, Pair{0, 0});
        UP(rp, p->d_row_ptr)
        UP(pr, p->d_pairs)
    }
    UP(h.row_map, p->d_row_map)
    UP(h.tiles, p->d_tiles)
    UP(h.chunks, p->d_chunks)
    UP(h.long_rows, p->d_long_rows)
    UP(h.tiles_all, p->d_tiles_all)
    UP(h.chunks_all, p->d_chunks_all)
    UP(h.long_rows_all, p->d_long_rows_all)
    if (h.num_bricks) {
        // the producer lanes prefetch a group (4 brick slots) beyond the one in use: keep that readable
        std::vector<uint32_t> bc(h.brick_cols);
        bc.resize(bc.size() + 96, 0u);
        UP(bc, p->d_bcols)
        UP(h.brick_recs, p->d_brecs)
        UP(h.panel_first_brick, p->d_panel_first)
        UP(h.panel_last_brick, p->d_panel_last)
    }
    if (h.slab_steps) {
        std::vector<uint32_t> sc(h.slab_cols), so(h.slab_rec_off);
        sc.resize(sc.size() + 96, 0u);
        so.resize(so.size() + 16, so.back());
        UP(sc, p->d_scols)
        UP(h.slab_recs, p->d_srecs)
        UP(so, p->d_srec_off)
        UP(h.slab_first, p->d_sfirst)
        UP(h.slab_last, p->d_slast)
        UP(h.slab_ids, p->d_sids)
    }
#undef UP
    const char *what = "";
    if ((e = reserve_long_row_state(p, by, &what)) != cudaSuccess) return fail_cuda(e, what);
    if ((e = cudaMalloc(&p->d_status, 256)) != cudaSuccess || (e = cudaMemset(p->d_status, 0, 256)) != cudaSuccess)
        return fail_cuda(e, "status word");
    by += 256;
    return CUTESPMM_OK;
}

}  // extern "C"

// for plan_io.cu: a complete host-side plan goes to the current device
int cutespmm_internal_upload_plan(cutespmm_plan *p)
{
    int dev = -1, sms = 0;
    const int st = usable_device(&dev, &sms);
    return st != CUTESPMM_OK ? st : upload_plan(p, dev, sms);
}

extern "C" {

int cutespmm_plan_create(cutespmm_plan_t **plan, uint64_t M, uint64_t K, const uint64_t *rowPtr, const uint32_t *cols,
                         const float *vals, const cutespmm_options_t *opts)
{
    // fail before the (possibly long) host build when there is no usable device
    int dev = -1, sms = 0;
    int st = usable_device(&dev, &sms);
    if (st != CUTESPMM_OK) return st;
    NvtxRange range("cutespmm: plan creation");
    if ((st = build_common(plan, M, K, rowPtr, cols, vals, opts)) != CUTESPMM_OK) return st;
    if ((st = upload_plan(*plan, dev, sms)) != CUTESPMM_OK) {
        delete *plan;
        *plan = nullptr;
    }
    return st;
}

int cutespmm_plan_create_device(cutespmm_plan_t **plan, uint64_t M, uint64_t K, const uint32_t *rowPtr_dev, const uint32_t *cols_dev,
                                const float *vals_dev, const cutespmm_options_t *opts, void *stream)
{
    if (!plan) return fail(CUTESPMM_EINVAL, "plan is NULL");
    *plan = nullptr;
    if (!rowPtr_dev) return fail(CUTESPMM_EINVAL, "rowPtr is NULL");
    if (M >= (1ull << 32) - kPanelRows || K >= (1ull << 32)) return fail(CUTESPMM_EUNSUPPORTED, "M and K must be below 2^32");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    NvtxRange range("cutespmm: plan creation (device CSR)");
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice (libcutespmm needs a CUDA device; there is no CPU path)");
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, dev)) != cudaSuccess) return fail_cuda(e, "cudaGetDeviceProperties");
    if (prop.major < 10)
        return fail(CUTESPMM_EUNSUPPORTED, "this library is built for sm_100a (B200) only; found compute capability " +
                                               std::to_string(prop.major) + "." + std::to_string(prop.minor));
    // the row pointers come to the host (4 bytes per row): tiles, chunks and the list of long rows are cut from them alone
    std::vector<uint32_t> rp;
    try {
        rp.resize(M + 1);
    } catch (const std::bad_alloc &) {
        return fail(CUTESPMM_ENOMEM, "host allocation failed");
    }
    if ((e = cudaMemcpyAsync(rp.data(), rowPtr_dev, (M + 1) * sizeof(uint32_t), cudaMemcpyDeviceToHost, s)) != cudaSuccess ||
        (e = cudaStreamSynchronize(s)) != cudaSuccess)
        return fail_cuda(e, "reading the row pointers");
    cutespmm_plan *p = new (std::nothrow) cutespmm_plan();
    if (!p) return fail(CUTESPMM_ENOMEM, "host allocation failed");
    std::string err;
    int st;
    try {
        st = build_rows_plan_from_row_ptr(p->host, M, K, std::move(rp), opts, err);
    } catch (const std::bad_alloc &) {
        st = CUTESPMM_ENOMEM;
        err = "host allocation failed while building the plan";
    }
    if (st != CUTESPMM_OK) { delete p; return fail(st, err); }
    HostPlan &h = p->host;
    if (h.nnz && (!cols_dev || !vals_dev)) { delete p; return fail(CUTESPMM_EINVAL, "cols/vals is NULL"); }
    p->device = dev;
    p->sm_count = prop.multiProcessorCount;
    p->on_device = true;
    uint64_t &by = p->device_bytes;
    auto bail = [&](cudaError_t ce, const char *what) { delete p; return fail_cuda(ce, what); };
    // row pointers: device-to-device, with the slack the tile copies may read behind the end
    if ((e = cudaMalloc(&p->d_row_ptr, (M + 1 + 8) * sizeof(uint32_t))) != cudaSuccess) return bail(e, "row pointers");
    by += (M + 1 + 8) * sizeof(uint32_t);
    const uint32_t tail[8] = {h.row_ptr[M], h.row_ptr[M], h.row_ptr[M], h.row_ptr[M], h.row_ptr[M], h.row_ptr[M], h.row_ptr[M], h.row_ptr[M]};
    if ((e = cudaMemcpyAsync(p->d_row_ptr, rowPtr_dev, (M + 1) * sizeof(uint32_t), cudaMemcpyDeviceToDevice, s)) != cudaSuccess ||
        (e = cudaMemcpyAsync(static_cast<uint32_t *>(p->d_row_ptr) + M + 1, tail, sizeof(tail), cudaMemcpyHostToDevice, s)) != cudaSuccess)
        return bail(e, "row pointers");
    if ((e = cudaMalloc(&p->d_status, 256)) != cudaSuccess || (e = cudaMemsetAsync(p->d_status, 0, 256, s)) != cudaSuccess)
        return bail(e, "status word");
    by += 256;
    // nonzeros: packed on the device; the second status word collects the column-range check
    if ((e = cudaMalloc(&p->d_pairs, (h.nnz + 2) * sizeof(Pair))) != cudaSuccess) return bail(e, "packed nonzeros");
    by += (h.nnz + 2) * sizeof(Pair);
    e = launch_pack_pairs(cols_dev, vals_dev, p->d_pairs, h.nnz, (uint32_t)K, p->d_status + 1, p->sm_count, s);
    if (e != cudaSuccess) return bail(e, "packing the nonzeros");
    {   // largest column of every panel (4 bytes per panel to the host): what the row-block host-buffer call schedules by
        const uint64_t P = h.num_panels();
        uint32_t *d_max = nullptr;
        try {
            h.panel_max_col.assign(P, 0u);
        } catch (const std::bad_alloc &) {
            delete p;
            return fail(CUTESPMM_ENOMEM, "host allocation failed");
        }
        if (P && h.nnz) {
            if ((e = cudaMalloc(&d_max, P * sizeof(uint32_t))) != cudaSuccess ||
                (e = launch_panel_max_col(static_cast<const uint32_t *>(p->d_row_ptr), p->d_pairs, (uint32_t)M, (uint32_t)P, d_max, p->sm_count, s)) != cudaSuccess ||
                (e = cudaMemcpyAsync(h.panel_max_col.data(), d_max, P * sizeof(uint32_t), cudaMemcpyDeviceToHost, s)) != cudaSuccess ||
                (e = cudaStreamSynchronize(s)) != cudaSuccess) {
                if (d_max) cudaFree(d_max);
                return bail(e, "panel column ranges");
            }
            cudaFree(d_max);
        }
    }
    // panel analysis and brick packing on the device (paths auto and brick); the per-panel column counts visit the host,
    // where each panel's kernel is chosen and the brick slots and work lists are laid out
    uint32_t *d_ncols = nullptr, *d_acols = nullptr, *d_which = nullptr;
    auto drop_temps = [&]() {
        for (uint32_t *t : {d_ncols, d_acols, d_which})
            if (t) cudaFree(t);
        d_ncols = d_acols = d_which = nullptr;
    };
    try {
        if (h.opts.path != CUTESPMM_PATH_ROWS && h.nnz) {
            const uint64_t P = h.num_panels();
            std::vector<uint32_t> ncols(P);
            if ((e = cudaMalloc(&d_ncols, P * sizeof(uint32_t))) != cudaSuccess || (e = cudaMalloc(&d_acols, h.nnz * sizeof(uint32_t))) != cudaSuccess ||
                (e = launch_panel_columns(static_cast<const uint32_t *>(p->d_row_ptr), p->d_pairs, (uint32_t)M, (uint32_t)P, d_ncols, d_acols,
                                          p->sm_count, s)) != cudaSuccess ||
                (e = cudaMemcpyAsync(ncols.data(), d_ncols, P * sizeof(uint32_t), cudaMemcpyDeviceToHost, s)) != cudaSuccess ||
                (e = cudaStreamSynchronize(s)) != cudaSuccess) {
                drop_temps();
                return bail(e, "panel analysis");
            }
            if (h.opts.path == CUTESPMM_PATH_BRICK && std::find(ncols.begin(), ncols.end(), kPanelTooLarge) != ncols.end()) {
                drop_temps();
                delete p;
                return fail(CUTESPMM_EUNSUPPORTED, "path brick on the device: a 16-row panel holds more than " + std::to_string(kDevPanelMax) +
                                                       " nonzeros; use path auto (such panels run on the row kernel) or the host builder");
            }
            finish_device_plan(h, &ncols);
            if (h.brick_panels) {
                const uint64_t col_words = h.brick_slots * kBrickCols + 96, rec_words = h.brick_slots * kBrickRecWords;
                if ((e = cudaMalloc(&p->d_bcols, col_words * 4)) != cudaSuccess || (e = cudaMalloc(&p->d_brecs, rec_words * 4)) != cudaSuccess ||
                    (e = cudaMemsetAsync(p->d_bcols, 0, col_words * 4, s)) != cudaSuccess || (e = cudaMemsetAsync(p->d_brecs, 0, rec_words * 4, s)) != cudaSuccess ||
                    (e = cudaMalloc(&d_which, h.brick_panels * sizeof(uint32_t))) != cudaSuccess ||
                    (e = cudaMemcpyAsync(d_which, h.brick_panel_ids.data(), h.brick_panels * sizeof(uint32_t), cudaMemcpyHostToDevice, s)) != cudaSuccess ||
                    (e = upload(h.panel_first_brick, &p->d_panel_first, by)) != cudaSuccess || (e = upload(h.panel_last_brick, &p->d_panel_last, by)) != cudaSuccess ||
                    (e = launch_brick_fill(static_cast<const uint32_t *>(p->d_row_ptr), p->d_pairs, (uint32_t)M, d_which,
                                           static_cast<const uint32_t *>(p->d_panel_first), static_cast<const uint32_t *>(p->d_panel_last),
                                           (uint32_t)h.brick_panels, d_ncols, d_acols, static_cast<uint32_t *>(p->d_bcols),
                                           static_cast<uint32_t *>(p->d_brecs), p->sm_count, s)) != cudaSuccess ||
                    (e = cudaStreamSynchronize(s)) != cudaSuccess) {
                    drop_temps();
                    return bail(e, "brick packing");
                }
                by += (col_words + rec_words) * 4;
            }
            drop_temps();
        } else {
            finish_device_plan(h, nullptr);
        }
    } catch (const std::bad_alloc &) {
        drop_temps();
        delete p;
        return fail(CUTESPMM_ENOMEM, "host allocation failed while building the plan");
    }
    if ((e = upload(h.tiles, &p->d_tiles, by)) != cudaSuccess || (e = upload(h.chunks, &p->d_chunks, by)) != cudaSuccess ||
        (e = upload(h.long_rows, &p->d_long_rows, by)) != cudaSuccess || (e = upload(h.tiles_all, &p->d_tiles_all, by)) != cudaSuccess ||
        (e = upload(h.chunks_all, &p->d_chunks_all, by)) != cudaSuccess || (e = upload(h.long_rows_all, &p->d_long_rows_all, by)) != cudaSuccess)
        return bail(e, "uploading the work lists");
    const char *what = "";
    if ((e = reserve_long_row_state(p, by, &what)) != cudaSuccess) return bail(e, what);
    uint32_t bad = 0;
    if ((e = cudaMemcpyAsync(&bad, p->d_status + 1, sizeof(bad), cudaMemcpyDeviceToHost, s)) != cudaSuccess ||
        (e = cudaStreamSynchronize(s)) != cudaSuccess)
        return bail(e, "packing the nonzeros");
    if (bad) { delete p; return fail(CUTESPMM_EINVAL, "column index out of range (>= K)"); }
    *plan = p;
    return CUTESPMM_OK;
}

int cutespmm_plan_create_u32(cutespmm_plan_t **plan, uint32_t M, uint32_t K, const uint32_t *rowPtr,
                             const uint32_t *cols, const float *vals, const cutespmm_options_t *opts)
{
    if (!rowPtr) return fail(CUTESPMM_EINVAL, "rowPtr is NULL");
    std::vector<uint64_t> rp((size_t)M + 1);
    for (size_t i = 0; i <= M; ++i) rp[i] = rowPtr[i];
    return cutespmm_plan_create(plan, M, K, rp.data(), cols, vals, opts);
}

int cutespmm_plan_destroy(cutespmm_plan_t *plan)
{
    delete plan;
    return CUTESPMM_OK;
}

int cutespmm_plan_info(const cutespmm_plan_t *p, cutespmm_plan_info_t *info)
{
    if (!p || !info) return fail(CUTESPMM_EINVAL, "null argument");
    const HostPlan &h = p->host;
    std::memset(info, 0, sizeof(*info));
    info->M = h.M; info->K = h.K; info->nnz = h.nnz;
    info->num_panels = h.num_panels();
    info->num_blocks = h.blocked_row_ptr.empty() ? 0 : h.blocked_row_ptr.back();
    info->num_tiles = h.tiles.size();
    info->num_long_rows = h.long_rows.size();
    info->num_chunks = h.chunks.size();
    info->brick_panels = h.brick_panels;
    info->num_bricks = h.num_bricks;
    info->device_bytes = p->device_bytes;
    info->scratch_bytes_per_col = std::max(h.chunks.size(), h.chunks_all.size()) * sizeof(float);
    return CUTESPMM_OK;
}

static const char *kNoViews =
    "this plan was built on the device without the panel analysis (path rows, or a panel beyond the device sort): "
    "the panel views come with path auto / brick, or from the host builder";

static bool device_plan_has_views(const cutespmm_plan *p)
{
    return !p->host.device_built || p->host.blocked_row_ptr.size() == p->host.num_panels() + 1;
}

int cutespmm_plan_blocked_row_ptr(const cutespmm_plan_t *p, uint32_t *out)
{
    if (!p || !out) return fail(CUTESPMM_EINVAL, "null argument");
    if (!device_plan_has_views(p)) return fail(CUTESPMM_EUNSUPPORTED, kNoViews);
    std::memcpy(out, p->host.blocked_row_ptr.data(), p->host.blocked_row_ptr.size() * sizeof(uint32_t));
    return CUTESPMM_OK;
}
int cutespmm_plan_active_cols(const cutespmm_plan_t *p, uint32_t *out)
{
    if (!p || !out) return fail(CUTESPMM_EINVAL, "null argument");
    if (!device_plan_has_views(p)) return fail(CUTESPMM_EUNSUPPORTED, kNoViews);
    const HostPlan &h = p->host;
    if (!h.device_built) {
        std::memcpy(out, h.active_cols.data(), h.active_cols.size() * sizeof(uint32_t));
        return CUTESPMM_OK;
    }
    // a device-built plan does not keep the column lists: run the panel analysis again and bring them back
    const uint64_t P = h.num_panels();
    if (h.nnz == 0 || P == 0) return CUTESPMM_OK;
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != p->device) cudaSetDevice(p->device);
    uint32_t *d_ncols = nullptr, *d_acols = nullptr;
    std::vector<uint32_t> ncols(P), acols(h.nnz);
    cudaError_t e;
    if ((e = cudaMalloc(&d_ncols, P * sizeof(uint32_t))) == cudaSuccess && (e = cudaMalloc(&d_acols, h.nnz * sizeof(uint32_t))) == cudaSuccess &&
        (e = launch_panel_columns(static_cast<const uint32_t *>(p->d_row_ptr), p->d_pairs, (uint32_t)h.M, (uint32_t)P, d_ncols, d_acols, p->sm_count, nullptr)) == cudaSuccess &&
        (e = cudaMemcpy(ncols.data(), d_ncols, P * sizeof(uint32_t), cudaMemcpyDeviceToHost)) == cudaSuccess)
        e = cudaMemcpy(acols.data(), d_acols, h.nnz * sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (d_ncols) cudaFree(d_ncols);
    if (d_acols) cudaFree(d_acols);
    if (cur != p->device && cur >= 0) cudaSetDevice(cur);
    if (e != cudaSuccess) return fail_cuda(e, "panel analysis");
    for (uint64_t q = 0; q < P; ++q) {  // per panel: its columns, zero-padded to a multiple of 16 (data.cu:160,204-209)
        uint32_t *dst = out + (uint64_t)h.blocked_row_ptr[q] * kBlockCols;
        const uint32_t width = (h.blocked_row_ptr[q + 1] - h.blocked_row_ptr[q]) * kBlockCols;
        const uint32_t *src = acols.data() + h.row_ptr[q * kPanelRows];
        for (uint32_t c = 0; c < width; ++c) dst[c] = c < ncols[q] ? src[c] : 0u;
    }
    return CUTESPMM_OK;
}
int cutespmm_plan_decode_csr(const cutespmm_plan_t *p, uint64_t *rowPtr, uint32_t *cols, float *vals)
{
    if (!p || !rowPtr || (p->host.nnz && (!cols || !vals))) return fail(CUTESPMM_EINVAL, "null argument");
    if ((p->host.device_built || p->host.values_on_device) && p->on_device) {  // the current pairs live on the device, in CSR order
        const HostPlan &h = p->host;
        for (uint64_t r = 0; r <= h.M; ++r) rowPtr[r] = h.row_ptr[r];
        std::vector<Pair> pr(h.nnz);
        if (h.nnz) {
            cudaError_t e = cudaMemcpy(pr.data(), p->d_pairs, h.nnz * sizeof(Pair), cudaMemcpyDeviceToHost);
            if (e != cudaSuccess) return fail_cuda(e, "reading the packed nonzeros back");
        }
        for (uint64_t j = 0; j < h.nnz; ++j) {
            cols[j] = pr[j].col;
            std::memcpy(&vals[j], &pr[j].val_bits, 4);
        }
        return CUTESPMM_OK;
    }
    decode_host_plan(p->host, rowPtr, cols, vals);
    return CUTESPMM_OK;
}

static RowsArgs rows_args(const cutespmm_plan *p, bool all_rows, const float *B, uint64_t ldb, float *C, uint64_t ldc,
                          uint32_t N, const cutespmm_item_range *rg = nullptr)
{
    const HostPlan &h = p->host;
    RowsArgs a{};
    a.row_ptr = static_cast<const uint32_t *>(p->d_row_ptr);
    a.pairs = p->d_pairs;
    a.tiles = all_rows ? p->d_tiles_all : p->d_tiles;
    a.chunks = all_rows ? p->d_chunks_all : p->d_chunks;
    a.long_rows = all_rows ? p->d_long_rows_all : p->d_long_rows;
    a.num_tiles = (uint32_t)(all_rows ? h.tiles_all.size() : h.tiles.size());
    a.num_chunks = (uint32_t)(all_rows ? h.chunks_all.size() : h.chunks.size());
    a.chunk_owner = static_cast<const uint32_t *>(all_rows ? p->d_chunk_owner_all : p->d_chunk_owner);
    a.arrivals = p->d_arrivals;
    a.split_nnz = h.opts.split_nnz;
    a.avg_row_nnz = (uint32_t)(h.nnz / std::max<uint64_t>(h.M, 1));
    a.B = B; a.C = C; a.scratch = p->d_scratch;
    a.ldb = ldb; a.ldc = ldc; a.ld_scratch = kScratchCols;
    a.N = N;
    a.status = p->d_status;
    a.row_map = static_cast<const uint32_t *>(p->d_row_map);
    if (rg) {  // a sub-range of the lists: 16-byte tiles and chunks (a chunk names its scratch slot and, through it, its long row)
        const uint32_t t0 = all_rows ? rg->ta0 : rg->t0, t1 = all_rows ? rg->ta1 : rg->t1;
        const uint32_t c0 = all_rows ? rg->ca0 : rg->c0, c1 = all_rows ? rg->ca1 : rg->c1;
        a.tiles = static_cast<const char *>(a.tiles) + (size_t)t0 * sizeof(Tile);
        a.chunks = static_cast<const char *>(a.chunks) + (size_t)c0 * sizeof(Chunk);
        a.num_tiles = t1 - t0;
        a.num_chunks = c1 - c0;
    }
    return a;
}
static BrickArgs brick_args(const cutespmm_plan *p, const float *B, uint64_t ldb, float *C, uint64_t ldc, uint32_t N,
                            const cutespmm_item_range *rg = nullptr)
{
    BrickArgs a{};
    a.cols = static_cast<const uint32_t *>(p->d_bcols);
    a.recs = static_cast<const uint32_t *>(p->d_brecs);
    a.panel_first = static_cast<const uint32_t *>(p->d_panel_first);
    a.panel_last = static_cast<const uint32_t *>(p->d_panel_last);
    a.num_bricks = (uint32_t)p->host.num_bricks;
    a.num_panels = (uint32_t)p->host.brick_panels;
    a.M = (uint32_t)p->host.M;
    a.K = (uint32_t)p->host.K;
    a.B = B; a.C = C;
    a.ldb = ldb; a.ldc = ldc;
    a.N = N;
    a.round_b = (p->host.opts.flags & CUTESPMM_FLAG_ROUND_B_NEAREST) ? 1u : 0u;
    a.status = p->d_status;
    a.row_map = static_cast<const uint32_t *>(p->d_row_map);
    if (rg) {  // the kernel numbers its panels from panel_first[0]: hand it the sub-list
        a.panel_first += rg->p0;
        a.panel_last += rg->p0;
        a.num_panels = rg->p1 - rg->p0;
        if (a.num_panels == 0) a.num_bricks = 0;
    }
    return a;
}

static SlabArgs slab_args(const cutespmm_plan *p, const float *B, uint64_t ldb, float *C, uint64_t ldc, uint32_t N)
{
    SlabArgs a{};
    a.cols = static_cast<const uint32_t *>(p->d_scols);
    a.recs = static_cast<const uint32_t *>(p->d_srecs);
    a.rec_off = static_cast<const uint32_t *>(p->d_srec_off);
    a.panel_first = static_cast<const uint32_t *>(p->d_sfirst);
    a.panel_last = static_cast<const uint32_t *>(p->d_slast);
    a.panel_ids = static_cast<const uint32_t *>(p->d_sids);
    a.num_panels = (uint32_t)p->host.slab_panels;
    a.M = (uint32_t)p->host.M;
    a.K = (uint32_t)p->host.K;
    a.B = B; a.C = C;
    a.ldb = ldb; a.ldc = ldc;
    a.N = N;
    a.status = p->d_status;
    return a;
}

// Whether a window of N columns at these addresses runs the brick kernel for the brick panels; if
// not, the row kernel executes every row from its all-rows work list.
// Path auto leaves products narrower than 64 columns to the row kernel even where the plan has brick panels: with a
// group of N/4 lanes per row it is the faster of the two there (stencil512 at N = 32: 0.035 against 0.041 ms,
// elasticity40: 0.045 against 0.047 ms; at N = 64 the brick kernel wins, 0.048 / 0.053 against 0.057 / 0.070 ms).
// A plan created with path brick runs its bricks at every width the brick kernel takes.
static bool brick_wanted(const HostPlan &h, uint32_t N)
{
    return h.num_bricks && (N >= 64 || h.opts.path == CUTESPMM_PATH_BRICK);
}
static bool use_brick(const cutespmm_plan *p, const float *B, uint64_t ldb, const float *C, uint64_t ldc, uint32_t N)
{
    return brick_wanted(p->host, N) && brick_supports(N, ldb, ldc, B, C);
}

// Kernels of one column window of width nw (bit 0 row kernel, bit 1 brick kernel, bit 2 slab kernel).  The alignment of
// the caller's pointers is unknown here: the aligned case is assumed.
static int window_kernels(const HostPlan &h, uint32_t nw)
{
    const bool brick = brick_wanted(h, nw) && nw % 32 == 0;
    const bool slab = h.slab_panels && nw % 128 == 0;
    const bool all_rows = (!brick && h.num_bricks) || (!slab && h.slab_panels);
    int mask = (brick ? 2 : 0) | (slab ? 4 : 0);
    if (all_rows ? (!h.tiles_all.empty() || !h.chunks_all.empty()) : (!h.tiles.empty() || !h.chunks.empty())) mask |= 1;
    return mask;
}

int cutespmm_spmm_kernels(const cutespmm_plan_t *p, uint32_t N)
{
    if (!p || N == 0 || p->host.M == 0) return 0;
    int mask = 0;
    for (uint32_t n0 = 0; n0 < N; n0 += kScratchCols) mask |= window_kernels(p->host, N - n0 < kScratchCols ? N - n0 : kScratchCols);
    return mask;
}

int cutespmm_spmm_launch_count(const cutespmm_plan_t *p, uint32_t N)
{
    if (!p || N == 0 || p->host.M == 0) return 0;
    int total = 0;
    for (uint32_t n0 = 0; n0 < N; n0 += kScratchCols) {
        const int mask = window_kernels(p->host, N - n0 < kScratchCols ? N - n0 : kScratchCols);
        total += (mask & 1) + ((mask >> 1) & 1) + ((mask >> 2) & 1);
    }
    return total;
}

int cutespmm_spmm(const cutespmm_plan_t *p, const float *B, uint64_t ldb, float *C, uint64_t ldc, uint32_t N,
                  void *stream)
{
    return cutespmm_internal_spmm_range(p, B, ldb, C, ldc, N, stream, nullptr);
}

}  // extern "C"

int cutespmm_internal_spmm_range(const cutespmm_plan *p, const float *B, uint64_t ldb, float *C, uint64_t ldc, uint32_t N, void *stream,
                                 const cutespmm_item_range *rg)
{
    if (!p) return fail(CUTESPMM_EINVAL, "plan is NULL");
    if (!p->on_device) return fail(CUTESPMM_EUNSUPPORTED, "host-only plan: build it with cutespmm_plan_create on a CUDA device to execute it");
    if (N == 0) return CUTESPMM_OK;
    if (!C && p->host.M) return fail(CUTESPMM_EINVAL, "C is NULL");
    if (!B && p->host.nnz) return fail(CUTESPMM_EINVAL, "B is NULL");
    if (ldb < N || ldc < N) return fail(CUTESPMM_EINVAL, "leading dimension smaller than N");
    if (ldb >= (1ull << 32) || ldc >= (1ull << 32)) return fail(CUTESPMM_EUNSUPPORTED, "leading dimensions must be below 2^32 elements");
    if ((reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 3) return fail(CUTESPMM_EINVAL, "B and C must be 4-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (p->host.M == 0) return CUTESPMM_OK;
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != p->device)
        return fail(CUTESPMM_EINVAL, "the current CUDA device (" + std::to_string(cur) + ") is not the one the plan was created on (" +
                                         std::to_string(p->device) + "): call cudaSetDevice first");
    for (uint32_t n0 = 0; n0 < N; n0 += kScratchCols) {
        const uint32_t nw = N - n0 < kScratchCols ? N - n0 : kScratchCols;
        cudaError_t e;
        const bool slab = p->host.slab_panels && slab_supports(nw, ldb, ldc, B + n0, C + n0);
        if (slab && rg) return fail(CUTESPMM_EUNSUPPORTED, "a plan with slab panels runs whole");
        if (slab) {
            SlabArgs sa = slab_args(p, B + n0, ldb, C + n0, ldc, nw);
            if ((e = launch_slab(sa, p->sm_count, s)) != cudaSuccess) return fail_cuda(e, "slab kernel launch");
        }
        const bool brick = use_brick(p, B + n0, ldb, C + n0, ldc, nw);
        if (brick) {
            BrickArgs ba = brick_args(p, B + n0, ldb, C + n0, ldc, nw, rg);
            if ((e = launch_brick(ba, p->sm_count, s)) != cudaSuccess) return fail_cuda(e, "brick kernel launch");
        }
        // brick panels whose shape the brick kernel does not take (N not a multiple of 32, unaligned
        // operands) are executed by the row kernel from its all-rows work list
        RowsArgs ra = rows_args(p, (!brick && p->host.num_bricks) || (!slab && p->host.slab_panels), B + n0, ldb, C + n0, ldc, nw, rg);
        if ((e = launch_rows(ra, p->sm_count, s)) != cudaSuccess) return fail_cuda(e, "row kernel launch");
    }
    return CUTESPMM_OK;
}

extern "C" {

int cutespmm_sddmm(const cutespmm_plan_t *p, const float *X, uint64_t ldx, const float *Y, uint64_t ldy, uint32_t N, int scale_by_values,
                   float *out, void *stream)
{
    if (!p) return fail(CUTESPMM_EINVAL, "plan is NULL");
    if (!p->on_device) return fail(CUTESPMM_EUNSUPPORTED, "host-only plan cannot execute");
    if (!p->host.row_map.empty()) return fail(CUTESPMM_EUNSUPPORTED, "SDDMM is not available for a plan with row reordering");
    const HostPlan &h = p->host;
    if (h.nnz == 0) return CUTESPMM_OK;
    if (!out) return fail(CUTESPMM_EINVAL, "out is NULL");
    if (N && (!X || !Y)) return fail(CUTESPMM_EINVAL, "X or Y is NULL");
    if (ldx < N || ldy < N) return fail(CUTESPMM_EINVAL, "leading dimension smaller than N");
    if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(Y) | reinterpret_cast<uintptr_t>(out)) & 3)
        return fail(CUTESPMM_EINVAL, "X, Y and out must be 4-byte aligned");
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != p->device)
        return fail(CUTESPMM_EINVAL, "the current CUDA device is not the one the plan was created on");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (N == 0) {  // an empty sum
        cudaError_t e = cudaMemsetAsync(out, 0, h.nnz * sizeof(float), s);
        return e == cudaSuccess ? CUTESPMM_OK : fail_cuda(e, "cudaMemsetAsync");
    }
    const bool all = h.num_bricks || h.slab_panels;  // the work list that covers every row
    SddmmArgs a{};
    a.row_ptr = static_cast<const uint32_t *>(p->d_row_ptr);
    a.pairs = p->d_pairs;
    a.tiles = all ? p->d_tiles_all : p->d_tiles;
    a.chunks = all ? p->d_chunks_all : p->d_chunks;
    a.num_tiles = (uint32_t)(all ? h.tiles_all.size() : h.tiles.size());
    a.num_chunks = (uint32_t)(all ? h.chunks_all.size() : h.chunks.size());
    a.X = X; a.Y = Y; a.ldx = ldx; a.ldy = ldy; a.out = out; a.N = N;
    a.scale = scale_by_values ? 1u : 0u;
    a.status = p->d_status;
    a.vec4 = !((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(Y)) & 15) && !((ldx | ldy) & 3) ? 1u : 0u;
    cudaError_t e = launch_sddmm(a, p->sm_count, s);
    return e == cudaSuccess ? CUTESPMM_OK : fail_cuda(e, "SDDMM kernel launch");
}

int cutespmm_plan_set_values(cutespmm_plan_t *p, const float *vals_dev, void *stream)
{
    if (!p) return fail(CUTESPMM_EINVAL, "plan is NULL");
    if (!p->on_device) return fail(CUTESPMM_EUNSUPPORTED, "host-only plan has no device arrays");
    const HostPlan &h = p->host;
    if (h.num_bricks || h.slab_panels)
        return fail(CUTESPMM_EUNSUPPORTED, "values can be replaced in a plan whose rows all run on the row kernel (path rows, or auto without dense panels)");
    if (!h.row_map.empty()) return fail(CUTESPMM_EUNSUPPORTED, "values cannot be replaced in a plan with row reordering");
    if (h.nnz == 0) return CUTESPMM_OK;
    if (!vals_dev) return fail(CUTESPMM_EINVAL, "vals is NULL");
    if (reinterpret_cast<uintptr_t>(vals_dev) & 3) return fail(CUTESPMM_EINVAL, "vals must be 4-byte aligned");
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != p->device)
        return fail(CUTESPMM_EINVAL, "the current CUDA device is not the one the plan was created on");
    const cudaError_t e = launch_set_values(p->d_pairs, vals_dev, h.nnz, p->sm_count, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail_cuda(e, "replacing the values");
    p->host.values_on_device = true;
    return CUTESPMM_OK;
}

int cutespmm_plan_device_status(const cutespmm_plan_t *p, uint32_t *status)
{
    if (!p || !status) return fail(CUTESPMM_EINVAL, "null argument");
    *status = 0;
    if (!p->on_device) return CUTESPMM_OK;
    cudaError_t e = cudaMemcpy(status, p->d_status, sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail_cuda(e, "reading the status word");
    // clear on read: a reported timeout does not stick to the launches that follow
    if (*status && (e = cudaMemset(p->d_status, 0, sizeof(uint32_t))) != cudaSuccess) return fail_cuda(e, "clearing the status word");
    return CUTESPMM_OK;
}

int cutespmm_partition_rows(uint64_t M, const uint64_t *rowPtr, uint32_t nparts, uint32_t align_rows, uint32_t row_cost,
                            uint64_t *bounds)
{
    std::string err;
    int st = partition_rows(M, rowPtr, nparts, align_rows, row_cost, bounds, err);
    return st == CUTESPMM_OK ? st : fail(st, err);
}

}  // extern "C"
