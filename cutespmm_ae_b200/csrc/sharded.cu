// Communicators and the sharded / host-buffer forms of the product.
//
// The reference runs one GPU (run.cu:8-72).  Here row panels are cut into one contiguous range per rank
// (cutespmm_partition_rows), every rank owns a plan over its rows, C stays row-sharded, and the single
// exchange of the path -- B into every rank's own memory -- goes through NCCL over NVLink: one broadcast
// when B starts on one rank, one all-gather (in place) when B is itself row-sharded, which is the shape of
// an iterative or layered use where the previous product's C is the next B.  Kernels only ever read local
// memory.
//
// NCCL is not a link dependency: it is opened at run time (libnccl.so.2, or the file $CUTESPMM_NCCL_LIB
// names) when the first communicator is created, so a single-GPU host needs no NCCL at all and a process
// that already loaded one (a PyTorch process) shares it.  Only the handful of entry points used here are
// declared, with the types of NCCL's public 2.x ABI.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "nvtx.hpp"
#include "plan_object.hpp"

using namespace cutespmm;

namespace {

// ---- the slice of NCCL's ABI this file uses -------------------------------------------------------
using nccl_comm_t = void *;
struct nccl_uid {
    char internal[CUTESPMM_COMM_ID_BYTES];
};
constexpr int kNcclSuccess = 0;
constexpr int kNcclFloat32 = 7;
struct NcclApi {
    int (*GetUniqueId)(nccl_uid *) = nullptr;
    int (*CommInitRank)(nccl_comm_t *, int, nccl_uid, int) = nullptr;
    int (*CommInitAll)(nccl_comm_t *, int, const int *) = nullptr;
    int (*CommDestroy)(nccl_comm_t) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    int (*Broadcast)(const void *, void *, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, nccl_comm_t, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    void *handle = nullptr;
    std::string error;
};

const NcclApi &nccl()
{
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char *names[] = {std::getenv("CUTESPMM_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
        for (const char *n : names) {
            if (!n || !*n) continue;
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
            api.error = dlerror();
        }
        if (!api.handle) {
            api.error = "cannot load NCCL (libnccl.so.2): " + api.error;
            return;
        }
        bool ok = true;
        auto sym = [&](const char *name) {
            void *p = dlsym(api.handle, name);
            if (!p) {
                ok = false;
                api.error = std::string("NCCL lacks ") + name;
            }
            return p;
        };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommInitAll = reinterpret_cast<decltype(api.CommInitAll)>(sym("ncclCommInitAll"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        api.Broadcast = reinterpret_cast<decltype(api.Broadcast)>(sym("ncclBroadcast"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
        if (!ok) api.handle = nullptr;
    });
    return api;
}

int fail_nccl(int r, const char *what)
{
    const NcclApi &n = nccl();
    return fail_status(CUTESPMM_ECOMM, std::string(what) + ": " + (n.GetErrorString ? n.GetErrorString(r) : "NCCL error"));
}

// One collective of the exchange: `count` floats at element `offset` of a contiguous block go from `root` to all.
struct Transfer {
    int root;
    uint64_t offset, count;
};

}  // namespace

struct cutespmm_comm {
    nccl_comm_t nccl = nullptr;
    int nranks = 1, rank = 0, device = -1;
    bool owned = false, stub = false;
    std::vector<Transfer> log;  // stub: what would have been sent
};

namespace {

// The exchange of a K x ld block of B (rows contiguous).  Pure bookkeeping.
int list_transfers(int nranks, int b_mode, int root, uint64_t K, uint64_t ld, const uint64_t *bounds, std::vector<Transfer> &out)
{
    out.clear();
    if (nranks <= 1 || b_mode == CUTESPMM_B_RESIDENT) return CUTESPMM_OK;
    if (b_mode == CUTESPMM_B_FROM_ROOT) {
        if (root < 0 || root >= nranks) return fail_status(CUTESPMM_EINVAL, "root is not a rank of the communicator");
        if (K != 0 && ld != 0) out.push_back(Transfer{root, 0, K * ld});
        return CUTESPMM_OK;
    }
    if (b_mode != CUTESPMM_B_ROW_SHARDED) return fail_status(CUTESPMM_EINVAL, "unknown b_mode");
    if (!bounds) return fail_status(CUTESPMM_EINVAL, "b_bounds is NULL");
    if (bounds[0] != 0 || bounds[nranks] != K) return fail_status(CUTESPMM_EINVAL, "b_bounds must start at 0 and end at K");
    for (int r = 0; r < nranks; ++r) {
        if (bounds[r + 1] < bounds[r]) return fail_status(CUTESPMM_EINVAL, "b_bounds is not non-decreasing");
        if (bounds[r + 1] > bounds[r]) out.push_back(Transfer{r, bounds[r] * ld, (bounds[r + 1] - bounds[r]) * ld});
    }
    return CUTESPMM_OK;
}

// Equal slices in rank order are one in-place all-gather; anything else is one broadcast per slice, grouped.
bool is_all_gather(const std::vector<Transfer> &t, int nranks)
{
    if ((int)t.size() != nranks || nranks < 2) return false;
    for (int r = 0; r < nranks; ++r)
        if (t[r].root != r || t[r].count != t[0].count || t[r].offset != (uint64_t)r * t[0].count) return false;
    return true;
}

int run_exchange(cutespmm_comm *comm, const std::vector<Transfer> &t, float *block, cudaStream_t s)
{
    if (t.empty()) return CUTESPMM_OK;
    if (comm->stub) {
        comm->log.insert(comm->log.end(), t.begin(), t.end());
        return CUTESPMM_OK;
    }
    const NcclApi &n = nccl();
    if (!n.handle) return fail_status(CUTESPMM_ECOMM, n.error);
    NvtxRange range("cutespmm: exchange of B");
    int r;
    if (is_all_gather(t, comm->nranks)) {
        r = n.AllGather(block + (uint64_t)comm->rank * t[0].count, block, t[0].count, kNcclFloat32, comm->nccl, s);
        return r == kNcclSuccess ? CUTESPMM_OK : fail_nccl(r, "ncclAllGather");
    }
    if (t.size() > 1 && (r = n.GroupStart()) != kNcclSuccess) return fail_nccl(r, "ncclGroupStart");
    int first_bad = kNcclSuccess;
    for (const Transfer &x : t) {
        r = n.Broadcast(block + x.offset, block + x.offset, x.count, kNcclFloat32, x.root, comm->nccl, s);
        if (r != kNcclSuccess && first_bad == kNcclSuccess) first_bad = r;
    }
    if (t.size() > 1 && (r = n.GroupEnd()) != kNcclSuccess && first_bad == kNcclSuccess) first_bad = r;
    return first_bad == kNcclSuccess ? CUTESPMM_OK : fail_nccl(first_bad, "ncclBroadcast");
}

int new_comm(cutespmm_comm_t **out, nccl_comm_t c, int nranks, int rank, int device, bool owned, bool stub)
{
    cutespmm_comm *m = new (std::nothrow) cutespmm_comm();
    if (!m) return fail_status(CUTESPMM_ENOMEM, "host allocation failed");
    m->nccl = c; m->nranks = nranks; m->rank = rank; m->device = device; m->owned = owned; m->stub = stub;
    *out = m;
    return CUTESPMM_OK;
}

}  // namespace

namespace {

// How a host-buffer call cuts N columns into windows, and the staging it needs on the device.
struct Windows {
    uint32_t count = 1, width = 0;
    uint64_t ldd = 0;  // leading dimension of a window on the device
};

// Column windows are independent products (C[:, w] = A * B[:, w]), so a host-buffer call is a pipeline over them: while
// window w is exchanged, multiplied and copied out, window w+1 is already coming in; the two copy directions run on
// different engines.  Small operands go in one piece.  With several ranks the cut must be the same on all of them (the
// exchanges pair up window by window), so it depends on K and N only.  Allocates (or grows) the plan's staging buffers,
// streams and events; a call that finds them large enough allocates nothing.
int ensure_staging(cutespmm_plan *p, uint32_t N, bool sharded, Windows &w)
{
    const uint64_t M = p->host.M, K = p->host.K;
    const uint64_t rows_for_cut = sharded ? K : std::max(M, K);
    uint32_t nw = 1;
    if ((uint64_t)N * rows_for_cut * sizeof(float) >= (8u << 20)) nw = std::max(1u, std::min<uint32_t>(cutespmm_plan::kMaxWindows, N / 64));
    // window width: a multiple of 64 columns (the last may be narrower); strided copies of rows shorter than 256 bytes
    // were measured at 2/3 of the link rate, 256-byte rows at the full rate
    w.width = ((N + nw - 1) / nw + 63) / 64 * 64;
    w.count = (N + w.width - 1) / w.width;
    w.ldd = w.count == 1 ? (uint64_t)(N + 3) / 4 * 4 : w.width;  // rows start 16-byte aligned
    const uint64_t needB = (uint64_t)w.count * K * w.ldd * sizeof(float), needC = (uint64_t)w.count * M * w.ldd * sizeof(float);
    cudaError_t e;
    if (needB > p->staged_B) {
        if (p->d_B) cudaFree(p->d_B);
        p->d_B = nullptr; p->staged_B = 0;
        if ((e = cudaMalloc(&p->d_B, needB)) != cudaSuccess) return fail_cuda_status(e, "staging buffer for B");
        p->staged_B = needB;
    }
    if (needC > p->staged_C) {
        if (p->d_C) cudaFree(p->d_C);
        p->d_C = nullptr; p->staged_C = 0;
        if ((e = cudaMalloc(&p->d_C, needC)) != cudaSuccess) return fail_cuda_status(e, "staging buffer for C");
        p->staged_C = needC;
    }
    if (!p->s_in) {
        if ((e = cudaStreamCreateWithFlags(&p->s_in, cudaStreamNonBlocking)) != cudaSuccess ||
            (e = cudaStreamCreateWithFlags(&p->s_x, cudaStreamNonBlocking)) != cudaSuccess ||
            (e = cudaStreamCreateWithFlags(&p->s_out, cudaStreamNonBlocking)) != cudaSuccess)
            return fail_cuda_status(e, "cudaStreamCreate");
        if ((e = cudaEventCreateWithFlags(&p->ev_entry, cudaEventDisableTiming)) != cudaSuccess ||
            (e = cudaEventCreateWithFlags(&p->ev_done, cudaEventDisableTiming)) != cudaSuccess)
            return fail_cuda_status(e, "cudaEventCreate");
        for (int i = 0; i < cutespmm_plan::kMaxWindows; ++i)
            if ((e = cudaEventCreateWithFlags(&p->ev_in[i], cudaEventDisableTiming)) != cudaSuccess ||
                (e = cudaEventCreate(&p->ev_x0[i])) != cudaSuccess || (e = cudaEventCreate(&p->ev_x1[i])) != cudaSuccess ||
                (e = cudaEventCreate(&p->ev_k0[i])) != cudaSuccess || (e = cudaEventCreate(&p->ev_k1[i])) != cudaSuccess)
                return fail_cuda_status(e, "cudaEventCreate");
    }
    return CUTESPMM_OK;
}

// ---- the single-GPU host-buffer call in blocks of rows -------------------------------------------------------------
// For a matrix whose rows name a bounded, advancing range of columns (banded and block-structured matrices) the rows
// of C of an early block need only the leading rows of B.  The call then uploads B in row order, launches the product
// block of rows by block of rows as soon as the rows of B a block needs are on the device, and sends each block's
// rows of C back while later rows of B are still arriving: the two PCIe directions overlap at full width (no column
// windows, so every launch keeps the full-width kernels).

// Cuts the plan's rows into blocks and finds, per block, its work items and how many leading rows of B it needs.
// Returns false when the matrix does not qualify (half of the rows already need more than 80 % of B, too small, ...).
bool cut_row_blocks(cutespmm_plan *p, uint32_t N)
{
    const HostPlan &h = p->host;
    p->row_blocks.clear();
    if (!h.row_map.empty() || h.slab_panels || h.panel_max_col.size() != h.num_panels() || h.M < 4096) return false;
    const uint64_t c_bytes = h.M * (uint64_t)N * sizeof(float);
    // blocks of about 16 MiB of C: every block costs about 40 us of hand-over between the copy engines and its kernel
    // (measured: 6-8 blocks are best for 134 MB, 16 blocks lose what the finer overlap gains)
    int R = (int)std::min<uint64_t>(cutespmm_plan::kMaxRowBlocks, c_bytes / (16u << 20));
    if (R < 2) return false;
    // boundaries: near equal row counts, on 16-row panel boundaries, never inside a tile of either tile list
    auto snap = [&](uint64_t target, const std::vector<Tile> &tiles) {
        auto it = std::upper_bound(tiles.begin(), tiles.end(), target, [](uint64_t r, const Tile &t) { return r < t.row_begin; });
        if (it != tiles.begin()) {
            const Tile &t = *(it - 1);
            if (t.row_begin < target && target < t.row_end) return (uint64_t)t.row_begin;
        }
        return target;
    };
    std::vector<uint32_t> bounds(1, 0u);
    for (int i = 1; i < R; ++i) {
        uint64_t r = (uint64_t)i * h.M / R / kPanelRows * kPanelRows;
        for (int pass = 0; pass < 4; ++pass) {  // the two tile lists may pull the boundary down in turn
            const uint64_t before = r;
            r = snap(r, h.tiles);
            r = snap(r, h.tiles_all);
            if (r == before) break;
        }
        if (r > bounds.back()) bounds.push_back((uint32_t)r);
    }
    bounds.push_back((uint32_t)h.M);
    auto first_at = [](const auto &list, uint32_t row, auto key) {
        return (uint32_t)(std::lower_bound(list.begin(), list.end(), row, [&](const auto &x, uint32_t r) { return key(x) < r; }) - list.begin());
    };
    uint32_t need = 0;
    for (size_t i = 0; i + 1 < bounds.size(); ++i) {
        cutespmm_row_block b;
        b.row0 = bounds[i];
        b.row1 = bounds[i + 1];
        auto &it = b.items;
        it.t0 = first_at(h.tiles, b.row0, [](const Tile &t) { return t.row_begin; });
        it.t1 = first_at(h.tiles, b.row1, [](const Tile &t) { return t.row_begin; });
        it.c0 = first_at(h.chunks, b.row0, [](const Chunk &c) { return c.row; });
        it.c1 = first_at(h.chunks, b.row1, [](const Chunk &c) { return c.row; });
        it.ta0 = first_at(h.tiles_all, b.row0, [](const Tile &t) { return t.row_begin; });
        it.ta1 = first_at(h.tiles_all, b.row1, [](const Tile &t) { return t.row_begin; });
        it.ca0 = first_at(h.chunks_all, b.row0, [](const Chunk &c) { return c.row; });
        it.ca1 = first_at(h.chunks_all, b.row1, [](const Chunk &c) { return c.row; });
        it.p0 = first_at(h.brick_panel_ids, b.row0 / kPanelRows, [](uint32_t q) { return q; });
        it.p1 = first_at(h.brick_panel_ids, (b.row1 + kPanelRows - 1) / kPanelRows, [](uint32_t q) { return q; });
        for (uint64_t q = b.row0 / kPanelRows; q < (b.row1 + kPanelRows - 1) / kPanelRows; ++q)
            if (h.row_ptr[std::min<uint64_t>(h.M, (q + 1) * kPanelRows)] > h.row_ptr[q * kPanelRows]) need = std::max(need, h.panel_max_col[q] + 1);
        b.need = need;  // running maximum: B arrives in row order
        p->row_blocks.push_back(b);
    }
    if (h.brick_panels && h.brick_panel_ids.size() != h.brick_panels) { p->row_blocks.clear(); return false; }
    const size_t half = p->row_blocks.size() / 2;
    if (p->row_blocks.size() < 2 || (uint64_t)p->row_blocks[half - 1].need * 10 > h.K * 8) {
        p->row_blocks.clear();
        return false;
    }
    return true;
}

// rows x N floats between host and device; one plain copy when both sides are contiguous (faster than the 2-D form)
cudaError_t copy_rows(void *dst, uint64_t ld_dst, const void *src, uint64_t ld_src, uint32_t N, uint64_t rows, cudaMemcpyKind kind, cudaStream_t s)
{
    if (ld_dst == N && ld_src == N) return cudaMemcpyAsync(dst, src, rows * N * sizeof(float), kind, s);
    return cudaMemcpy2DAsync(dst, ld_dst * sizeof(float), src, ld_src * sizeof(float), (size_t)N * sizeof(float), rows, kind, s);
}

int run_row_blocks(cutespmm_plan *p, const float *B_host, uint64_t ldb, float *C_host, uint64_t ldc, uint32_t N, cudaStream_t s, float *kernel_ms)
{
    const uint64_t M = p->host.M, K = p->host.K;
    const uint64_t ldd = (uint64_t)(N + 3) / 4 * 4;
    cudaError_t e;
    if (!p->rb_in[0])
        for (int i = 0; i < cutespmm_plan::kMaxRowBlocks; ++i)
            if ((e = cudaEventCreateWithFlags(&p->rb_in[i], cudaEventDisableTiming)) != cudaSuccess || (e = cudaEventCreate(&p->rb_k0[i])) != cudaSuccess ||
                (e = cudaEventCreate(&p->rb_k1[i])) != cudaSuccess)
                return fail_cuda_status(e, "cudaEventCreate");
    auto drain = [&]() {
        cudaStreamSynchronize(p->s_in);
        cudaStreamSynchronize(p->s_out);
        cudaStreamSynchronize(s);
    };
    NvtxRange range("cutespmm: product from host buffers, in blocks of rows");
    cudaEventRecord(p->ev_entry, s);  // whatever the caller queued on `stream` comes first
    cudaStreamWaitEvent(p->s_in, p->ev_entry, 0);
    // All uploads are queued before the first download, so that no download waiting for its kernel sits in front of an
    // upload in a copy queue.
    uint64_t have = 0;  // rows of B already queued for upload
    const size_t nb = p->row_blocks.size();
    for (size_t i = 0; i < nb; ++i) {
        const uint64_t upto = std::min<uint64_t>(K, p->row_blocks[i].need);  // rows of B beyond the last column any row names are never read
        if (upto > have) {
            if ((e = copy_rows(p->d_B + have * ldd, ldd, B_host + have * ldb, ldb, N, upto - have, cudaMemcpyHostToDevice, p->s_in)) != cudaSuccess) {
                drain();
                return fail_cuda_status(e, "copy of B to the device");
            }
            have = upto;
        }
        cudaEventRecord(p->rb_in[i], p->s_in);
    }
    for (size_t i = 0; i < nb; ++i) {
        const cutespmm_row_block &b = p->row_blocks[i];
        cudaStreamWaitEvent(s, p->rb_in[i], 0);
        cudaEventRecord(p->rb_k0[i], s);
        const int st = cutespmm_internal_spmm_range(p, p->d_B, ldd, p->d_C, ldd, N, s, &b.items);
        if (st != CUTESPMM_OK) {
            drain();
            return st;
        }
        cudaEventRecord(p->rb_k1[i], s);
        cudaStreamWaitEvent(p->s_out, p->rb_k1[i], 0);
        if (b.row1 > b.row0 && (e = copy_rows(C_host + (uint64_t)b.row0 * ldc, ldc, p->d_C + (uint64_t)b.row0 * ldd, ldd, N, b.row1 - b.row0,
                                              cudaMemcpyDeviceToHost, p->s_out)) != cudaSuccess) {
            drain();
            return fail_cuda_status(e, "copy of C to the host");
        }
    }
    (void)M;
    cudaEventRecord(p->ev_done, p->s_out);
    cudaStreamWaitEvent(s, p->ev_done, 0);
    if ((e = cudaStreamSynchronize(s)) != cudaSuccess) return fail_cuda_status(e, "SpMM execution");
    if (kernel_ms) {
        *kernel_ms = 0.f;
        for (size_t i = 0; i < nb; ++i) {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, p->rb_k0[i], p->rb_k1[i]) == cudaSuccess) *kernel_ms += ms;
        }
    }
    uint32_t dev_status = 0;
    cutespmm_plan_device_status(p, &dev_status);
    if (dev_status) return fail_status(CUTESPMM_ETIMEOUT, "a device-side wait ran out (status " + std::to_string(dev_status) + ")");
    return CUTESPMM_OK;
}

}  // namespace

extern "C" {

int cutespmm_plan_reserve_host_staging(cutespmm_plan_t *p, uint32_t N, int sharded)
{
    if (!p) return fail_status(CUTESPMM_EINVAL, "plan is NULL");
    if (!p->on_device) return fail_status(CUTESPMM_EUNSUPPORTED, "host-only plan cannot execute");
    if (N == 0) return CUTESPMM_OK;
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != p->device)
        return fail_status(CUTESPMM_EINVAL, "the current CUDA device is not the one the plan was created on");
    Windows w;
    return ensure_staging(p, N, sharded != 0, w);
}

int cutespmm_comm_unique_id(void *id_out)
{
    if (!id_out) return fail_status(CUTESPMM_EINVAL, "id_out is NULL");
    const NcclApi &n = nccl();
    if (!n.handle) return fail_status(CUTESPMM_ECOMM, n.error);
    nccl_uid id;
    const int r = n.GetUniqueId(&id);
    if (r != kNcclSuccess) return fail_nccl(r, "ncclGetUniqueId");
    std::memcpy(id_out, &id, sizeof(id));
    return CUTESPMM_OK;
}

int cutespmm_comm_create(cutespmm_comm_t **comm, int nranks, int rank, const void *id)
{
    if (!comm || !id) return fail_status(CUTESPMM_EINVAL, "null argument");
    *comm = nullptr;
    if (nranks < 1 || rank < 0 || rank >= nranks) return fail_status(CUTESPMM_EINVAL, "rank outside [0, nranks)");
    const NcclApi &n = nccl();
    if (!n.handle) return fail_status(CUTESPMM_ECOMM, n.error);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail_cuda_status(e, "cudaGetDevice");
    nccl_uid uid;
    std::memcpy(&uid, id, sizeof(uid));
    nccl_comm_t c = nullptr;
    const int r = n.CommInitRank(&c, nranks, uid, rank);
    if (r != kNcclSuccess) return fail_nccl(r, "ncclCommInitRank");
    const int st = new_comm(comm, c, nranks, rank, dev, true, false);
    if (st != CUTESPMM_OK) n.CommDestroy(c);
    return st;
}

int cutespmm_comm_create_all(cutespmm_comm_t **comms, int ndev, const int *devices)
{
    if (!comms || ndev < 1) return fail_status(CUTESPMM_EINVAL, "bad argument");
    for (int i = 0; i < ndev; ++i) comms[i] = nullptr;
    const NcclApi &n = nccl();
    if (!n.handle) return fail_status(CUTESPMM_ECOMM, n.error);
    std::vector<int> devs(ndev);
    for (int i = 0; i < ndev; ++i) devs[i] = devices ? devices[i] : i;
    std::vector<nccl_comm_t> cs(ndev, nullptr);
    const int r = n.CommInitAll(cs.data(), ndev, devs.data());
    if (r != kNcclSuccess) return fail_nccl(r, "ncclCommInitAll");
    for (int i = 0; i < ndev; ++i) {
        const int st = new_comm(&comms[i], cs[i], ndev, i, devs[i], true, false);
        if (st != CUTESPMM_OK) {
            for (int j = 0; j < ndev; ++j) {
                if (j < i) { comms[j]->owned = false; delete comms[j]; comms[j] = nullptr; }
                n.CommDestroy(cs[j]);
            }
            return st;
        }
    }
    return CUTESPMM_OK;
}

int cutespmm_comm_adopt(cutespmm_comm_t **comm, void *nccl_comm, int nranks, int rank)
{
    if (!comm || !nccl_comm) return fail_status(CUTESPMM_EINVAL, "null argument");
    *comm = nullptr;
    if (nranks < 1 || rank < 0 || rank >= nranks) return fail_status(CUTESPMM_EINVAL, "rank outside [0, nranks)");
    const NcclApi &n = nccl();
    if (!n.handle) return fail_status(CUTESPMM_ECOMM, n.error);
    int dev = -1;
    cudaGetDevice(&dev);
    return new_comm(comm, nccl_comm, nranks, rank, dev, false, false);
}

int cutespmm_comm_create_stub(cutespmm_comm_t **comm, int nranks, int rank)
{
    if (!comm) return fail_status(CUTESPMM_EINVAL, "null argument");
    *comm = nullptr;
    if (nranks < 1 || rank < 0 || rank >= nranks) return fail_status(CUTESPMM_EINVAL, "rank outside [0, nranks)");
    return new_comm(comm, nullptr, nranks, rank, -1, false, true);
}

int cutespmm_comm_info(const cutespmm_comm_t *comm, int *nranks, int *rank)
{
    if (!comm) return fail_status(CUTESPMM_EINVAL, "comm is NULL");
    if (nranks) *nranks = comm->nranks;
    if (rank) *rank = comm->rank;
    return CUTESPMM_OK;
}

int cutespmm_comm_stub_log(cutespmm_comm_t *comm, uint32_t max, int *roots, uint64_t *offsets, uint64_t *counts, uint32_t *n)
{
    if (!comm || !n) return fail_status(CUTESPMM_EINVAL, "null argument");
    if (!comm->stub) return fail_status(CUTESPMM_EINVAL, "not a stub communicator");
    *n = (uint32_t)comm->log.size();
    for (uint32_t i = 0; i < comm->log.size() && i < max; ++i) {
        if (roots) roots[i] = comm->log[i].root;
        if (offsets) offsets[i] = comm->log[i].offset;
        if (counts) counts[i] = comm->log[i].count;
    }
    comm->log.clear();
    return CUTESPMM_OK;
}

int cutespmm_comm_destroy(cutespmm_comm_t *comm)
{
    if (!comm) return CUTESPMM_OK;
    if (comm->owned && comm->nccl) {
        int cur = -1;
        cudaGetDevice(&cur);
        if (comm->device >= 0 && cur != comm->device) cudaSetDevice(comm->device);
        nccl().CommDestroy(comm->nccl);
        if (comm->device >= 0 && cur >= 0 && cur != comm->device) cudaSetDevice(cur);
    }
    delete comm;
    return CUTESPMM_OK;
}

int cutespmm_sharded_transfers(const cutespmm_comm_t *comm, int b_mode, int root, uint64_t K, uint64_t N, const uint64_t *b_bounds,
                               uint32_t max, int *roots, uint64_t *offsets, uint64_t *counts, uint32_t *n)
{
    if (!comm || !n) return fail_status(CUTESPMM_EINVAL, "null argument");
    std::vector<Transfer> t;
    const int st = list_transfers(comm->nranks, b_mode, root, K, N, b_bounds, t);
    if (st != CUTESPMM_OK) return st;
    *n = (uint32_t)t.size();
    for (uint32_t i = 0; i < t.size() && i < max; ++i) {
        if (roots) roots[i] = t[i].root;
        if (offsets) offsets[i] = t[i].offset;
        if (counts) counts[i] = t[i].count;
    }
    return CUTESPMM_OK;
}

int cutespmm_spmm_sharded(const cutespmm_plan_t *plan, cutespmm_comm_t *comm, int b_mode, int root, float *B_dev, uint64_t ldb,
                          const uint64_t *b_bounds, float *C_dev, uint64_t ldc, uint32_t N, void *stream)
{
    if (!plan) return fail_status(CUTESPMM_EINVAL, "plan is NULL");
    if (N == 0) return CUTESPMM_OK;
    const int nranks = comm ? comm->nranks : 1;
    if (nranks > 1 && b_mode != CUTESPMM_B_RESIDENT) {
        if (!B_dev) return fail_status(CUTESPMM_EINVAL, "B is NULL");
        if (ldb != N) return fail_status(CUTESPMM_EUNSUPPORTED, "the exchange needs the rows of B contiguous (ldb == N)");
        std::vector<Transfer> t;
        int st = list_transfers(nranks, b_mode, root, plan->host.K, ldb, b_bounds, t);
        if (st != CUTESPMM_OK) return st;
        if ((st = run_exchange(comm, t, B_dev, static_cast<cudaStream_t>(stream))) != CUTESPMM_OK) return st;
    }
    if (comm && comm->stub && !plan->on_device) return CUTESPMM_OK;  // bookkeeping only: nothing to execute
    NvtxRange range("cutespmm: product");
    return cutespmm_spmm(plan, B_dev, ldb, C_dev, ldc, N, stream);
}

int cutespmm_spmm_sharded_host(cutespmm_plan_t *p, cutespmm_comm_t *comm, const float *B_host_rows, uint64_t ldb,
                               const uint64_t *b_bounds, float *C_host, uint64_t ldc, uint32_t N, void *stream, float *kernel_ms,
                               float *exchange_ms)
{
    if (!p) return fail_status(CUTESPMM_EINVAL, "plan is NULL");
    if (!p->on_device) return fail_status(CUTESPMM_EUNSUPPORTED, "host-only plan cannot execute");
    if (N == 0) return CUTESPMM_OK;
    const uint64_t M = p->host.M, K = p->host.K;
    const int nranks = comm ? comm->nranks : 1, rank = comm ? comm->rank : 0;
    const uint64_t whole[2] = {0, K};
    if (!b_bounds) {
        if (nranks > 1) return fail_status(CUTESPMM_EINVAL, "b_bounds is NULL");
        b_bounds = whole;
    }
    std::vector<Transfer> unit;  // the exchange of a K x 1 block; scaled by the window's leading dimension below
    int st = list_transfers(nranks, nranks > 1 ? CUTESPMM_B_ROW_SHARDED : CUTESPMM_B_RESIDENT, 0, K, 1, b_bounds, unit);
    if (st != CUTESPMM_OK) return st;
    if (nranks == 1 && (b_bounds[0] != 0 || b_bounds[1] != K)) return fail_status(CUTESPMM_EINVAL, "b_bounds must be {0, K} for one rank");
    const uint64_t k0 = b_bounds[rank], k1 = b_bounds[rank + 1];
    if ((k1 > k0 && !B_host_rows) || (M && !C_host)) return fail_status(CUTESPMM_EINVAL, "null host buffer");
    if (ldb < N || ldc < N) return fail_status(CUTESPMM_EINVAL, "leading dimension smaller than N");
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != p->device)
        return fail_status(CUTESPMM_EINVAL, "the current CUDA device is not the one the plan was created on");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    Windows wn;
    if ((st = ensure_staging(p, N, nranks > 1, wn)) != CUTESPMM_OK) return st;
    if (nranks == 1 && N <= kScratchCols && (uint64_t)N * std::max(M, K) * sizeof(float) >= (8u << 20)) {
        // large operands on one GPU: blocks of rows where the matrix allows it, column windows otherwise
        if (!p->row_blocks_tried || p->row_blocks_n != N) {
            p->row_blocks_tried = true;
            p->row_blocks_n = N;
            try {
                cut_row_blocks(p, N);
            } catch (const std::bad_alloc &) {
                p->row_blocks.clear();
            }
        }
        if (!p->row_blocks.empty()) {
            if (exchange_ms) *exchange_ms = 0.f;
            return run_row_blocks(p, B_host_rows, ldb, C_host, ldc, N, s, kernel_ms);
        }
    }
    const uint32_t nw = wn.count, wcols = wn.width;
    const uint64_t ldd = wn.ldd;
    auto drain = [&]() {
        cudaStreamSynchronize(p->s_in);
        cudaStreamSynchronize(p->s_x);
        cudaStreamSynchronize(p->s_out);
        cudaStreamSynchronize(s);
    };
    NvtxRange range("cutespmm: product from host buffers");
    // whatever the caller queued on `stream` comes first
    cudaEventRecord(p->ev_entry, s);
    cudaStreamWaitEvent(p->s_in, p->ev_entry, 0);
    std::vector<Transfer> t(unit.size());
    // every upload is queued before the first download, so that no download waiting for its kernel sits in front of
    // an upload in a copy queue
    for (uint32_t w = 0; w < nw; ++w) {
        const uint32_t c0 = w * wcols, cw = std::min(wcols, N - c0);
        float *dB = p->d_B + (uint64_t)w * K * ldd;
        if (k1 > k0 && (e = cudaMemcpy2DAsync(dB + k0 * ldd, ldd * sizeof(float), B_host_rows + c0, ldb * sizeof(float),
                                              (size_t)cw * sizeof(float), k1 - k0, cudaMemcpyHostToDevice, p->s_in)) != cudaSuccess) {
            drain();
            return fail_cuda_status(e, "copy of B to the device");
        }
        cudaEventRecord(p->ev_in[w], p->s_in);
    }
    for (uint32_t w = 0; w < nw; ++w) {
        const uint32_t c0 = w * wcols, cw = std::min(wcols, N - c0);
        float *dB = p->d_B + (uint64_t)w * K * ldd, *dC = p->d_C + (uint64_t)w * M * ldd;
        if (!unit.empty()) {  // the slices of this window meet on every rank
            cudaStreamWaitEvent(p->s_x, p->ev_in[w], 0);
            cudaEventRecord(p->ev_x0[w], p->s_x);
            for (size_t i = 0; i < unit.size(); ++i) t[i] = Transfer{unit[i].root, unit[i].offset * ldd, unit[i].count * ldd};
            if ((st = run_exchange(comm, t, dB, p->s_x)) != CUTESPMM_OK) {
                drain();
                return st;
            }
            cudaEventRecord(p->ev_x1[w], p->s_x);
            cudaStreamWaitEvent(s, p->ev_x1[w], 0);
        } else {
            cudaStreamWaitEvent(s, p->ev_in[w], 0);
        }
        cudaEventRecord(p->ev_k0[w], s);
        st = cutespmm_spmm(p, dB, ldd, dC, ldd, cw, s);
        if (st != CUTESPMM_OK) {
            drain();
            return st;
        }
        cudaEventRecord(p->ev_k1[w], s);
        cudaStreamWaitEvent(p->s_out, p->ev_k1[w], 0);
        if (M && (e = cudaMemcpy2DAsync(C_host + c0, ldc * sizeof(float), dC, ldd * sizeof(float), (size_t)cw * sizeof(float), M,
                                        cudaMemcpyDeviceToHost, p->s_out)) != cudaSuccess) {
            drain();
            return fail_cuda_status(e, "copy of C to the host");
        }
    }
    cudaEventRecord(p->ev_done, p->s_out);
    cudaStreamWaitEvent(s, p->ev_done, 0);  // later work on `stream` sees the finished call
    if ((e = cudaStreamSynchronize(s)) != cudaSuccess) return fail_cuda_status(e, "SpMM execution");
    if (kernel_ms) *kernel_ms = 0.f;
    if (exchange_ms) *exchange_ms = 0.f;
    for (uint32_t w = 0; w < nw; ++w) {
        float ms = 0.f;
        if (kernel_ms && cudaEventElapsedTime(&ms, p->ev_k0[w], p->ev_k1[w]) == cudaSuccess) *kernel_ms += ms;
        if (exchange_ms && !unit.empty() && !(comm && comm->stub) && cudaEventElapsedTime(&ms, p->ev_x0[w], p->ev_x1[w]) == cudaSuccess)
            *exchange_ms += ms;
    }
    uint32_t dev_status = 0;
    cutespmm_plan_device_status(p, &dev_status);
    if (dev_status) return fail_status(CUTESPMM_ETIMEOUT, "a device-side wait ran out (status " + std::to_string(dev_status) + ")");
    return CUTESPMM_OK;
}

int cutespmm_spmm_host(cutespmm_plan_t *p, const float *B_host, uint64_t ldb, float *C_host, uint64_t ldc, uint32_t N, void *stream,
                       float *kernel_ms)
{
    return cutespmm_spmm_sharded_host(p, nullptr, B_host, ldb, nullptr, C_host, ldc, N, stream, kernel_ms, nullptr);
}

}  // extern "C"
