// Saving a plan to a file and loading it back: preprocessing done once can be reused by a later run (the
// reference preprocesses every matrix at every start, run.cu:17-20, and times it as preprocessing_time).
//
// File layout (little-endian, as the machine writes it; the tag word detects the other kind):
//     16 bytes  "CUTESPMM-PLAN\0\0\0"
//     u32 version, u32 byte-order tag 0x01020304, u64 M, K, nnz, cutespmm_options_t, u32 device_built, u32 0
//     u64 num_bricks, brick_panels, brick_slots, slab_steps, slab_panels
//     sections  { u32 id, u32 element size, u64 count, count * size bytes }   one per array of the plan
//     u32 id 0, u32 0, u64 checksum (FNV-1a over everything before this section)
// A plan built on the device keeps its nonzeros and bricks in device memory only: saving brings them back first.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "plan_object.hpp"

using namespace cutespmm;

int cutespmm_internal_upload_plan(cutespmm_plan *p);  // capi.cu: current device checked, arrays uploaded

namespace {

constexpr char kMagic[16] = {'C', 'U', 'T', 'E', 'S', 'P', 'M', 'M', '-', 'P', 'L', 'A', 'N', 0, 0, 0};
constexpr uint32_t kVersion = 1, kOrderTag = 0x01020304u;

struct Writer {
    FILE *f;
    uint64_t hash = 1469598103934665603ull;
    bool ok = true;
    void bytes(const void *p, size_t n)
    {
        if (!ok || n == 0) return;
        const unsigned char *c = static_cast<const unsigned char *>(p);
        for (size_t i = 0; i < n; ++i) hash = (hash ^ c[i]) * 1099511628211ull;
        ok = std::fwrite(p, 1, n, f) == n;
    }
    template <class T> void pod(const T &v) { bytes(&v, sizeof(T)); }
    template <class T> void section(uint32_t id, const std::vector<T> &v)
    {
        pod(id);
        pod((uint32_t)sizeof(T));
        pod((uint64_t)v.size());
        bytes(v.data(), v.size() * sizeof(T));
    }
};

struct Reader {
    FILE *f;
    uint64_t hash = 1469598103934665603ull;
    bool ok = true;
    void bytes(void *p, size_t n)
    {
        if (!ok || n == 0) return;
        ok = std::fread(p, 1, n, f) == n;
        if (!ok) return;
        const unsigned char *c = static_cast<const unsigned char *>(p);
        for (size_t i = 0; i < n; ++i) hash = (hash ^ c[i]) * 1099511628211ull;
    }
    template <class T> void pod(T &v) { bytes(&v, sizeof(T)); }
};

// The arrays of a plan by section id.  One table for both directions keeps writer and reader in step.
template <class Fn> void for_each_array(HostPlan &h, Fn &&fn)
{
    fn(1, h.row_ptr); fn(2, h.pairs); fn(3, h.tiles); fn(4, h.row_path); fn(5, h.chunks); fn(6, h.long_rows);
    fn(7, h.blocked_row_ptr); fn(8, h.active_cols); fn(9, h.tiles_all); fn(10, h.chunks_all); fn(11, h.long_rows_all);
    fn(12, h.brick_cols); fn(13, h.brick_recs); fn(14, h.brick_rec_off); fn(15, h.panel_first_brick); fn(16, h.panel_last_brick);
    fn(17, h.brick_panel_ids); fn(18, h.slab_cols); fn(19, h.slab_recs); fn(20, h.slab_rec_off); fn(21, h.slab_first);
    fn(22, h.slab_last); fn(23, h.slab_ids); fn(24, h.slab_path); fn(25, h.row_map); fn(26, h.panel_max_col);
}

}  // namespace

extern "C" {

int cutespmm_plan_save(const cutespmm_plan_t *plan, const char *path)
{
    if (!plan || !path) return fail_status(CUTESPMM_EINVAL, "null argument");
    HostPlan h;  // a copy: a device-built plan gets its device-only arrays filled in below
    try {
        h = plan->host;
        if ((plan->host.device_built || plan->host.values_on_device) && plan->on_device) {
            int cur = -1;
            cudaGetDevice(&cur);
            if (cur != plan->device) cudaSetDevice(plan->device);
            cudaError_t e = cudaSuccess;
            h.pairs.resize(h.nnz);
            if (h.nnz) e = cudaMemcpy(h.pairs.data(), plan->d_pairs, h.nnz * sizeof(Pair), cudaMemcpyDeviceToHost);
            if (e == cudaSuccess && h.brick_slots) {
                h.brick_cols.resize(h.brick_slots * kBrickCols);
                h.brick_recs.resize(h.brick_slots * kBrickRecWords);
                h.brick_rec_off.resize(h.brick_slots + 1);
                for (uint64_t k = 0; k <= h.brick_slots; ++k) h.brick_rec_off[k] = (uint32_t)(k * (kBrickRecWords / 4));
                e = cudaMemcpy(h.brick_cols.data(), plan->d_bcols, h.brick_cols.size() * 4, cudaMemcpyDeviceToHost);
                if (e == cudaSuccess) e = cudaMemcpy(h.brick_recs.data(), plan->d_brecs, h.brick_recs.size() * 4, cudaMemcpyDeviceToHost);
            }
            if (cur != plan->device && cur >= 0) cudaSetDevice(cur);
            if (e != cudaSuccess) return fail_cuda_status(e, "reading the plan back from the device");
        }
    } catch (const std::bad_alloc &) {
        return fail_status(CUTESPMM_ENOMEM, "host allocation failed");
    }
    FILE *f = std::fopen(path, "wb");
    if (!f) return fail_status(CUTESPMM_EIO, std::string("cannot write ") + path);
    Writer w{f};
    w.bytes(kMagic, sizeof(kMagic));
    w.pod(kVersion);
    w.pod(kOrderTag);
    w.pod(h.M); w.pod(h.K); w.pod(h.nnz);
    w.pod(h.opts);
    w.pod((uint32_t)(h.device_built ? 1 : 0));
    w.pod((uint32_t)0);
    w.pod(h.num_bricks); w.pod(h.brick_panels); w.pod(h.brick_slots); w.pod(h.slab_steps); w.pod(h.slab_panels);
    for_each_array(h, [&](uint32_t id, auto &v) { w.section(id, v); });
    const uint64_t sum = w.hash;
    w.pod((uint32_t)0);
    w.pod((uint32_t)0);
    w.pod(sum);
    const bool ok = w.ok;
    if (std::fclose(f) != 0 || !ok) return fail_status(CUTESPMM_EIO, std::string("short write to ") + path);
    return CUTESPMM_OK;
}

int cutespmm_plan_load(cutespmm_plan_t **plan, const char *path, int host_only)
{
    if (!plan || !path) return fail_status(CUTESPMM_EINVAL, "null argument");
    *plan = nullptr;
    FILE *f = std::fopen(path, "rb");
    if (!f) return fail_status(CUTESPMM_EIO, std::string("cannot open ") + path);
    cutespmm_plan *p = new (std::nothrow) cutespmm_plan();
    if (!p) {
        std::fclose(f);
        return fail_status(CUTESPMM_ENOMEM, "host allocation failed");
    }
    auto bad = [&](const std::string &what) {
        std::fclose(f);
        delete p;
        return fail_status(CUTESPMM_EIO, std::string(path) + ": " + what);
    };
    HostPlan &h = p->host;
    Reader r{f};
    char magic[16];
    uint32_t version = 0, tag = 0, built = 0, zero = 0;
    r.bytes(magic, sizeof(magic));
    r.pod(version);
    r.pod(tag);
    if (!r.ok || std::memcmp(magic, kMagic, sizeof(kMagic)) != 0) return bad("not a plan file");
    if (tag != kOrderTag) return bad("written on a machine of the other byte order");
    if (version != kVersion) return bad("plan file version " + std::to_string(version) + ", this library reads version " + std::to_string(kVersion));
    r.pod(h.M); r.pod(h.K); r.pod(h.nnz);
    r.pod(h.opts);
    r.pod(built);
    r.pod(zero);
    r.pod(h.num_bricks); r.pod(h.brick_panels); r.pod(h.brick_slots); r.pod(h.slab_steps); r.pod(h.slab_panels);
    if (!r.ok || h.opts.struct_size != sizeof(cutespmm_options_t)) return bad("damaged header");
    h.device_built = built != 0;
    bool fine = true;
    std::string why;
    try {
        for_each_array(h, [&](uint32_t id, auto &v) {
            if (!fine) return;
            uint32_t got_id = 0, esize = 0;
            uint64_t count = 0;
            r.pod(got_id); r.pod(esize); r.pod(count);
            using T = typename std::remove_reference<decltype(v)>::type::value_type;
            if (!r.ok || got_id != id || esize != sizeof(T) || count > (1ull << 40)) {
                fine = false;
                why = "damaged section " + std::to_string(id);
                return;
            }
            v.resize(count);
            r.bytes(v.data(), count * sizeof(T));
            if (!r.ok) {
                fine = false;
                why = "file ends inside section " + std::to_string(id);
            }
        });
    } catch (const std::bad_alloc &) {
        std::fclose(f);
        delete p;
        return fail_status(CUTESPMM_ENOMEM, "host allocation failed while loading the plan");
    }
    if (!fine) return bad(why);
    const uint64_t sum = r.hash;
    uint32_t end_id = 1, end_size = 1;
    uint64_t stored = 0;
    r.pod(end_id); r.pod(end_size); r.pod(stored);
    if (!r.ok || end_id != 0 || stored != sum) return bad("checksum mismatch");
    std::fclose(f);
    // consistency of what the kernels will index with
    if (h.row_ptr.size() != h.M + 1 || h.pairs.size() != h.nnz || (h.nnz && h.row_ptr.back() != h.nnz) ||
        (!h.row_map.empty() && h.row_map.size() != h.M) || h.brick_recs.size() != h.brick_slots * kBrickRecWords ||
        h.brick_cols.size() != h.brick_slots * kBrickCols || h.panel_first_brick.size() != h.brick_panels ||
        h.panel_last_brick.size() != h.brick_panels) {
        delete p;
        return fail_status(CUTESPMM_EIO, std::string(path) + ": inconsistent plan");
    }
    if (!host_only) {
        const int st = cutespmm_internal_upload_plan(p);
        if (st != CUTESPMM_OK) {
            delete p;
            return st;
        }
    }
    *plan = p;
    return CUTESPMM_OK;
}

}  // extern "C"
