// The plan object behind the opaque cutespmm_plan_t handle: the host-side description, the device arrays it
// owns and the streams / events / staging buffers of the host-buffer calls.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <string>
#include <vector>

#include "plan.hpp"

// A contiguous range of the plan's work items (tiles and chunks of the row kernel -- of its own list and
// of the list over every row -- and panels of the brick kernel): what one launch covers when a product is issued in
// blocks of rows.
struct cutespmm_item_range {
    uint32_t t0 = 0, t1 = 0, c0 = 0, c1 = 0;      // row kernel: tiles, chunks
    uint32_t ta0 = 0, ta1 = 0, ca0 = 0, ca1 = 0;  // the same lists over every row
    uint32_t p0 = 0, p1 = 0;                                        // brick panels (ordinals)
};
// One block of rows of the row-block host-buffer call: rows [row0, row1) of C, computed once rows [0, need) of B are
// on the device.
struct cutespmm_row_block {
    uint32_t row0 = 0, row1 = 0, need = 0;
    cutespmm_item_range items;
};

struct cutespmm_plan {
    cutespmm::HostPlan host;
    bool on_device = false;
    int device = -1;
    int sm_count = 0;
    uint64_t device_bytes = 0;
    // device arrays
    void *d_row_ptr = nullptr, *d_pairs = nullptr, *d_tiles = nullptr, *d_chunks = nullptr, *d_long_rows = nullptr;
    void *d_tiles_all = nullptr, *d_chunks_all = nullptr, *d_long_rows_all = nullptr;
    void *d_bcols = nullptr, *d_brecs = nullptr, *d_panel_first = nullptr, *d_panel_last = nullptr;
    void *d_scols = nullptr, *d_srecs = nullptr, *d_srec_off = nullptr, *d_sfirst = nullptr, *d_slast = nullptr, *d_sids = nullptr;
    void *d_row_map = nullptr;
    void *d_chunk_owner = nullptr, *d_chunk_owner_all = nullptr;  // per scratch slot: its long row
    uint32_t *d_arrivals = nullptr;                               // per long row and column slab: chunks finished
    float *d_scratch = nullptr;
    uint32_t *d_status = nullptr;
    // staging for the host-buffer call
    float *d_B = nullptr, *d_C = nullptr;
    uint64_t staged_B = 0, staged_C = 0;
    // the host-buffer calls pipeline column windows: copy-in, exchange between ranks, product and copy-out each on a
    // stream of their own
    static constexpr int kMaxWindows = 4;
    cudaStream_t s_in = nullptr, s_x = nullptr, s_out = nullptr;
    cudaEvent_t ev_entry = nullptr, ev_done = nullptr;
    cudaEvent_t ev_in[kMaxWindows] = {}, ev_x0[kMaxWindows] = {}, ev_x1[kMaxWindows] = {}, ev_k0[kMaxWindows] = {}, ev_k1[kMaxWindows] = {};

    // the single-GPU host-buffer call in blocks of rows (banded matrices): C rows leave while later rows of B arrive
    static constexpr int kMaxRowBlocks = 16;
    std::vector<cutespmm_row_block> row_blocks;  // cut at the first such call
    bool row_blocks_tried = false;
    uint32_t row_blocks_n = 0;                   // the N they were cut for
    cudaEvent_t rb_in[kMaxRowBlocks] = {}, rb_k0[kMaxRowBlocks] = {}, rb_k1[kMaxRowBlocks] = {};

    ~cutespmm_plan()
    {
        if (!on_device) return;
        int cur = -1;
        cudaGetDevice(&cur);
        if (cur != device) cudaSetDevice(device);
        for (void *p : {d_row_ptr, d_pairs, d_tiles, d_chunks, d_long_rows, d_tiles_all, d_chunks_all, d_long_rows_all,
                        d_bcols, d_brecs, d_panel_first, d_panel_last, d_scols, d_srecs, d_srec_off, d_sfirst,
                        d_slast, d_sids, d_row_map, d_chunk_owner, d_chunk_owner_all, (void *)d_arrivals, (void *)d_scratch, (void *)d_status, (void *)d_B, (void *)d_C})
            if (p) cudaFree(p);
        for (cudaEvent_t ev : {ev_entry, ev_done})
            if (ev) cudaEventDestroy(ev);
        for (int w = 0; w < kMaxWindows; ++w)
            for (cudaEvent_t ev : {ev_in[w], ev_x0[w], ev_x1[w], ev_k0[w], ev_k1[w]})
                if (ev) cudaEventDestroy(ev);
        for (int i = 0; i < kMaxRowBlocks; ++i)
            for (cudaEvent_t ev : {rb_in[i], rb_k0[i], rb_k1[i]})
                if (ev) cudaEventDestroy(ev);
        for (cudaStream_t st : {s_in, s_x, s_out})
            if (st) cudaStreamDestroy(st);
        if (cur != device && cur >= 0) cudaSetDevice(cur);
    }
};


namespace cutespmm {
// shared by the translation units that implement the C ABI
int fail_status(int status, const std::string &msg);          // records the message, returns status
int fail_cuda_status(cudaError_t e, const char *what);        // same for a CUDA error
}  // namespace cutespmm

// cutespmm_spmm restricted to a range of work items (nullptr: everything).  capi.cu
int cutespmm_internal_spmm_range(const cutespmm_plan *p, const float *B, uint64_t ldb, float *C, uint64_t ldc, uint32_t N, void *stream,
                                 const cutespmm_item_range *range);
