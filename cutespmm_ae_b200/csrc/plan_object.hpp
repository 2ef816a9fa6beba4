// The plan object behind the opaque cutespmm_plan_t handle: the host-side description, the device arrays it
// owns and the streams / events / staging buffers of the host-buffer calls.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "plan.hpp"

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

    ~cutespmm_plan()
    {
        if (!on_device) return;
        int cur = -1;
        cudaGetDevice(&cur);
        if (cur != device) cudaSetDevice(device);
        for (void *p : {d_row_ptr, d_pairs, d_tiles, d_chunks, d_long_rows, d_tiles_all, d_chunks_all, d_long_rows_all,
                        d_bcols, d_brecs, d_panel_first, d_panel_last, d_scols, d_srecs, d_srec_off, d_sfirst,
                        d_slast, d_sids, d_row_map, (void *)d_scratch, (void *)d_status, (void *)d_B, (void *)d_C})
            if (p) cudaFree(p);
        for (cudaEvent_t ev : {ev_entry, ev_done})
            if (ev) cudaEventDestroy(ev);
        for (int w = 0; w < kMaxWindows; ++w)
            for (cudaEvent_t ev : {ev_in[w], ev_x0[w], ev_x1[w], ev_k0[w], ev_k1[w]})
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
