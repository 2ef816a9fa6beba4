// NVTX3 ranges around the phases a profiler timeline should show (plan creation, the exchange of B, the
// product), where the reference marks its preprocessing and kernel phases (run.cu:31-35,52).  NVTX3 is
// header-only and costs a predicted branch when no tool is attached; without the header the ranges
// compile to nothing.
#pragma once

#if defined(__has_include)
#if __has_include(<nvtx3/nvToolsExt.h>)
#include <nvtx3/nvToolsExt.h>
#define CUTESPMM_HAVE_NVTX 1
#endif
#endif

namespace cutespmm {

struct NvtxRange {
#ifdef CUTESPMM_HAVE_NVTX
    explicit NvtxRange(const char *name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
#else
    explicit NvtxRange(const char *) {}
#endif
    NvtxRange(const NvtxRange &) = delete;
    NvtxRange &operator=(const NvtxRange &) = delete;
};

}  // namespace cutespmm
