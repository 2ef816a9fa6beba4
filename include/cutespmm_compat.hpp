// Source-compatible stand-ins for the three classes a driver of the reference project uses
// (aFatCa/cuTeSpMM_AE run.cu:11-50): MTX_READER (IO.cu:1-88), HRPB (data.cu:54-340) and SPMM_TC
// (spmm.cu:260-840), implemented over the C ABI of libcutespmm.  A program written against the
// reference keeps its code:
//
//     MTX_READER reader(path);
//     HRPB hrpb(reader.M, reader.K, reader.rowPtr, reader.cols, reader.vals);
//     SPMM_TC spmm(M, K, N, hrpb.blockedRowPtr);
//     spmm.run(hrpb.blocksDevice, b_device, c_device, hrpb.activeColsDevice, hrpb.sizePtrDevice);
//
// Same constructor and run() signatures, same public field names.  What the fields hold differs
// where the reference exposed its internal device format: blocksDevice, activeColsDevice and
// sizePtrDevice are opaque tokens that only SPMM_TC::run understands (they all identify the plan
// that owns the real device arrays); blockedRowPtr, activeCols, numRowPanels keep their meaning.
//
// Error behaviour: the reference prints "ERROR!!!:<text> at line <n>" and calls exit(-1)
// (chkerr, inc.h:61-69).  This header does the same by default; define CUTESPMM_COMPAT_THROW before
// including it to get a std::runtime_error instead.
//
// The tile macros of the reference build line (-DTM=16 -DTK=16 -DTN=4 -DMachine=0, compile.sh:1)
// are accepted and ignored: panel height and brick shape are properties of the library.
#pragma once
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <vector>

#include "cutespmm.h"

namespace cutespmm_compat {
inline void check(int status, int line)
{
    if (status == CUTESPMM_OK) return;
#ifdef CUTESPMM_COMPAT_THROW
    throw std::runtime_error(std::string("libcutespmm: ") + cutespmm_last_error() + " (" +
                             cutespmm_status_string(status) + ")");
#else
    std::fprintf(stderr, "ERROR!!!:%s (%s) at line %d\n", cutespmm_last_error(), cutespmm_status_string(status), line);
    std::exit(-1);
#endif
}
}  // namespace cutespmm_compat

// IO.cu:2-88.  Public fields as in the reference; values are all 1.0, M and K are padded to
// multiples of 16, a symmetric header mirrors the entries.
class MTX_READER {
public:
    unsigned int M = 0;
    unsigned int K = 0;
    unsigned int nnz = 0;
    unsigned int *rowPtr = nullptr;
    unsigned int *cols = nullptr;
    float *vals = nullptr;
    explicit MTX_READER(std::string file_path)
    {
        int st = cutespmm_mtx_open(&mtx_, file_path.c_str(), 1);
        if (st != CUTESPMM_OK) {
            std::fprintf(stderr, "ERROR!!!:cannot read MatrixMarket file %s (%s)\n", file_path.c_str(),
                         cutespmm_status_string(st));
#ifdef CUTESPMM_COMPAT_THROW
            throw std::runtime_error("cannot read " + file_path);
#else
            std::exit(-1);
#endif
        }
        cutespmm_mtx_dims(mtx_, &M, &K, &nnz);
        const uint32_t *rp, *cc;
        const float *vv;
        cutespmm_mtx_arrays(mtx_, &rp, &cc, &vv);
        // the reference hands out mutable arrays it never frees; these live as long as the reader
        rowPtr = const_cast<unsigned int *>(rp);
        cols = const_cast<unsigned int *>(cc);
        vals = const_cast<float *>(vv);
    }
    ~MTX_READER() { cutespmm_mtx_close(mtx_); }
    MTX_READER(const MTX_READER &) = delete;
    MTX_READER &operator=(const MTX_READER &) = delete;

private:
    cutespmm_mtx_t *mtx_ = nullptr;
};

// data.cu:54-340.  Construction preprocesses A and uploads it to the current device.
class HRPB {
public:
    unsigned int *cols;
    unsigned int *rowPtr;
    float *vals;
    unsigned int M;
    unsigned int K;
    unsigned int numRowPanels;
    // the public members of the reference class, in its order (data.cu:62-79), so code that reads them still compiles;
    // members the reference declares but never fills (num_bricks stays 0 there, the float statistics are never assigned)
    // carry this plan's figures instead
    unsigned int *blocksData = nullptr;                // the reference's host copy of its packed stream: not kept here
    unsigned long long int dataStructSize = 0;         // bytes of device memory the plan owns
    unsigned int num_bricks = 0;                       // non-empty 16 x 8 bricks of the panels on the tensor-core kernel
    unsigned int *blocksDevice = nullptr;              // token for SPMM_TC::run
    unsigned int *blockedRowPtr = nullptr;             // host, numRowPanels + 1 entries (data.cu:65)
    unsigned int *blockedRowPtrDevice = nullptr;       // token (the kernels here do not read this view)
    unsigned long long int *sizePtr = nullptr;         // the reference's per-block offsets: records here have a fixed size
    unsigned long long int *sizePtrDevice = nullptr;   // token for SPMM_TC::run
    unsigned int numActiveCols = 0;
    unsigned int *activeCols = nullptr;                // host, blockedRowPtr[numRowPanels] * 16 entries (data.cu:70)
    unsigned int *activeColsDevice = nullptr;          // token for SPMM_TC::run
    float averageNNZcol = 0.f;                         // nonzeros per active column
    unsigned int numNNZ = 0;
    float block_density = 0.f;                         // nonzeros per cell of the 16 x 16 active-column blocks
    unsigned int atomic_blocks = 0;                    // the reference counts split panels it adds with atomics; here: chunks of long rows
    float atomic_ratio = 0.f;                          // ... as a share of the row panels
    float waves = 0.f;                                 // occupancy-table figure of the reference's work list; no such table here
    std::vector<std::vector<unsigned int>> blocks_nnz_counter_vec;  // never filled by the reference either
    cutespmm_plan_t *plan = nullptr;                   // the object behind the tokens

    HRPB(unsigned int M_, unsigned int K_, unsigned int *rowPtr_, unsigned int *cols_, float *vals_,
         const cutespmm_options_t *opts = nullptr)
        : cols(cols_), rowPtr(rowPtr_), vals(vals_), M(M_), K(K_), numRowPanels((M_ + 15) / 16)
    {
        cutespmm_compat::check(cutespmm_plan_create_u32(&plan, M, K, rowPtr, cols, vals, opts), __LINE__);
        cutespmm_plan_info_t info;
        cutespmm_compat::check(cutespmm_plan_info(plan, &info), __LINE__);
        numNNZ = (unsigned int)info.nnz;
        blocked_.resize(info.num_panels + 1);
        active_.resize(info.num_blocks * 16 + 1);
        cutespmm_compat::check(cutespmm_plan_blocked_row_ptr(plan, blocked_.data()), __LINE__);
        cutespmm_compat::check(cutespmm_plan_active_cols(plan, active_.data()), __LINE__);
        blockedRowPtr = blocked_.data();
        activeCols = active_.data();
        numActiveCols = (unsigned int)(info.num_blocks * 16);
        dataStructSize = info.device_bytes;
        num_bricks = (unsigned int)info.num_bricks;
        averageNNZcol = numActiveCols ? (float)numNNZ / (float)numActiveCols : 0.f;
        block_density = info.num_blocks ? (float)numNNZ / (float)(info.num_blocks * 256) : 0.f;
        atomic_blocks = (unsigned int)info.num_chunks;
        atomic_ratio = numRowPanels ? (float)info.num_long_rows / (float)numRowPanels : 0.f;
        blockedRowPtrDevice = reinterpret_cast<unsigned int *>(plan);
        blocksDevice = reinterpret_cast<unsigned int *>(plan);
        activeColsDevice = reinterpret_cast<unsigned int *>(plan);
        sizePtrDevice = reinterpret_cast<unsigned long long int *>(plan);
    }
    // data.cu:336-339 frees two of its four device arrays; this one releases everything the plan owns.
    void freeDevice()
    {
        if (plan) cutespmm_plan_destroy(plan);
        plan = nullptr;
        blocksDevice = activeColsDevice = blockedRowPtrDevice = nullptr;
        sizePtrDevice = nullptr;
    }
    ~HRPB() { freeDevice(); }
    HRPB(const HRPB &) = delete;
    HRPB &operator=(const HRPB &) = delete;

private:
    std::vector<uint32_t> blocked_, active_;
};

// spmm.cu:260-840.  The constructor's work list (partition, spmm.cu:691-822) is part of the plan
// already and does not depend on N, so construction is free; run() launches on the legacy default
// stream like the reference (spmm.cu:171-174) and does not synchronise.
class SPMM_TC {
public:
    unsigned int M;
    unsigned int N;
    unsigned int K;
    unsigned int numRowPanelsSplit = 0;
    SPMM_TC(unsigned int M_, unsigned int K_, unsigned int N_, unsigned int *blockedRowPtr) : M(M_), N(N_), K(K_)
    {
        (void)blockedRowPtr;
    }
    // MatA: HRPB::blocksDevice.  MatB: K x N device, row-major.  MatC: M x N device, row-major; every
    // row is written, a preceding cudaMemset (run.cu:43,49) is harmless and unnecessary.
    void run(unsigned int *MatA, float *MatB, float *MatC, unsigned int *active_cols_vec, unsigned long long int *sizePtr)
    {
        (void)active_cols_vec;
        (void)sizePtr;
        cutespmm_plan_t *plan = reinterpret_cast<cutespmm_plan_t *>(MatA);
        cutespmm_compat::check(cutespmm_spmm(plan, MatB, N, MatC, N, N, nullptr), __LINE__);
    }
};
