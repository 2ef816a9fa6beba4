/*
 * extern "C" wrapper around the REFERENCE project's own GPU path -- its host preprocessing (HRPB, data.cu),
 * its work-list builder and launcher (SPMM_TC, spmm.cu) and its kernel SpMM<NUM_WARPS, ILP_LEVEL>
 * (kernel.cu:119-288) -- compiled for sm_100a from the reference sources where they lie (-I<reference root>,
 * see oracle/Makefile), so the benchmark can put "the reference's kernel on the same GPU" beside this
 * project's numbers.
 *
 * TEST / MEASUREMENT INFRASTRUCTURE ONLY.  No reference source is copied; the output goes to oracle/_ref/ and is
 * not part of the product.  The call follows the reference's driver loop (run.cu:38-53): B and C on the
 * device, C zeroed (the kernel relies on it for empty panels and adds into split panels), one launch.
 * Its occupancy table has no entry for a 148-SM part (spmm.cu:290-690); the build selects the table of
 * machine 0 (-DMachine=0, as compile.sh does), i.e. the reference runs with the work list it would cut for
 * a 108-SM GPU.  The reference addresses B and C with 32-bit element offsets and allocates
 * (M/16)*(K/16) offsets on the host (data.cu:91): callers keep to matrices it can hold.
 */
#include <cstdint>
#include <cstring>

#include "spmm.cu" /* reference: SPMM_TC, SpMM kernel, HRPB, MTX_READER, inc.h */

extern "C" {

/* Preprocesses (host, timed into *prep_ms), uploads, runs once cold (*cold_ms: the first launch, library
 * start-up included), `iters` times back to back (*warm_ms: their mean; L2 as the previous launch left it)
 * and `iters` times with the L2 cache flushed before each launch by a 256 MiB write (*flushed_ms: the
 * protocol of this project's benchmark).  Each launch runs alone between CUDA events after a cudaMemset
 * of C that is not timed.  C_host receives the last result.  Rows must have ascending unique columns and
 * M, K be multiples of 16 (data.cu:80-93).  Returns 0, or a CUDA error code. */
int ref_gpu_spmm(unsigned M, unsigned K, unsigned N, unsigned *rowPtr, unsigned *cols, float *vals, const float *B_host, float *C_host,
                 int iters, float *prep_ms, float *cold_ms, float *warm_ms, float *flushed_ms)
{
    cudaEvent_t e0, e1;
    cudaError_t err;
    if ((err = cudaEventCreate(&e0)) != cudaSuccess || (err = cudaEventCreate(&e1)) != cudaSuccess) return (int)err;
    const double t0 = omp_get_wtime();
    HRPB hrpb(M, K, rowPtr, cols, vals);
    SPMM_TC spmmTc(M, K, N, hrpb.blockedRowPtr);
    *prep_ms = (float)((omp_get_wtime() - t0) * 1e3);
    float *b_device = nullptr, *c_device = nullptr;
    if ((err = cudaMalloc(&b_device, (size_t)K * N * sizeof(float))) != cudaSuccess) return (int)err;
    if ((err = cudaMalloc(&c_device, (size_t)M * N * sizeof(float))) != cudaSuccess) return (int)err;
    if ((err = cudaMemcpy(b_device, B_host, (size_t)K * N * sizeof(float), cudaMemcpyHostToDevice)) != cudaSuccess) return (int)err;
    const size_t flush_bytes = 256u << 20;
    void *flush = nullptr;
    if ((err = cudaMalloc(&flush, flush_bytes)) != cudaSuccess) return (int)err;
    float total = 0.f, total_flushed = 0.f;
    *cold_ms = *warm_ms = *flushed_ms = 0.f;
    for (int it = 0; it <= 2 * iters; ++it) {
        if ((err = cudaMemset(c_device, 0, (size_t)M * N * sizeof(float))) != cudaSuccess) return (int)err;
        if (it > iters && (err = cudaMemset(flush, 1, flush_bytes)) != cudaSuccess) return (int)err;
        cudaEventRecord(e0);
        spmmTc.run(hrpb.blocksDevice, b_device, c_device, hrpb.activeColsDevice, hrpb.sizePtrDevice);
        cudaEventRecord(e1);
        if ((err = cudaEventSynchronize(e1)) != cudaSuccess) return (int)err;
        if ((err = cudaGetLastError()) != cudaSuccess) return (int)err;
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (it == 0) *cold_ms = ms;
        else if (it <= iters) total += ms;
        else total_flushed += ms;
    }
    if (iters > 0) {
        *warm_ms = total / iters;
        *flushed_ms = total_flushed / iters;
    }
    cudaFree(flush);
    err = cudaMemcpy(C_host, c_device, (size_t)M * N * sizeof(float), cudaMemcpyDeviceToHost);
    cudaFree(b_device);
    cudaFree(c_device);
    hrpb.freeDevice();
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return (int)err;
}

}
