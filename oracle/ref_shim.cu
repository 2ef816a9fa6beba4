/*
 * Thin extern "C" wrapper that exposes the REFERENCE project's own host
 * routines as a shared library, so the CPU oracle (spmm_oracle.c) and the
 * host-side format code of this project can be pinned against them.
 *
 * TEST INFRASTRUCTURE ONLY.  No reference source is copied: this file
 * textually includes the reference's data.cu (which pulls in IO.cu and inc.h)
 * from wherever the reference tree is mounted (-I<reference root> on the
 * command line, see oracle/Makefile).  The output goes to oracle/_ref/ and is
 * not part of the product.
 *
 * The reference's preprocessing uploads its arrays with cudaMalloc/cudaMemcpy
 * (data.cu:327-334); the two macros below redirect those calls to host
 * malloc/memcpy so the routine runs without a GPU and its "device" arrays can
 * be read back here.
 */
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <cuda_runtime.h>

template <class T> static cudaError_t host_malloc_(T **p, size_t n)
{
    *p = static_cast<T *>(malloc(n ? n : 1));
    return *p ? cudaSuccess : cudaErrorMemoryAllocation;
}
static cudaError_t host_memcpy_(void *d, const void *s, size_t n, cudaMemcpyKind)
{
    memcpy(d, s, n);
    return cudaSuccess;
}
#define cudaMalloc host_malloc_
#define cudaMemcpy host_memcpy_

#include "data.cu" /* reference: HRPB, MTX_READER (IO.cu), spmm_coo (inc.h) */

#include <omp.h>

extern "C" {

/* thread count of the reference's OpenMP regions, set by the caller instead of inherited */
void ref_set_threads(int n)
{
    if (n > 0) omp_set_num_threads(n);
}
int ref_max_threads(void) { return omp_get_max_threads(); }

/* inc.h:71-83 verbatim */
void ref_spmm_coo(unsigned int *rows, unsigned int *cols, float *vals, float *B, float *C,
                  uint32_t M, uint32_t K, uint32_t N, unsigned int nnz)
{
    spmm_coo(rows, cols, vals, B, C, M, K, N, nnz);
}

/* inc.h:84-110 verbatim */
float ref_check_gemm_correctness_coo(float *C, float *C_host, uint32_t M, uint32_t N)
{
    return check_gemm_correctness_coo(C, C_host, M, N);
}

/* IO.cu:10-87: returns an opaque reader; fields are fetched with the getters. */
void *ref_mtx_open(const char *path) { return new MTX_READER(std::string(path)); }
unsigned ref_mtx_M(void *h) { return static_cast<MTX_READER *>(h)->M; }
unsigned ref_mtx_K(void *h) { return static_cast<MTX_READER *>(h)->K; }
unsigned ref_mtx_nnz(void *h) { return static_cast<MTX_READER *>(h)->nnz; }
void ref_mtx_copy(void *h, unsigned *rowPtr, unsigned *cols, float *vals)
{
    MTX_READER *r = static_cast<MTX_READER *>(h);
    memcpy(rowPtr, r->rowPtr, (size_t)(r->M + 1) * sizeof(unsigned));
    memcpy(cols, r->cols, (size_t)r->rowPtr[r->M] * sizeof(unsigned));
    memcpy(vals, r->vals, (size_t)r->rowPtr[r->M] * sizeof(float));
}

/* data.cu:80-335: row panels -> active-column blocks.  Only the quantities
 * that are independent of the packed value stream are exposed. */
void *ref_hrpb_build(unsigned M, unsigned K, unsigned *rowPtr, unsigned *cols, float *vals)
{
    omp_set_dynamic(0);
    return new HRPB(M, K, rowPtr, cols, vals);
}
unsigned ref_hrpb_num_panels(void *h) { return static_cast<HRPB *>(h)->numRowPanels; }
unsigned ref_hrpb_num_blocks(void *h)
{
    HRPB *p = static_cast<HRPB *>(h);
    return p->blockedRowPtr[p->numRowPanels];
}
void ref_hrpb_copy(void *h, unsigned *blockedRowPtr, unsigned *activeCols)
{
    HRPB *p = static_cast<HRPB *>(h);
    memcpy(blockedRowPtr, p->blockedRowPtr, (size_t)(p->numRowPanels + 1) * sizeof(unsigned));
    memcpy(activeCols, p->activeCols, (size_t)p->blockedRowPtr[p->numRowPanels] * TK * sizeof(unsigned));
}
unsigned long long ref_hrpb_stream_words(void *h)
{
    HRPB *p = static_cast<HRPB *>(h);
    return p->sizePtr[p->blockedRowPtr[p->numRowPanels]];
}

} /* extern "C" */
