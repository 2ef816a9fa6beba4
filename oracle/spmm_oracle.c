/*
 * CPU oracle for the sparse x dense product  C[M x N] = A[M x K] * B[K x N].
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing that ships may call into this file: it is
 * the checker used by the test-suite, by the smoke check and by the
 * "cpu_baseline" / "--impl reference" legs of the benchmark driver.
 *
 * Every function restates one routine of the reference project
 * (aFatCa/cuTeSpMM_AE); the file:line it follows is given beside it.  The
 * restatement is pinned: tests/test_oracle.py compares it bit-for-bit with the
 * reference's own routines compiled from the reference sources (oracle/_ref,
 * built by oracle/Makefile) and with golden vectors those routines produced
 * (tests/golden/).
 *
 * Floating-point contract: one fp32 multiply followed by one fp32 add per
 * nonzero and output column, in the order the nonzeros are stored.  The build
 * recipe passes -ffp-contract=off so that the compiler can not fuse the two
 * into an FMA; this is what the reference gets from "nvcc -O2" host code on
 * x86-64 (no -mfma), and oracle/_ref confirms it bit-for-bit.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Thread count of the OpenMP loops below (a launcher may have exported
 * OMP_NUM_THREADS=1 for its children; a timed CPU baseline states its own). */
void oracle_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0)
        omp_set_num_threads(n);
#else
    (void)n;
#endif
}
int oracle_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* inc.h:71-83  (spmm_coo).  The reference opens an OpenMP region over the N
 * columns for every nonzero; the arithmetic per output element is a plain
 * in-order accumulation over the nonzeros, which is what this loop does. */
void oracle_spmm_coo(const uint32_t *rows, const uint32_t *cols,
                     const float *vals, const float *B, float *C,
                     uint32_t M, uint32_t K, uint32_t N, uint64_t nnz)
{
    (void)K;
    memset(C, 0, (size_t)M * N * sizeof(float));
    for (uint64_t i = 0; i < nnz; ++i) {
        const float v = vals[i];
        const float *b = B + (size_t)cols[i] * N;
        float *c = C + (size_t)rows[i] * N;
        for (uint32_t j = 0; j < N; ++j)
            c[j] += v * b[j];
    }
}

/* Same arithmetic as oracle_spmm_coo for a row-sorted COO (= CSR): every
 * output element accumulates its row's nonzeros in storage order, so the
 * result is bit-identical to inc.h:71-83 on the expanded COO.  Rows are
 * independent, which lets OpenMP split them (static schedule). */
void oracle_spmm_csr(const uint64_t *rowPtr, const uint32_t *cols,
                     const float *vals, const float *B, float *C,
                     uint64_t M, uint64_t K, uint32_t N,
                     uint64_t ldb, uint64_t ldc)
{
    (void)K;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)M; ++r) {
        float *c = C + (size_t)r * ldc;
        for (uint32_t j = 0; j < N; ++j)
            c[j] = 0.0f;
        for (uint64_t i = rowPtr[r]; i < rowPtr[r + 1]; ++i) {
            const float v = vals[i];
            const float *b = B + (size_t)cols[i] * ldb;
            for (uint32_t j = 0; j < N; ++j)
                c[j] += v * b[j];
        }
    }
}

/* Rows listed in `which` only (used to check a sample of a matrix whose full
 * product is too slow for the CPU).  Output row i of C holds row which[i]. */
void oracle_spmm_csr_rows(const uint64_t *rowPtr, const uint32_t *cols,
                          const float *vals, const float *B, float *C,
                          const uint64_t *which, uint64_t nwhich, uint32_t N,
                          uint64_t ldb)
{
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t w = 0; w < (int64_t)nwhich; ++w) {
        const uint64_t r = which[w];
        float *c = C + (size_t)w * N;
        for (uint32_t j = 0; j < N; ++j)
            c[j] = 0.0f;
        for (uint64_t i = rowPtr[r]; i < rowPtr[r + 1]; ++i) {
            const float v = vals[i];
            const float *b = B + (size_t)cols[i] * ldb;
            for (uint32_t j = 0; j < N; ++j)
                c[j] += v * b[j];
        }
    }
}

/* inc.h:84-110  (check_gemm_correctness_coo): the largest element-wise
 * relative difference |C - C_host| / |C| over the entries where C != 0.
 * The reference indexes with a 32-bit counter; so does this (count <= 2^32-1). */
float oracle_max_rel_err(const float *C, const float *C_host, uint32_t M,
                         uint32_t N)
{
    float diff = 0.0f;
    const uint32_t count = M * N;
    for (uint32_t i = 0; i < count; ++i) {
        if (C[i] == 0.0f)
            continue;
        const float d = fabsf(C[i] - C_host[i]) / fabsf(C[i]);
        if (d > diff)
            diff = d;
    }
    return diff;
}

/* The acceptance metric of this project: ||C_test - C_ref||_F / ||C_ref||_F,
 * accumulated in double.  (No counterpart in the reference, which computes
 * the metric above and discards it, run.cu:62-63.) */
double oracle_rel_fro(const float *C_ref, const float *C_test, uint64_t count)
{
    double num = 0.0, den = 0.0;
#pragma omp parallel for reduction(+ : num, den) schedule(static)
    for (int64_t i = 0; i < (int64_t)count; ++i) {
        const double d = (double)C_test[i] - (double)C_ref[i];
        num += d * d;
        den += (double)C_ref[i] * (double)C_ref[i];
    }
    if (den == 0.0)
        return num == 0.0 ? 0.0 : INFINITY;
    return sqrt(num / den);
}

/* SDDMM over a CSR pattern: out[j] = (vals ? vals[j] : 1) * sum_n X[row(j)][n] * Y[cols[j]][n], one fp32 multiply
 * and one fp32 add per term, in column order n = 0 .. N-1.  The checker of cutespmm_sddmm.  The reference's own
 * kernels have no such operator; the definition is the one of the TC-GNN baseline that travels with it
 * (TC-GNN_ATC23/TCGNN_conv/TCGNN_kernel.cu:582, sddmm_forward_cuda_kernel: the dot product of the two
 * endpoints' feature rows per edge). */
void oracle_sddmm_csr(const uint64_t *rowPtr, const uint32_t *cols, const float *vals, const float *X, const float *Y,
                      float *out, uint64_t M, uint32_t N, uint64_t ldx, uint64_t ldy)
{
#pragma omp parallel for schedule(dynamic, 256)
    for (int64_t r = 0; r < (int64_t)M; ++r) {
        const float *x = X + (size_t)r * ldx;
        for (uint64_t j = rowPtr[r]; j < rowPtr[r + 1]; ++j) {
            const float *y = Y + (size_t)cols[j] * ldy;
            float s = 0.0f;
            for (uint32_t n = 0; n < N; ++n)
                s += x[n] * y[n];
            out[j] = vals ? vals[j] * s : s;
        }
    }
}
