/*
 * extern "C" access to the REFERENCE project's own SparseCoo / CSR_Matrix loaders (inc/SparseCoo.hpp,
 * inc/CSR.hpp), compiled from the reference sources where they lie (-I<reference root>/inc), so the
 * loaders in include/cutespmm_loaders.hpp can be pinned against them.  TEST INFRASTRUCTURE ONLY; no
 * reference source is copied.  The reference prints progress to stdout; callers may ignore it.
 */
#include <cstdint>
#include <cstring>
#include <string>
using COMPUTETYPE = float;
#include "CSR.hpp"

extern "C" {
void *ref_csr_from_mtx(const char *path)
{
    SparseCoo<float> coo{std::string(path)};
    return new CSR_Matrix<float>(coo);
}
int ref_csr_nrows(void *h) { return static_cast<CSR_Matrix<float> *>(h)->nrows; }
int ref_csr_ncols(void *h) { return static_cast<CSR_Matrix<float> *>(h)->ncols; }
int ref_csr_nnz(void *h) { return static_cast<CSR_Matrix<float> *>(h)->nnz; }
void ref_csr_copy(void *h, int *rowPtr, int *cols, float *vals)
{
    CSR_Matrix<float> *m = static_cast<CSR_Matrix<float> *>(h);
    memcpy(rowPtr, m->rowPtr, sizeof(int) * (m->nrows + 1));
    memcpy(cols, m->cols, sizeof(int) * m->nnz);
    memcpy(vals, m->values, sizeof(float) * m->nnz);
}
}
