// A driver written the way the reference's run.cu is (run.cu:8-72): read a MatrixMarket file,
// preprocess, then for every feature size allocate B and C on the device, construct SPMM_TC, call
// run() and copy C back -- compiled against include/cutespmm_compat.hpp instead of the reference's
// sources.  Unlike run.cu, which computes an error figure and drops it (run.cu:62-63), the result
// is compared with the CPU oracle and the exit code says whether every N passed.
//
//   compat_driver <file.mtx>      prints one line per N: "N=<n> relFro=<e> maxRel=<e>"
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#define TM 16
#define TN 4
#include "cutespmm_compat.hpp"

extern "C" {
void oracle_spmm_coo(const uint32_t *rows, const uint32_t *cols, const float *vals, const float *B, float *C,
                     uint32_t M, uint32_t K, uint32_t N, uint64_t nnz);
float oracle_max_rel_err(const float *C, const float *C_host, uint32_t M, uint32_t N);
double oracle_rel_fro(const float *C_ref, const float *C_test, uint64_t count);
}

inline void chkerr(cudaError_t code, int line)
{
    if (code != cudaSuccess) {
        std::fprintf(stderr, "ERROR!!!:%s at line %d\n", cudaGetErrorString(code), line);
        std::exit(-1);
    }
}

int main(int argc, char *argv[])
{
    if (argc < 2) {
        std::fprintf(stderr, "usage: %s file.mtx\n", argv[0]);
        return 2;
    }
    MTX_READER *mtxReader = new MTX_READER(std::string(argv[1]));
    unsigned int M = mtxReader->M, K = mtxReader->K, nnz = mtxReader->nnz;
    unsigned int feature_size_list[3] = {32, 128, 512};
    const unsigned int MAX_N = 512;
    HRPB hrpb(M, K, mtxReader->rowPtr, mtxReader->cols, mtxReader->vals);
    std::vector<float> c_host((size_t)M * MAX_N), c_ref((size_t)M * MAX_N), b((size_t)K * MAX_N);
    unsigned int seed = 12345u;
    for (size_t i = 0; i < b.size(); ++i) {
        seed = seed * 1664525u + 1013904223u;
        b[i] = (float)(seed >> 8) / (float)(1u << 24);  // [0, 1) like rand()/RAND_MAX in run.cu:26, but seeded
    }
    std::vector<uint32_t> coo_rows(nnz);
    for (unsigned int r = 0; r < M; ++r)
        for (unsigned int j = mtxReader->rowPtr[r]; j < mtxReader->rowPtr[r + 1]; ++j) coo_rows[j] = r;
    int failures = 0;
    for (int n = 0; n < 3; ++n) {
        unsigned int N = feature_size_list[n];
        float *b_device, *c_device;
        chkerr(cudaMalloc(&b_device, (size_t)K * N * sizeof(float)), __LINE__);
        chkerr(cudaMemcpy(b_device, b.data(), (size_t)K * N * sizeof(float), cudaMemcpyHostToDevice), __LINE__);
        chkerr(cudaMalloc(&c_device, (size_t)M * N * sizeof(float)), __LINE__);
        chkerr(cudaMemset(c_device, 0xff, (size_t)M * N * sizeof(float)), __LINE__);  // NaNs: every element must be written

        SPMM_TC spmmTc(M, K, N, hrpb.blockedRowPtr);
        unsigned int *data = hrpb.blocksDevice;
        unsigned long long int *sizePtr = hrpb.sizePtrDevice;
        unsigned int *active_cols_vec = hrpb.activeColsDevice;
        spmmTc.run(data, b_device, c_device, active_cols_vec, sizePtr);
        chkerr(cudaMemcpy(c_host.data(), c_device, (size_t)M * N * sizeof(float), cudaMemcpyDeviceToHost), __LINE__);
        chkerr(cudaFree(c_device), __LINE__);
        chkerr(cudaFree(b_device), __LINE__);
        chkerr(cudaDeviceSynchronize(), __LINE__);

        oracle_spmm_coo(coo_rows.data(), mtxReader->cols, mtxReader->vals, b.data(), c_ref.data(), M, K, N, nnz);
        const double fro = oracle_rel_fro(c_ref.data(), c_host.data(), (uint64_t)M * N);
        const float mx = oracle_max_rel_err(c_ref.data(), c_host.data(), M, N);
        std::printf("N=%u relFro=%.3e maxRel=%.3e\n", N, fro, mx);
        if (!(fro <= 1e-3)) ++failures;  // TF32 multiply, fp32 accumulate: the stated bound
    }
    delete mtxReader;
    return failures ? 1 : 0;
}
