// The call shape of the reference's harness (gpu_kernels.cu:1290-1291: SparseCoo<float> coo(path);
// CSR_Matrix<float> csr(coo);) carried through to the GPU: the CSR the loaders produce, with the
// file's own values, becomes a plan (cutespmm_plan_from_csr), the product runs on the device, and
// the result is compared with the CPU oracle on the same CSR.
//
//   loaders_gpu_driver file.mtx [N]     prints "M=<m> K=<k> nnz=<n> N=<N> relFro=<e>"; exit 0 = within 1e-3
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "cutespmm_loaders.hpp"

extern "C" {
void oracle_spmm_csr(const uint64_t *rowPtr, const uint32_t *cols, const float *vals, const float *B, float *C, uint64_t M, uint64_t K,
                     uint32_t N, uint64_t ldb, uint64_t ldc);
double oracle_rel_fro(const float *C_ref, const float *C_test, uint64_t count);
}

int main(int argc, char **argv)
{
    if (argc < 2) return 2;
    const uint32_t N = argc > 2 ? (uint32_t)std::atoi(argv[2]) : 64u;
    SparseCoo<float> coo{std::string(argv[1])};
    CSR_Matrix<float> csr(coo);
    cutespmm_plan_t *plan = nullptr;
    if (cutespmm_plan_from_csr(&plan, csr) != CUTESPMM_OK) {
        std::fprintf(stderr, "plan: %s\n", cutespmm_last_error());
        return 1;
    }
    const uint64_t M = (uint64_t)csr.nrows, K = (uint64_t)csr.ncols;
    std::vector<float> B(K * N), C(M * N), ref(M * N);
    unsigned s = 99u;
    for (auto &x : B) {
        s = s * 1664525u + 1013904223u;
        x = (float)(s >> 8) / (float)(1u << 23) - 1.0f;
    }
    float *dB = nullptr, *dC = nullptr;
    if (cudaMalloc(&dB, B.size() * 4) != cudaSuccess || cudaMalloc(&dC, C.size() * 4) != cudaSuccess) return 1;
    cudaMemcpy(dB, B.data(), B.size() * 4, cudaMemcpyHostToDevice);
    cudaMemset(dC, 0xff, C.size() * 4);  // NaNs: every element must be written
    if (cutespmm_spmm(plan, dB, N, dC, N, N, nullptr) != CUTESPMM_OK) {
        std::fprintf(stderr, "spmm: %s\n", cutespmm_last_error());
        return 1;
    }
    if (cudaMemcpy(C.data(), dC, C.size() * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return 1;
    std::vector<uint64_t> rp(M + 1);
    std::vector<uint32_t> cols(csr.nnz);
    for (uint64_t i = 0; i <= M; ++i) rp[i] = (uint64_t)csr.rowPtr[i];
    for (int i = 0; i < csr.nnz; ++i) cols[i] = (uint32_t)csr.cols[i];
    oracle_spmm_csr(rp.data(), cols.data(), csr.values, B.data(), ref.data(), M, K, N, N, N);
    const double fro = oracle_rel_fro(ref.data(), C.data(), M * N);
    std::printf("M=%llu K=%llu nnz=%d N=%u relFro=%.3e\n", (unsigned long long)M, (unsigned long long)K, csr.nnz, N, fro);
    cudaFree(dB);
    cudaFree(dC);
    cutespmm_plan_destroy(plan);
    return fro <= 1e-3 ? 0 : 1;
}
