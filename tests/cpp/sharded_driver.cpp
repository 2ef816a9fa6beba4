// One process, one host thread per GPU: the shape of a C++ host that scales the reference's driver loop
// (run.cu:8-72) past one device.  The matrix (a seeded random graph with a few hub rows) is cut into
// nnz-balanced row ranges with cutespmm_partition_rows; every thread selects its device, creates a plan
// over its rows and runs the product three ways through the C ABI:
//   1. cutespmm_spmm_sharded, B on rank 0 only            (broadcast over NVLink, then the product)
//   2. cutespmm_spmm_sharded, B row-sharded in place      (all-gather, then the product)
//   3. cutespmm_spmm_sharded_host, host slices in, host C out
// and every result is compared with the CPU oracle on that rank's rows.  All allocation and the first launch of
// every kernel happen before the first collective (see cutespmm_plan_reserve_host_staging in cutespmm.h).
//
//   sharded_driver [ngpus]     prints "rank r mode m relFro=e" lines; exit 0 = all passed,
//                              exit 77 = fewer than two GPUs visible (nothing to test)
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "cutespmm.h"

extern "C" {
void oracle_spmm_csr(const uint64_t *rowPtr, const uint32_t *cols, const float *vals, const float *B, float *C, uint64_t M, uint64_t K,
                     uint32_t N, uint64_t ldb, uint64_t ldc);
double oracle_rel_fro(const float *C_ref, const float *C_test, uint64_t count);
}

static uint32_t lcg(uint32_t &s) { return s = s * 1664525u + 1013904223u; }

#define CK(call)                                                                                       \
    do {                                                                                               \
        int st_ = (call);                                                                              \
        if (st_ != 0) {                                                                                \
            std::fprintf(stderr, "rank %d: %s failed: %s\n", rank, #call, cutespmm_last_error());      \
            failures.fetch_add(1);                                                                     \
            return;                                                                                    \
        }                                                                                              \
    } while (0)
#define CU(call)                                                                                       \
    do {                                                                                               \
        cudaError_t e_ = (call);                                                                       \
        if (e_ != cudaSuccess) {                                                                       \
            std::fprintf(stderr, "rank %d: %s failed: %s\n", rank, #call, cudaGetErrorString(e_));     \
            failures.fetch_add(1);                                                                     \
            return;                                                                                    \
        }                                                                                              \
    } while (0)

int main(int argc, char **argv)
{
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess) ndev = 0;
    int want = argc > 1 ? std::atoi(argv[1]) : ndev;
    if (want > ndev) want = ndev;
    if (want < 2) {
        std::printf("SKIP: %d GPU(s) visible, the sharded path needs two\n", ndev);
        return 77;
    }
    const int R = want;
    // ---- the matrix: M x K, ~12 nonzeros per row, every 997th row a hub of 3000 nonzeros ----
    const uint64_t M = 40000, K = 30000;
    const uint32_t N = 128;
    std::vector<uint64_t> rp(M + 1, 0);
    std::vector<uint32_t> cols;
    std::vector<float> vals;
    uint32_t seed = 2024u;
    for (uint64_t r = 0; r < M; ++r) {
        const uint32_t len = (r % 997 == 5) ? 3000u : 4u + lcg(seed) % 17u;
        std::vector<uint32_t> c(len);
        for (auto &x : c) x = lcg(seed) % K;
        std::sort(c.begin(), c.end());
        c.erase(std::unique(c.begin(), c.end()), c.end());
        for (uint32_t x : c) {
            cols.push_back(x);
            vals.push_back((float)(lcg(seed) >> 8) / (float)(1u << 23) - 1.0f);
        }
        rp[r + 1] = cols.size();
    }
    std::vector<float> B((size_t)K * N);
    for (auto &x : B) x = (float)(lcg(seed) >> 8) / (float)(1u << 23) - 1.0f;
    std::vector<uint64_t> bounds(R + 1), bb(R + 1);
    if (cutespmm_partition_rows(M, rp.data(), R, 16, 2, bounds.data()) != 0) {
        std::fprintf(stderr, "partition failed: %s\n", cutespmm_last_error());
        return 1;
    }
    for (int r = 0; r <= R; ++r) bb[r] = std::min<uint64_t>(K, (uint64_t)r * ((K + R - 1) / R));  // equal slices of B
    std::vector<cutespmm_comm_t *> comms(R, nullptr);
    if (cutespmm_comm_create_all(comms.data(), R, nullptr) != 0) {
        std::fprintf(stderr, "communicator: %s\n", cutespmm_last_error());
        return 1;
    }
    std::atomic<int> failures{0}, arrived{0};
    // Host-side gate in front of every collective: a rank enters a collective only after every rank has come this
    // far without an error, so a failure on one rank ends the run instead of leaving the others waiting on the GPU.
    auto gate = [&](int phase) {
        arrived.fetch_add(1);
        while (arrived.load() < R * phase && failures.load() == 0) std::this_thread::yield();
        return failures.load() == 0;
    };
    auto worker = [&](int rank) {
        CU(cudaSetDevice(rank));
        const uint64_t r0 = bounds[rank], r1 = bounds[rank + 1], m = r1 - r0;
        std::vector<uint64_t> my_rp(m + 1);
        for (uint64_t r = 0; r <= m; ++r) my_rp[r] = rp[r0 + r] - rp[r0];
        const uint32_t *my_cols = cols.data() + rp[r0];
        const float *my_vals = vals.data() + rp[r0];
        cutespmm_plan_t *plan = nullptr;
        CK(cutespmm_plan_create(&plan, m, K, my_rp.data(), my_cols, my_vals, nullptr));
        std::vector<float> ref(m * N), got(m * N);
        oracle_spmm_csr(my_rp.data(), my_cols, my_vals, B.data(), ref.data(), m, K, N, N, N);
        cudaStream_t s;
        CU(cudaStreamCreate(&s));
        float *dB, *dC;
        CU(cudaMalloc(&dB, (size_t)K * N * sizeof(float)));
        CU(cudaMalloc(&dC, std::max<size_t>(m, 1) * N * sizeof(float)));
        auto check = [&](const char *mode, const float *c) {
            const double fro = m ? oracle_rel_fro(ref.data(), c, m * N) : 0.0;
            std::printf("rank %d rows [%llu, %llu) mode %s relFro=%.3e\n", rank, (unsigned long long)r0, (unsigned long long)r1, mode, fro);
            if (!(fro <= 1e-3)) failures.fetch_add(1);
        };
        // Before the first collective: everything that allocates or loads code on this device -- the staging of the
        // host-buffer call, and one local product so that the kernels are resident.  A cudaMalloc or a first launch
        // synchronises with all devices of the process and must not meet another thread's collective in flight.
        CK(cutespmm_plan_reserve_host_staging(plan, N, 1));
        CU(cudaMemsetAsync(dB, 0, (size_t)K * N * sizeof(float), s));
        CK(cutespmm_spmm(plan, dB, N, dC, N, N, s));
        CU(cudaStreamSynchronize(s));
        // 1. B on rank 0 only
        CU(cudaMemsetAsync(dB, 0xff, (size_t)K * N * sizeof(float), s));
        if (rank == 0) CU(cudaMemcpyAsync(dB, B.data(), (size_t)K * N * sizeof(float), cudaMemcpyHostToDevice, s));
        CU(cudaMemsetAsync(dC, 0xff, std::max<size_t>(m, 1) * N * sizeof(float), s));
        CU(cudaStreamSynchronize(s));
        if (!gate(1)) return;
        CK(cutespmm_spmm_sharded(plan, comms[rank], CUTESPMM_B_FROM_ROOT, 0, dB, N, nullptr, dC, N, N, s));
        CU(cudaMemcpyAsync(got.data(), dC, m * N * sizeof(float), cudaMemcpyDeviceToHost, s));
        CU(cudaStreamSynchronize(s));
        check("from_root", got.data());
        // 2. B row-sharded in place
        CU(cudaMemsetAsync(dB, 0xff, (size_t)K * N * sizeof(float), s));
        CU(cudaMemcpyAsync(dB + bb[rank] * N, B.data() + bb[rank] * N, (bb[rank + 1] - bb[rank]) * N * sizeof(float), cudaMemcpyHostToDevice, s));
        CU(cudaMemsetAsync(dC, 0xff, std::max<size_t>(m, 1) * N * sizeof(float), s));
        CU(cudaStreamSynchronize(s));
        if (!gate(2)) return;
        CK(cutespmm_spmm_sharded(plan, comms[rank], CUTESPMM_B_ROW_SHARDED, 0, dB, N, bb.data(), dC, N, N, s));
        CU(cudaMemcpyAsync(got.data(), dC, m * N * sizeof(float), cudaMemcpyDeviceToHost, s));
        CU(cudaStreamSynchronize(s));
        check("row_sharded", got.data());
        // 3. host slices in, host rows of C out
        std::fill(got.begin(), got.end(), -12345.0f);
        float kms = 0.f, xms = 0.f;
        if (!gate(3)) return;
        CK(cutespmm_spmm_sharded_host(plan, comms[rank], B.data() + bb[rank] * N, N, bb.data(), got.data(), N, N, s, &kms, &xms));
        check("host", got.data());
        uint32_t status = 0;
        CK(cutespmm_plan_device_status(plan, &status));
        if (status) failures.fetch_add(1);
        cudaFree(dB);
        cudaFree(dC);
        cudaStreamDestroy(s);
        cutespmm_plan_destroy(plan);
    };
    std::vector<std::thread> threads;
    for (int r = 0; r < R; ++r) threads.emplace_back(worker, r);
    for (auto &t : threads) t.join();
    for (auto *c : comms) cutespmm_comm_destroy(c);
    std::printf("%s (%d ranks)\n", failures.load() ? "FAILED" : "PASSED", R);
    return failures.load() ? 1 : 0;
}
