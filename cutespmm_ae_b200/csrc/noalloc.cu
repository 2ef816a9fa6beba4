// cutespmm_spmm_csr_noalloc: the product C = A * B for callers that are not allowed to allocate.
//
// Some hosts of this library run where device memory cannot be requested at call time: inside a
// framework that has handed all of HBM to its own pool, inside a real-time loop that forbids calls
// which may synchronise the device, or in a process whose memory budget was fixed at start-up.  Such
// a caller cannot create a plan (plan creation uploads arrays and reserves the partial-sum scratch
// with cudaMalloc).  This entry point takes plain CSR arrays that already sit in device memory and
// computes the product with the row kernel's method -- a warp per row, long rows cut into chunks
// whose partial sums are added in a fixed order -- keeping the partial sums in a scratch array that
// is part of the library image instead of an allocation.
//
// The scratch is the file-scope array g_scratch below (16 MiB).  Every GPU on which the library is
// loaded holds it until the process exits.  All calls on one device share it, and it keeps whatever
// the previous call left there; nothing in it has to start at zero, because every slot a call reads
// was written earlier by the same call.  Two calls that overlap on the same GPU (different streams,
// or different host threads) race on it: order them on one stream or with events.
//
// In host code the name g_scratch is only a stand-in, not a device address.  The address the
// kernels receive comes from cudaGetSymbolAddress, looked up once per device, with that device
// current, by the first call made on it; that first call should be made outside any stream capture.
//
// No counterpart in the reference project.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <mutex>
#include <string>

#include "../../include/cutespmm.h"

namespace cutespmm {
void set_last_error(const std::string &msg);  // capi.cu
}

namespace {

constexpr uint32_t kSplit = CUTESPMM_NOALLOC_SPLIT_NNZ;          // rows longer than this are cut into chunks of this length
constexpr uint64_t kScratchFloats = CUTESPMM_NOALLOC_SCRATCH_BYTES / 4;
constexpr int kWarps = 8;
constexpr int kSlab = 128;                                        // columns one block row covers (4 per lane)
constexpr unsigned kFull = 0xffffffffu;

static __device__ __align__(256) float g_scratch[kScratchFloats];
static __device__ uint32_t g_next_row[CUTESPMM_NOALLOC_MAX_N / kSlab];  // row counters of the rows kernel, one per column slab

// Slot of the chunk that starts at nonzero position `start`.  Chunks of one row start kSplit apart
// and two long rows start more than kSplit apart, so a window of kSplit positions holds at most one
// first chunk and one later chunk: two slots per window are enough and need no counter.
__device__ __forceinline__ uint64_t chunk_slot(uint32_t start, bool first_of_row)
{
    return 2ull * (start / kSplit) + (first_of_row ? 1u : 0u);
}

// Nonzero positions [j0, j1) of row r, forced into [0, nnz] and into order: every position the kernels derive a
// scratch slot or an array index from is then below the `nnz` the host sized its checks with, whatever rowPtr holds.
struct Range {
    uint32_t j0, j1;
};
__device__ __forceinline__ Range row_range(const uint32_t *__restrict__ rowPtr, uint64_t r, uint32_t nnz)
{
    Range g;
    g.j0 = min(__ldg(rowPtr + r), nnz);
    g.j1 = min(max(__ldg(rowPtr + r + 1), g.j0), nnz);
    return g;
}

// acc[i] += sum over nonzeros [j0, j1) of vals[j] * B[cols[j]][n0 + lane + 32 i].  A nonzero whose column is not
// below K is left out (B has no such row); the call cannot report it without reading something back.
__device__ __forceinline__ void accumulate(float (&acc)[4], const uint32_t *__restrict__ cols,
                                           const float *__restrict__ vals, uint32_t j0, uint32_t j1,
                                           const float *__restrict__ B, uint64_t ldb, uint32_t n0, uint32_t N, uint32_t K,
                                           int lane)
{
    constexpr int U = 4;  // nonzeros whose rows of B are in flight together
    for (uint32_t j = j0; j < j1; j += 32) {
        const uint32_t n = min(32u, j1 - j);
        uint32_t c = 0;
        float v = 0.f;
        if ((uint32_t)lane < n) {
            c = __ldg(cols + j + lane);
            v = __ldg(vals + j + lane);
        }
        for (uint32_t k = 0; k < n; k += U) {
            float vk[U], b[U][4];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int src = (int)min(k + u, n - 1);  // positions past the end repeat the last one and add nothing
                const uint32_t ck = __shfl_sync(kFull, c, src);
                vk[u] = __shfl_sync(kFull, v, src);
                const bool use = k + u < n && ck < K;    // uniform across the warp
                if (!use) vk[u] = 0.f;
                const float *row = B + (uint64_t)ck * ldb + n0 + lane;
#pragma unroll
                for (int i = 0; i < 4; ++i) b[u][i] = (use && n0 + lane + 32 * i < N) ? __ldg(row + 32 * i) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[i] = fmaf(vk[u], b[u][i], acc[i]);
        }
    }
}

// Rows of at most kSplit nonzeros: one warp per row, result straight to C.  Warps claim kClaim consecutive rows at a
// time from a counter per column slab (next_row, zeroed by the host before the launch): a fixed stride would hand the
// rows r, r + stride, ... of a power-law graph -- whose long rows sit at indices with few one-bits -- to the same few warps.
constexpr uint32_t kClaim = 4;
__global__ void __launch_bounds__(kWarps * 32) noalloc_rows_kernel(const uint32_t *__restrict__ rowPtr,
                                                                   const uint32_t *__restrict__ cols,
                                                                   const float *__restrict__ vals, uint32_t M,
                                                                   uint32_t K, uint32_t nnz,
                                                                   const float *__restrict__ B, uint64_t ldb,
                                                                   float *__restrict__ C, uint64_t ldc, uint32_t N,
                                                                   uint32_t *__restrict__ next_row)
{
    const int lane = threadIdx.x & 31;
    const uint32_t n0 = blockIdx.y * kSlab;
    for (;;) {
        uint32_t first = 0;
        if (lane == 0) first = atomicAdd(next_row + blockIdx.y, kClaim);
        first = __shfl_sync(kFull, first, 0);
        if (first >= M) break;  // also ends the loop should the counter ever wrap: M < 2^32 - kClaim * warps is not assumed
        const uint32_t last = min(M, first + kClaim);
        for (uint64_t r = first; r < last; ++r) {
            const Range rg = row_range(rowPtr, r, nnz);
            const uint32_t j0 = rg.j0, j1 = rg.j1;
            if (j1 - j0 > kSplit) continue;  // written by the fix-up kernel
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            accumulate(acc, cols, vals, j0, j1, B, ldb, n0, N, K, lane);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (n0 + lane + 32 * i < N) C[r * ldc + n0 + lane + 32 * i] = acc[i];
        }
    }
}

// Chunks of long rows.  A warp takes a window of kSplit nonzero positions, finds the row that holds
// the window's first position by bisection over rowPtr, and computes every chunk that starts inside
// the window (at most two) into its slot of the scratch.
__global__ void __launch_bounds__(kWarps * 32) noalloc_chunks_kernel(const uint32_t *__restrict__ rowPtr,
                                                                     const uint32_t *__restrict__ cols,
                                                                     const float *__restrict__ vals, uint32_t M,
                                                                     uint32_t K, uint32_t nnz, const float *__restrict__ B,
                                                                     uint64_t ldb, float *__restrict__ scratch,
                                                                     uint32_t lds, uint32_t N)
{
    const int lane = threadIdx.x & 31;
    const uint32_t n0 = blockIdx.y * kSlab;
    const uint32_t windows = (nnz + kSplit - 1) / kSplit;
    const uint64_t nw = (uint64_t)gridDim.x * kWarps;
    for (uint64_t w = (uint64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); w < windows; w += nw) {
        const uint32_t p0 = (uint32_t)w * kSplit, p1 = min(nnz, p0 + kSplit);
        // last row r with rowPtr[r] <= p0 (rows without nonzeros share a start; take the last of them)
        uint32_t lo = 0, hi = M;  // invariant: rowPtr[lo] <= p0 < rowPtr[hi] (rowPtr[M] = nnz > p0)
        while (hi - lo > 1) {
            const uint32_t mid = lo + (hi - lo) / 2;
            if (__ldg(rowPtr + mid) <= p0) lo = mid; else hi = mid;
        }
        for (uint32_t r = lo; r < M; ++r) {
            const Range rg = row_range(rowPtr, r, nnz);
            const uint32_t j0 = rg.j0, j1 = rg.j1;
            if (j0 >= p1) break;
            if (j1 - j0 <= kSplit) continue;
            // chunk starts of row r are j0, j0 + kSplit, ...; the one (if any) inside [p0, p1)
            uint32_t i = j0 >= p0 ? 0u : (p0 - j0 + kSplit - 1) / kSplit;
            const uint32_t start = j0 + i * kSplit;  // cannot wrap: start < j1 is checked before use below
            if (start < p0 || start >= p1 || start >= j1) continue;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            accumulate(acc, cols, vals, start, min(j1, start + kSplit), B, ldb, n0, N, K, lane);
            float *out = scratch + chunk_slot(start, i == 0) * lds + n0 + lane;
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (n0 + lane + 32 * k < N) out[32 * k] = acc[k];
        }
    }
}

// C[row] of every long row = its chunks' partial sums, added in chunk order.
__global__ void __launch_bounds__(kWarps * 32) noalloc_fixup_kernel(const uint32_t *__restrict__ rowPtr, uint32_t M,
                                                                    uint32_t nnz, const float *__restrict__ scratch, uint32_t lds,
                                                                    float *__restrict__ C, uint64_t ldc, uint32_t N)
{
    const int lane = threadIdx.x & 31;
    const uint32_t n0 = blockIdx.y * kSlab;
    const uint64_t nw = (uint64_t)gridDim.x * kWarps;
    for (uint64_t r = (uint64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); r < M; r += nw) {
        const Range rg = row_range(rowPtr, r, nnz);
        const uint32_t j0 = rg.j0, j1 = rg.j1;
        if (j1 - j0 <= kSplit) continue;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (uint32_t start = j0, i = 0; start < j1; start += kSplit, ++i) {
            const float *in = scratch + chunk_slot(start, i == 0) * lds + n0 + lane;
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (n0 + lane + 32 * k < N) acc[k] += in[32 * k];
            if (j1 - start <= kSplit) break;  // last chunk (also keeps start from wrapping past 2^32)
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (n0 + lane + 32 * k < N) C[r * ldc + n0 + lane + 32 * k] = acc[k];
    }
}

// Device address of g_scratch and the SM count, looked up once per device.
struct DeviceSetup {
    float *scratch = nullptr;
    uint32_t *next_row = nullptr;
    int sm_count = 0;
    int rows_blocks_per_sm = 0;  // resident blocks of the rows kernel: its grid is one resident wave
    int chunks_blocks_per_sm = 0;  // the same for the chunks kernel
};
constexpr int kMaxDevices = 64;
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;

int fail(int status, const std::string &msg)
{
    cutespmm::set_last_error(msg);
    return status;
}

}  // namespace

extern "C" int cutespmm_spmm_csr_noalloc(uint32_t M, uint32_t K, uint32_t nnz, const uint32_t *rowPtr_dev,
                                         const uint32_t *cols_dev, const float *vals_dev, const float *B_dev,
                                         uint64_t ldb, float *C_dev, uint64_t ldc, uint32_t N, void *stream)
{
    if (N == 0 || M == 0) return CUTESPMM_OK;
    if (!rowPtr_dev || !C_dev || (nnz && (!cols_dev || !vals_dev || !B_dev)))
        return fail(CUTESPMM_EINVAL, "cutespmm_spmm_csr_noalloc: null pointer");
    if (ldb < N || ldc < N) return fail(CUTESPMM_EINVAL, "cutespmm_spmm_csr_noalloc: leading dimension smaller than N");
    if (N > CUTESPMM_NOALLOC_MAX_N)
        return fail(CUTESPMM_EUNSUPPORTED, "cutespmm_spmm_csr_noalloc: N exceeds CUTESPMM_NOALLOC_MAX_N (" +
                                               std::to_string(CUTESPMM_NOALLOC_MAX_N) + "); call it per column window");
    const uint32_t lds = (N + 3) / 4 * 4;
    const uint64_t slots = 2ull * ((nnz + kSplit - 1) / kSplit) + 2;
    if (slots * lds > kScratchFloats)
        return fail(CUTESPMM_EUNSUPPORTED,
                    "cutespmm_spmm_csr_noalloc: the built-in scratch (" + std::to_string(CUTESPMM_NOALLOC_SCRATCH_BYTES >> 20) +
                        " MiB) holds (2*ceil(nnz/" + std::to_string(kSplit) + ")+2) x N partial sums; this call needs " +
                        std::to_string((slots * lds * 4) >> 20) + " MiB. Use a plan (cutespmm_plan_create) or split the rows.");
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(CUTESPMM_ECUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(CUTESPMM_EUNSUPPORTED, "cutespmm_spmm_csr_noalloc: device ordinal too large");
    DeviceSetup setup;
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (!g_setup[dev].scratch) {  // first call on this device: resolve the symbol with this device current
            float *ptr = nullptr;
            e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_scratch);
            if (e != cudaSuccess || !ptr)
                return fail(CUTESPMM_ECUDA, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
            int sms = 0;
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess || sms <= 0)
                return fail(CUTESPMM_ECUDA, std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
            uint32_t *ctr = nullptr;
            e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ctr), g_next_row);
            if (e != cudaSuccess || !ctr)
                return fail(CUTESPMM_ECUDA, std::string("cudaGetSymbolAddress(row counters): ") + cudaGetErrorString(e));
            int per_sm = 0;
            e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, noalloc_rows_kernel, kWarps * 32, 0);
            if (e != cudaSuccess) return fail(CUTESPMM_ECUDA, std::string("cudaOccupancyMaxActiveBlocksPerMultiprocessor: ") + cudaGetErrorString(e));
            int per_sm_chunks = 0;
            e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm_chunks, noalloc_chunks_kernel, kWarps * 32, 0);
            if (e != cudaSuccess) return fail(CUTESPMM_ECUDA, std::string("cudaOccupancyMaxActiveBlocksPerMultiprocessor: ") + cudaGetErrorString(e));
            g_setup[dev].sm_count = sms;
            g_setup[dev].rows_blocks_per_sm = per_sm > 0 ? per_sm : 1;
            g_setup[dev].chunks_blocks_per_sm = per_sm_chunks > 0 ? per_sm_chunks : 1;
            g_setup[dev].next_row = ctr;
            g_setup[dev].scratch = ptr;
        }
        setup = g_setup[dev];
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint32_t slabs = (N + kSlab - 1) / kSlab;
    const uint32_t max_blocks = (uint32_t)setup.sm_count * 8;
    auto blocks_for = [&](uint64_t items) {
        const uint64_t b = (items + kWarps - 1) / kWarps;
        return (uint32_t)(b < 1 ? 1 : (b > max_blocks ? max_blocks : b));
    };
    // the rows kernel: one resident wave of blocks whose warps claim rows from a counter per slab, zeroed here on the stream
    e = cudaMemsetAsync(setup.next_row, 0, sizeof(uint32_t) * (CUTESPMM_NOALLOC_MAX_N / kSlab), s);
    if (e != cudaSuccess) return fail(CUTESPMM_ECUDA, std::string("cutespmm_spmm_csr_noalloc: clearing the row counters: ") + cudaGetErrorString(e));
    {
        const uint64_t want = ((uint64_t)M + kClaim * kWarps - 1) / (kClaim * kWarps);
        const uint64_t wave = (uint64_t)setup.sm_count * setup.rows_blocks_per_sm;
        noalloc_rows_kernel<<<dim3((uint32_t)(want < wave ? (want ? want : 1) : wave), slabs), kWarps * 32, 0, s>>>(
            rowPtr_dev, cols_dev, vals_dev, M, K, nnz, B_dev, ldb, C_dev, ldc, N, setup.next_row);
    }
    if (nnz > kSplit) {  // a long row needs more than kSplit nonzeros
        const uint32_t chunk_wave = (uint32_t)setup.sm_count * (uint32_t)setup.chunks_blocks_per_sm;
        noalloc_chunks_kernel<<<dim3(std::min(blocks_for((nnz + kSplit - 1) / kSplit), chunk_wave), slabs), kWarps * 32, 0, s>>>(
            rowPtr_dev, cols_dev, vals_dev, M, K, nnz, B_dev, ldb, setup.scratch, lds, N);
        noalloc_fixup_kernel<<<dim3(blocks_for(M), slabs), kWarps * 32, 0, s>>>(rowPtr_dev, M, nnz, setup.scratch, lds,
                                                                                C_dev, ldc, N);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(CUTESPMM_ECUDA, std::string("cutespmm_spmm_csr_noalloc launch: ") + cudaGetErrorString(e));
    return CUTESPMM_OK;
}
