// Slab kernel: the Blackwell-native tensor-core path.  A 128-row panel of A times the gathered rows
// of B, one tcgen05.mma (128 x 128 x 8, kind::tf32) per step of 8 active columns, accumulator in
// tensor memory (TMEM).
//
// Role in the reference: SpMM<NUM_WARPS,ILP_LEVEL> (kernel.cu:119-288) -- panels, active columns,
// bitmask-compressed A -- but with the data flow of the 5th-generation tensor core:
//   * a producer warp gathers the step's eight rows of B (512 B each) and its record with TMA bulk
//     copies into a shared-memory stage, kStages deep, mbarrier-tracked;
//   * the four consumer warps transpose the eight rows into the MMA's canonical K-major layout
//     (column n's eight values as two 16-byte chunks at (n/8)*256 + (n%8)*16 + {0,128}; optionally
//     rounding to TF32 to nearest on the way) and expand the step's rows of A into the canonical K-major layout (a thread owns a row:
//     it writes the row's 8 values when the record lists the row, zeros when it wrote the row the
//     previous time this stage was used, nothing otherwise);
//   * one thread issues the MMA from shared-memory descriptors; B never passes through registers
//     as an MMA fragment, there is no per-lane fragment arithmetic, and the 128 x 128 fp32
//     accumulator lives in TMEM, not in registers;
//   * tcgen05.commit signals an mbarrier when the MMAs that read a stage are done, which frees the
//     stage; at the end of a panel the accumulator is read back with tcgen05.ld and stored to C.
// Every wait is bounded; a wait that runs out sets the plan's status word (3) and the block winds
// down: all threads still meet at the step barrier, leave the loops together, and TMEM is freed.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "device_plan.hpp"
#include "plan.hpp"
#include "ptx.cuh"

namespace cutespmm {

namespace {

#ifndef SLAB_STAGES
#define SLAB_STAGES 3
#endif
constexpr int kStages = SLAB_STAGES;
constexpr int kConsumers = 128;               // 4 warps, one TMEM lane quadrant each
constexpr int kThreads = kConsumers + 32;     // + the producer warp
constexpr int kN = 128;                       // columns of B / C per block
constexpr int kBStride = kN + 4;              // floats between staged rows of B (conflict-free re-layout reads)
constexpr unsigned kFull = 0xffffffffu;

// one stage (bytes)
constexpr int kOffA = 0;                              // canonical A tile, 128 x 8 tf32
constexpr int kOffB = 4096;                           // canonical B tile, 128 (N) x 8 (K) tf32
constexpr int kOffStage = 8192;                       // staged rows of B as gathered
constexpr int kOffRec = kOffStage + 8 * kBStride * 4; // the step's record
constexpr int kStageBytes = (kOffRec + (int)kSlabRecMaxWords * 4 + 127) / 128 * 128;
constexpr int kOffBars = kStages * kStageBytes;       // full[kStages], empty[kStages], mma_done[kStages], panel_done
constexpr int kSmemBytes = kOffBars + (3 * kStages + 1) * 8 + 16;

// ---- tcgen05 wrappers -------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ptx::smem_u32(bar))
                 : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], 128 x 128 x 8, tf32 inputs, fp32 accumulate
__device__ __forceinline__ void tc_mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Shared-memory matrix descriptor, no swizzle (layout type 0), descriptor version 1 (bits 46-47).
// lbo / sbo in bytes for a K-major operand: sbo = distance between 8-row groups, lbo = between the
// two 16-byte K chunks of a row.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo)
{
    return (uint64_t)((saddr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46);
}
// Instruction descriptor: D fp32 (bits 4-5 = 1), A and B tf32 (bits 7-9, 10-12 = 2), A and B K-major
// (bits 15, 16 = 0), N/8 in bits 17-22, M/16 in bits 24-28.  (With B MN-major and no swizzle the
// tensor core returned zeros for tf32 on this part, so B is transposed on the way into its tile.)
constexpr uint32_t kIdesc = (1u << 4) | (2u << 7) | (2u << 10) | ((kN / 8u) << 17) | ((kSlabRows / 16u) << 24);

}  // namespace

namespace {

template <bool ROUND_B>
__global__ void __launch_bounds__(kThreads, 4) spmm_slab_kernel(SlabArgs a)
{
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + kOffBars);
    uint64_t *empty = full + kStages, *mma_done = empty + kStages, *panel_done = mma_done + kStages;
    volatile uint32_t *misc = reinterpret_cast<volatile uint32_t *>(panel_done + 1);  // [0] TMEM base, [1] abort flag
    const uint32_t n0 = blockIdx.y * kN;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], 1);
            ptx::mbar_init(&mma_done[s], 1);
        }
        ptx::mbar_init(panel_done, 1);
        misc[1] = 0;
        ptx::fence_mbar_init();
    }
    // the A tiles start as zeros; afterwards every thread undoes exactly what it wrote
    for (int i = tid; i < kStages * 256; i += kThreads)
        *reinterpret_cast<uint4 *>(smem + (i / 256) * kStageBytes + kOffA + (i % 256) * 16) = make_uint4(0, 0, 0, 0);
#ifdef SLAB_DEBUG_ONES
    for (int i = tid; i < kStages * kStageBytes / 4; i += kThreads) reinterpret_cast<float *>(smem)[i] = 1.0f;
#endif
    if (warp == 0) tmem_alloc(ptx::smem_u32(const_cast<uint32_t *>(&misc[0])), kN);  // 128 fp32 columns x 128 lanes
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = misc[0];
    const uint32_t my_panels = blockIdx.x < a.num_panels ? (a.num_panels - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if (warp == 4) {
        // ================= producer warp: TMA gathers, kStages ahead =================
        auto load_cols = [&](uint32_t g) { return __ldg(a.cols + (size_t)g * 32 + lane); };
        auto load_offs = [&](uint32_t g) { return lane < 5 ? __ldg(a.rec_off + (size_t)g * 4 + lane) : 0u; };
        auto load_range = [&](uint32_t o, uint32_t &k0, uint32_t &k1) {
            k0 = k1 = 0;
            if (o < a.num_panels) {
                k0 = __ldg(a.panel_first + o);
                k1 = __ldg(a.panel_last + o);
            }
        };
        const float *Bn = a.B + n0;
        const uint32_t ldb32 = (uint32_t)a.ldb;
        uint32_t ord = blockIdx.x, issued = 0;
        uint32_t pk, pk_end, n_k0, n_k1;
        load_range(ord, pk, pk_end);
        load_range(ord + gridDim.x, n_k0, n_k1);
        uint32_t G = pk >> 2;
        uint32_t mc_cur = load_cols(G), mo_cur = load_offs(G), mc_nxt = load_cols(G + 1), mo_nxt = load_offs(G + 1);
        uint32_t n_mc = load_cols(n_k0 >> 2), n_mo = load_offs(n_k0 >> 2);
        while (pk < pk_end && !misc[1]) {
            if ((pk >> 2) != G) {
                ++G;
                mc_cur = mc_nxt; mo_cur = mo_nxt;
                mc_nxt = load_cols(G + 1); mo_nxt = load_offs(G + 1);
            }
            const int s = issued % kStages;
            if (!ptx::mbar_wait(&empty[s], ((issued / kStages) & 1u) ^ 1u)) {  // consumers never released the stage
                if (lane == 0) { atomicExch(a.status, 3u); misc[1] = 1; }
                break;
            }
            unsigned char *st = smem + s * kStageBytes;
            const uint32_t col = __shfl_sync(kFull, mc_cur, (pk & 3) * 8 + (lane & 7));
            const uint32_t o0 = __shfl_sync(kFull, mo_cur, pk & 3), o1 = __shfl_sync(kFull, mo_cur, (pk & 3) + 1);
            const uint32_t rec_bytes = (o1 - o0) * 16u;
            if (lane == 0) ptx::mbar_expect_tx(&full[s], 8u * kN * 4u + rec_bytes);
            __syncwarp();
            if (lane < 8)
                ptx::bulk_g2s(st + kOffStage + lane * kBStride * 4, Bn + (uint64_t)col * ldb32, kN * 4u, &full[s]);
            else if (lane == 8)
                ptx::bulk_g2s(st + kOffRec, a.recs + (size_t)o0 * 4, rec_bytes, &full[s]);
            ++issued;
            if (++pk == pk_end) {  // next panel of this block
                ord += gridDim.x;
                pk = n_k0; pk_end = n_k1;
                G = pk >> 2;
                mc_cur = n_mc; mo_cur = n_mo;
                if (pk < pk_end) {
                    mc_nxt = load_cols(G + 1); mo_nxt = load_offs(G + 1);
                    load_range(ord + gridDim.x, n_k0, n_k1);
                    n_mc = load_cols(n_k0 >> 2); n_mo = load_offs(n_k0 >> 2);
                }
            }
        }
    } else {
        // ================= consumer warps: build operands, issue MMAs, drain TMEM =================
        const int row = tid;                                   // the row of the panel this thread owns
        const uint32_t a_off = (row >> 3) * 256 + (row & 7) * 16;  // its two 16-byte K chunks: a_off, a_off + 128
        uint32_t dirty = 0;                                    // bit s: this thread's row in stage s holds values
        uint32_t step = 0, panels_done = 0, panel_idx = 0;
        bool first_of_panel = true;
#ifdef SLAB_DEBUG_PREFILL
        {
            const uint32_t seven = __float_as_uint(7.0f);
            for (int ch = 0; ch < 4; ++ch) {
                const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + ch * 32;
                asm volatile(
                    "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,"
                    "%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(taddr), "r"(seven) : "memory");
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            first_of_panel = false;
        }
#endif
        for (uint32_t p = 0; p < my_panels; ++p) {
            for (;;) {
                const int s = step % kStages;
                const uint32_t par = (step / kStages) & 1u;
                unsigned char *st = smem + s * kStageBytes;
                bool ok = ptx::mbar_wait(&full[s], par);             // the step's rows of B and record have landed
                ok = ok && ptx::mbar_wait(&mma_done[s], par ^ 1u);   // the MMA that last read this stage's tiles is done
                uint32_t last = 1;
                if (ok) {
                    const uint32_t *rec = reinterpret_cast<const uint32_t *>(st + kOffRec);
                    const uint4 head = *reinterpret_cast<const uint4 *>(rec);        // cnt|last<<16, panel, nvals, -
                    const uint4 present = *reinterpret_cast<const uint4 *>(rec + 4);  // one bit per row of the panel
                    last = (head.x >> 16) & 1u;
                    panel_idx = head.y;
                    const uint32_t cnt = head.x & 0xffffu;
                    // ---- A: this thread's row ----
                    const uint32_t w = row >> 5, bit = row & 31;
                    const uint32_t word = w == 0 ? present.x : w == 1 ? present.y : w == 2 ? present.z : present.w;
                    float4 *a_lo = reinterpret_cast<float4 *>(st + kOffA + a_off), *a_hi = reinterpret_cast<float4 *>(st + kOffA + a_off + 128);
                    if ((word >> bit) & 1u) {
                        const uint32_t before = (w > 0 ? __popc(present.x) : 0) + (w > 1 ? __popc(present.y) : 0) +
                                                (w > 2 ? __popc(present.z) : 0) + __popc(word & ((1u << bit) - 1u));
                        const uint32_t ent = rec[kSlabRecHeaderWords + before];
                        const uint32_t mask = (ent >> 8) & 0xffu;
                        const float *vals = reinterpret_cast<const float *>(rec + kSlabRecHeaderWords + (cnt + 3) / 4 * 4) + (ent >> 16);
                        float v[8];
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const float x = ((mask >> c) & 1u) ? vals[__popc(mask & ((1u << c) - 1u))] : 0.f;
                            v[c] = __uint_as_float(ptx::f32_to_tf32_rna(x));
                        }
                        *a_lo = make_float4(v[0], v[1], v[2], v[3]);
                        *a_hi = make_float4(v[4], v[5], v[6], v[7]);
                        dirty |= 1u << s;
                    } else if ((dirty >> s) & 1u) {
                        *a_lo = make_float4(0.f, 0.f, 0.f, 0.f);
                        *a_hi = make_float4(0.f, 0.f, 0.f, 0.f);
                        dirty &= ~(1u << s);
                    }
                    // ---- B: staged rows -> canonical K-major tile (the MMA's B operand is N x K) ----
                    // this thread owns column n = tid: its 8 K values are one 32-byte row of the operand
                    {
                        const float *col = reinterpret_cast<const float *>(st + kOffStage) + tid;
                        float x[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            x[k] = col[k * kBStride];
                            if (ROUND_B) x[k] = __uint_as_float(ptx::f32_to_tf32_rna(x[k]));
                        }
                        *reinterpret_cast<float4 *>(st + kOffB + a_off) = make_float4(x[0], x[1], x[2], x[3]);
                        *reinterpret_cast<float4 *>(st + kOffB + a_off + 128) = make_float4(x[4], x[5], x[6], x[7]);
                    }
                    ptx::fence_async_smem();  // the tensor core reads these tiles through the async proxy
                } else if (lane == 0) {
                    atomicExch(a.status, 3u);
                    misc[1] = 1;
                }
                tc_fence_before();
                consumer_barrier();
                tc_fence_after();
                if (misc[1]) break;
                if (tid == 0) {
                    ptx::mbar_arrive(&empty[s]);  // staged rows and record may be overwritten
                    const uint64_t adesc = smem_desc(ptx::smem_u32(st + kOffA), 128u, 256u);
                    const uint64_t bdesc = smem_desc(ptx::smem_u32(st + kOffB), 128u, 256u);
#ifdef SLAB_DEBUG
                    if (blockIdx.x == 0 && step < 2) {
                        const float *At = reinterpret_cast<const float *>(st + kOffA), *Bt = reinterpret_cast<const float *>(st + kOffB);
                        printf("step %u s %d tmem %08x adesc %016llx bdesc %016llx idesc %08x acc %u last %u\n", step, s, tmem,
                               (unsigned long long)adesc, (unsigned long long)bdesc, kIdesc, first_of_panel ? 0u : 1u, last);
                        printf("  A row0 k0..3 %g %g %g %g | row1 %g %g %g %g | row0 k4..7 %g %g %g %g\n", At[0], At[1], At[2], At[3], At[4], At[5], At[6],
                               At[7], At[32], At[33], At[34], At[35]);
                        printf("  B chunk0 k0 %g %g %g %g | k1 %g %g %g %g | chunk1 k0 %g %g %g %g\n", Bt[0], Bt[1], Bt[2], Bt[3], Bt[4], Bt[5], Bt[6],
                               Bt[7], Bt[32], Bt[33], Bt[34], Bt[35]);
                    }
#endif
                    tc_mma_tf32(tmem, adesc, bdesc, kIdesc, first_of_panel ? 0u : 1u);
                    tc_commit(&mma_done[s]);
                    if (last) tc_commit(panel_done);
                }
                first_of_panel = false;
                ++step;
                if (last) break;
            }
            if (misc[1]) break;
            // ---- end of panel: accumulator -> C ----
            if (ptx::mbar_wait(panel_done, panels_done & 1u)) {
                tc_fence_after();
                const uint64_t r = (uint64_t)panel_idx * kSlabRows + row;
                float *crow = a.C + r * a.ldc + n0;
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint32_t v[32];
                    tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + ch * 32, v);
#ifdef SLAB_DEBUG
                    if (blockIdx.x == 0 && (tid == 0 || tid == 33) && ch == 0)
                        printf("epilogue tid %d panel %u row %llu v %g %g %g %g\n", tid, panel_idx, (unsigned long long)r, __uint_as_float(v[0]),
                               __uint_as_float(v[1]), __uint_as_float(v[2]), __uint_as_float(v[3]));
#endif
                    if (r < a.M) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            __stcs(reinterpret_cast<float4 *>(crow + ch * 32 + j * 4),
                                   make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                               __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3])));
                    }
                }
                tc_fence_before();
            } else if (lane == 0) {
                atomicExch(a.status, 3u);
                misc[1] = 1;
            }
            ++panels_done;
            first_of_panel = true;
        }
    }
    // ---- wind down: everyone meets, then the allocating warp returns the tensor memory ----
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, kN);
    }
}

}  // namespace

bool slab_supports(uint32_t N, uint64_t ldb, uint64_t ldc, const void *B, const void *C)
{
    const uintptr_t pb = reinterpret_cast<uintptr_t>(B), pc = reinterpret_cast<uintptr_t>(C);
    return N > 0 && N % kN == 0 && !((pb | pc) & 15) && !((ldb | ldc) & 3);
}

cudaError_t launch_slab(const SlabArgs &a, int sm_count, cudaStream_t s)
{
    if (a.num_panels == 0) return cudaSuccess;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(spmm_slab_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(spmm_slab_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    // tensor memory holds 512 columns per SM and a block takes 128: at most 4 resident blocks per SM
    uint32_t blocks = (uint32_t)sm_count * 4u;
    if (blocks > a.num_panels) blocks = a.num_panels;
    const dim3 grid(blocks, a.N / kN);
    if (a.round_b) spmm_slab_kernel<true><<<grid, kThreads, kSmemBytes, s>>>(a);
    else spmm_slab_kernel<false><<<grid, kThreads, kSmemBytes, s>>>(a);
    return cudaGetLastError();
}

}  // namespace cutespmm
