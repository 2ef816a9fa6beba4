// Slab kernel: the Blackwell-native tensor-core path.  A 128-row panel of A times the gathered rows
// of B, one tcgen05.mma (128 x 128 x 8, kind::tf32) per step of 8 active columns, accumulator in
// tensor memory (TMEM).
//
// Role in the reference: SpMM<NUM_WARPS,ILP_LEVEL> (kernel.cu:119-288) -- panels, active columns,
// bitmask-compressed A -- with the data flow of the 5th-generation tensor core:
//   * B never passes through a thread.  The eight gathered rows of a step are placed by the copy
//     engine directly in the layout the MMA reads: eight cp.async.bulk.tensor...tile::gather4 loads
//     (four rows x 32 columns each, tensor map with the 128-byte swizzle on 32-byte atoms) fill the
//     step's 8 x 128 operand tile as an MN-major tf32 operand (the only shared-memory layout the
//     tensor core takes for MN-major tf32 is that swizzle; with any other it returns zeros);
//   * four producer warps take turns issuing a step's loads (issuing one TMA operation costs a thread
//     on the order of a hundred cycles); the column lists and record offsets they need are
//     themselves fetched by TMA one segment ahead;
//   * four builder warps expand the rows of A: the warp that owns a step zeroes the rows it wrote
//     the last time the stage was used and writes the rows the step's record lists (row, 8-bit
//     column mask, packed values) into the canonical K-major operand layout, rounding to TF32;
//   * one thread issues every MMA from shared-memory descriptors; tcgen05.commit signals an mbarrier
//     when the MMAs that read a stage are done, which frees the stage for the producers; at the end
//     of a panel the builder warps read the accumulator back with tcgen05.ld and store it to C.
// All roles are coupled by mbarriers only.  Every wait is bounded; a wait that runs out sets the
// plan's status word (3) and the block's abort flag, every role leaves its loop, the block meets at
// one final barrier and the warp that allocated the tensor memory frees it.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "device_plan.hpp"
#include "plan.hpp"
#include "ptx.cuh"
#include "tmap.hpp"

namespace cutespmm {

namespace {

constexpr int kStages = 8;  // steps of B in flight per block; a multiple of 4 (see static_assert)
constexpr unsigned kBlocksPerSm = 3;  // shared memory and tensor memory (128 of 512 columns each) allow this many per SM
// A stage is always refilled by the same producer warp and its step built by the same builder warp: a
// warp is in order on its own stages, so the one-bit phase parity of a barrier can never be two
// phases stale.
static_assert(kStages % 4 == 0, "stage i % kStages must belong to producer / builder warp i % 4");
constexpr int kATiles = 4;  // A operand tiles per block; a multiple of 4: step i uses tile i % kATiles, built by warp i & 3
// kATiles <= kStages: a builder waits for the MMA of step i - kATiles on that step's stage barrier, which must not
// have been reused in between (the one-bit phase parity cannot tell two phases apart).
static_assert(kATiles % 4 == 0 && kATiles <= kStages, "A tiles are owned by builder warps in turn");
constexpr int kBuilders = 4;                  // builder warps 0-3, one TMEM lane quadrant each
constexpr int kProducers = 4;                 // producer warps 4-7
constexpr int kThreads = (kBuilders + kProducers + 1) * 32;  // + the MMA warp
constexpr int kN = 128;                       // columns of B / C per block

// shared memory: kStages B stages (1024-byte aligned: the swizzle pattern is a function of the address),
// four A tiles, two metadata buffers, barriers
constexpr int kOffRec = 4096;                 // inside a B stage: the operand tile (4 column blocks x 2 K blocks x 512 B), then the record
static_assert(kSlabRecMaxWords * 4 <= 1024, "a step record must fit behind the B tile");
constexpr int kStageBytes = 4096 + 1024;
constexpr int kOffATiles = kStages * kStageBytes;
constexpr int kOffDirty = 4096;               // inside an A tile: the K-major operand tile, then the rows that hold values (count, row numbers)
constexpr int kATileBytes = 4096 + 128;
constexpr int kMetaSlots = 64;   // step slots whose metadata one buffer holds
constexpr int kMetaBytes = kMetaSlots * 32 + (kMetaSlots + 4) * 4;  // columns, then record offsets (+ next, padded)
constexpr int kOffMeta = kOffATiles + kATiles * kATileBytes;
constexpr int kOffBars = kOffMeta + 2 * kMetaBytes;
// full, seen, mma_done per B stage; built per A tile; panel_done, drained; meta_full[2], meta_free[2]
constexpr int kNumBars = 3 * kStages + kATiles + 2 + 4;
constexpr int kOffMisc = kOffBars + kNumBars * 8;
constexpr int kSmemBytes = kOffMisc + 16;

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

// Shared-memory matrix descriptor (descriptor version 1 in bits 46-47).  lbo / sbo in bytes.
//   A, K-major, no swizzle (layout type 0): sbo = distance between 8-row groups, lbo = between the two
//   16-byte K chunks of a row.
//   B, MN-major, 128-byte swizzle on 32-byte atoms (layout type 1): lbo = distance between blocks of 32
//   columns, sbo = between blocks of 4 K rows.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo, uint32_t layout_type)
{
    return (uint64_t)((saddr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46) | ((uint64_t)layout_type << 61);
}
// Instruction descriptor: D fp32 (bits 4-5 = 1), A and B tf32 (bits 7-9, 10-12 = 2), A K-major (bit 15 = 0),
// B MN-major (bit 16 = 1), N/8 in bits 17-22, M/16 in bits 24-28.
constexpr uint32_t kIdesc = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 16) | ((kN / 8u) << 17) | ((kSlabRows / 16u) << 24);

}  // namespace

namespace {

__global__ void __launch_bounds__(kThreads, kBlocksPerSm) spmm_slab_kernel(const __grid_constant__ CUtensorMap tmap_b, SlabArgs a)
{
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + kOffBars);  // TMA -> builders and MMA warp (1 arrival + bytes)
    uint64_t *seen = full + kStages;         // owning builder -> producer: the record has been consumed
    uint64_t *mma_done = seen + kStages;     // tcgen05.commit -> producer (B tile may be refilled) and builder (its A tile may be rewritten)
    uint64_t *built = mma_done + kStages;    // owning builder -> MMA warp: A tile w is ready
    uint64_t *panel_done = built + kATiles;     // tcgen05.commit -> builders: the accumulator is complete
    uint64_t *drained = panel_done + 1;      // builders -> MMA warp: the accumulator has been read (4 arrivals)
    uint64_t *meta_full = drained + 1, *meta_free = meta_full + 2;
    volatile uint32_t *misc = reinterpret_cast<volatile uint32_t *>(smem + kOffMisc);  // [0] TMEM base, [1] abort flag
    const uint32_t n0 = blockIdx.y * kN;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&seen[s], 1);
            ptx::mbar_init(&mma_done[s], 1);
        }
        for (int t = 0; t < kATiles; ++t) ptx::mbar_init(&built[t], 1);
        ptx::mbar_init(panel_done, 1);
        ptx::mbar_init(drained, kBuilders);
        for (int m = 0; m < 2; ++m) {
            ptx::mbar_init(&meta_full[m], 1);
            ptx::mbar_init(&meta_free[m], kProducers);
        }
        misc[1] = 0;
        ptx::fence_mbar_init();
    }
    // the A tiles start as zeros and hold no rows; afterwards the owning builder undoes exactly what it wrote
    for (int i = tid; i < kATiles * 256; i += kThreads)
        *reinterpret_cast<uint4 *>(smem + kOffATiles + (i / 256) * kATileBytes + (i % 256) * 16) = make_uint4(0, 0, 0, 0);
    if (tid < kATiles) *reinterpret_cast<volatile uint32_t *>(smem + kOffATiles + tid * kATileBytes + kOffDirty) = 0;
    if (warp == 0) tmem_alloc(ptx::smem_u32(const_cast<uint32_t *>(&misc[0])), kN);  // 128 fp32 columns x 128 lanes
    ptx::fence_async_smem();  // the zeroed tiles are read through the async proxy
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = misc[0];
    const uint32_t my_panels = blockIdx.x < a.num_panels ? (a.num_panels - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    auto abort_now = [&]() {
        atomicExch(a.status, 3u);
        misc[1] = 1;
    };

    if (warp >= kBuilders && warp < kBuilders + kProducers) {
        // ================= producer warps: TMA gathers, kStages ahead =================
        const uint32_t pw = warp - kBuilders;  // this warp issues the steps i with i % 4 == pw
        auto load_range = [&](uint32_t o, uint32_t &k0, uint32_t &k1) {
            k0 = k1 = 0;
            if (o < a.num_panels) {
                k0 = __ldg(a.panel_first + o);
                k1 = __ldg(a.panel_last + o);
            }
        };
        // segment generator: walks this block's panels, cutting each into segments of <= kMetaSlots slots
        uint32_t g_ord = blockIdx.x, g_k, g_k1, r1_k0, r1_k1, r2_k0, r2_k1;
        load_range(g_ord, g_k, g_k1);
        load_range(g_ord + gridDim.x, r1_k0, r1_k1);
        load_range(g_ord + 2 * gridDim.x, r2_k0, r2_k1);
        uint32_t fetched = 0;  // segments whose metadata fetch has been started
        auto fetch_next = [&](uint32_t &seg_begin, uint32_t &seg_end) {  // false when there is no further segment
            if (g_k >= g_k1) return false;
            seg_begin = g_k;
            seg_end = min(g_k1, g_k + kMetaSlots);
            const uint32_t slots = (seg_end - seg_begin + 3) & ~3u;
            const int m = fetched & 1;
            if (pw == 0 && lane == 0) {  // one warp fetches for all; the buffer's previous segment must have been read by all four
                if (!ptx::mbar_wait(&meta_free[m], ((fetched >> 1) & 1u) ^ 1u)) abort_now();
                unsigned char *mb = smem + kOffMeta + m * kMetaBytes;
                ptx::mbar_expect_tx(&meta_full[m], slots * 32u + (slots + 4u) * 4u);
                ptx::bulk_g2s(mb, a.cols + (size_t)seg_begin * 8, slots * 32u, &meta_full[m]);
                ptx::bulk_g2s(mb + kMetaSlots * 32, a.rec_off + seg_begin, (slots + 4u) * 4u, &meta_full[m]);
            }
            ++fetched;
            g_k = seg_end;
            if (g_k >= g_k1) {  // panel exhausted: this block's next panel (its range was loaded two panels ago)
                g_ord += gridDim.x;
                g_k = r1_k0; g_k1 = r1_k1;
                r1_k0 = r2_k0; r1_k1 = r2_k1;
                load_range(g_ord + 2 * gridDim.x, r2_k0, r2_k1);
            }
            return true;
        };
        uint32_t issued = 0, seg = 0;
        uint32_t cur_b = 0, cur_e = 0, nxt_b = 0, nxt_e = 0;
        bool have_cur = fetch_next(cur_b, cur_e);
        while (have_cur && !misc[1]) {
            const bool have_nxt = fetch_next(nxt_b, nxt_e);  // one segment ahead
            const int m = seg & 1;
            if (!ptx::mbar_wait(&meta_full[m], (seg >> 1) & 1u)) {
                if (lane == 0) abort_now();
                break;
            }
            const uint32_t *mcols = reinterpret_cast<const uint32_t *>(smem + kOffMeta + m * kMetaBytes);
            const uint32_t *moffs = mcols + kMetaSlots * 8;
            bool ok = true;
            for (uint32_t k = cur_b; k < cur_e; ++k, ++issued) {
                if (issued % kProducers != pw) continue;
                const int s = issued % kStages;
                const uint32_t par = ((issued / kStages) & 1u) ^ 1u;
                // lane l < 8 loads K rows 4*(l&1) .. +3 of column block l>>1; its four row coordinates:
                const uint4 rows4 = *reinterpret_cast<const uint4 *>(mcols + (k - cur_b) * 8 + (lane & 1) * 4);
                const uint32_t o0 = moffs[k - cur_b], o1 = moffs[k - cur_b + 1];
                // the stage is free once the MMA that read its B tile is done and its builder has consumed the record
                ok = ptx::mbar_wait(&mma_done[s], par) && ptx::mbar_wait(&seen[s], par);
                if (!ok) break;
                unsigned char *st = smem + s * kStageBytes;
                if (lane == 8) {
                    ptx::mbar_expect_tx(&full[s], 8u * kN * 4u + (o1 - o0) * 16u);
                    ptx::bulk_g2s(st + kOffRec, a.recs + (size_t)o0 * 4, (o1 - o0) * 16u, &full[s]);
                } else if (lane < 8) {
                    ptx::tma_gather4(st + (lane >> 1) * 1024 + (lane & 1) * 512, &tmap_b, (int)(n0 + 32 * (lane >> 1)), (int)rows4.x,
                                (int)rows4.y, (int)rows4.z, (int)rows4.w, &full[s]);
                }
            }
            if (!ok) {
                if (lane == 0) abort_now();
                break;
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&meta_free[m]);  // this warp is done with the segment's metadata
            ++seg;
            cur_b = nxt_b; cur_e = nxt_e;
            have_cur = have_nxt;
        }
    } else if (warp == kBuilders + kProducers) {
        // ================= MMA warp: one thread issues every tcgen05.mma of the block =================
        if (lane == 0) {
            const uint64_t adesc0 = smem_desc(ptx::smem_u32(smem + kOffATiles), 128u, 256u, 0u);
            const uint64_t bdesc0 = smem_desc(ptx::smem_u32(smem), 1024u, 512u, 1u);
            uint32_t step = 0;
            for (uint32_t p = 0; p < my_panels && !misc[1]; ++p) {
                const uint32_t ord = blockIdx.x + p * gridDim.x;
                const uint32_t nsteps = __ldg(a.panel_last + ord) - __ldg(a.panel_first + ord);
                // the previous panel's accumulator must have been read before it is overwritten
                if (p > 0 && !ptx::mbar_wait(drained, (p - 1) & 1u)) { abort_now(); break; }
                bool ok = true;
                for (uint32_t i = 0; i < nsteps; ++i, ++step) {
                    const int s = step % kStages, t = step % kATiles;
                    ok = ptx::mbar_wait(&built[t], (step / kATiles) & 1u) && ptx::mbar_wait(&full[s], (step / kStages) & 1u);
                    if (!ok) break;
                    tc_fence_after();
                    // descriptors differ from the first tile's only in the address field (16-byte units)
                    tc_mma_tf32(tmem, adesc0 + (uint64_t)(t * (kATileBytes >> 4)), bdesc0 + (uint64_t)(s * (kStageBytes >> 4)), kIdesc, i ? 1u : 0u);
                    tc_commit(&mma_done[s]);
                }
                if (!ok) { abort_now(); break; }
                tc_commit(panel_done);
            }
        }
    } else {
        // ================= builder warps 0-3: rows of A, then the accumulator read-back =================
        // Step i of the block is built by warp i & 3 into its own A tile.  The number of steps of each of
        // the block's panels comes from the panel table, so a warp touches only the steps it owns.
        uint32_t step0 = 0;  // block-wide index of the current panel's first step
        for (uint32_t p = 0; p < my_panels && !misc[1]; ++p) {
            const uint32_t ord = blockIdx.x + p * gridDim.x;
            const uint32_t nsteps = __ldg(a.panel_last + ord) - __ldg(a.panel_first + ord);
            const uint32_t panel_idx = __ldg(a.panel_ids + ord);
            bool ok = true;
            for (uint32_t step = step0 + ((warp - step0) & 3u); step < step0 + nsteps; step += 4) {
                const int s = step % kStages, t = step % kATiles;
                unsigned char *at = smem + kOffATiles + t * kATileBytes;  // the step's A tile (one of this warp's)
                // the step's record has landed; the MMA that read this A tile kATiles steps ago is done
                ok = ptx::mbar_wait(&full[s], (step / kStages) & 1u) &&
                     (step < (uint32_t)kATiles || ptx::mbar_wait(&mma_done[(step - kATiles) % kStages], ((step - kATiles) / kStages) & 1u));
                if (!ok) break;
                const uint32_t *rec = reinterpret_cast<const uint32_t *>(smem + s * kStageBytes + kOffRec);
                const uint32_t cnt = rec[0] & 0xffffu;
                // clear the rows written for that earlier step, then write this step's rows
                volatile uint32_t *dirty_cnt = reinterpret_cast<volatile uint32_t *>(at + kOffDirty);
                unsigned char *dirty_rows = at + kOffDirty + 16;
                const uint32_t old = *dirty_cnt;
                if ((uint32_t)lane < old) {
                    const uint32_t r = dirty_rows[lane];
                    float4 *d = reinterpret_cast<float4 *>(at + (r >> 3) * 256 + (r & 7) * 16);
                    d[0] = make_float4(0.f, 0.f, 0.f, 0.f);
                    d[8] = make_float4(0.f, 0.f, 0.f, 0.f);  // + 128 bytes: the row's second K chunk
                }
                __syncwarp();
                if ((uint32_t)lane < cnt) {  // a record lists at most 32 rows: one lane each
                    const uint32_t *entries = rec + kSlabRecHeaderWords;
                    const float *vals = reinterpret_cast<const float *>(entries + (cnt + 3) / 4 * 4);
                    const uint32_t ent = entries[lane];
                    const uint32_t r = ent & 0xffu, mask = (ent >> 8) & 0xffu;
                    const float *v0 = vals + (ent >> 16);
                    float v[8];
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const float x = ((mask >> c) & 1u) ? v0[__popc(mask & ((1u << c) - 1u))] : 0.f;
                        v[c] = __uint_as_float(ptx::f32_to_tf32_rna(x));
                    }
                    float4 *d = reinterpret_cast<float4 *>(at + (r >> 3) * 256 + (r & 7) * 16);
                    d[0] = make_float4(v[0], v[1], v[2], v[3]);
                    d[8] = make_float4(v[4], v[5], v[6], v[7]);
                    dirty_rows[lane] = (unsigned char)r;
                }
                if (lane == 0) *dirty_cnt = cnt;
                ptx::fence_async_smem();  // the tensor core reads the tile through the async proxy
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(&built[t]);
                    ptx::mbar_arrive(&seen[s]);
                }
            }
            if (!ok) {
                if (lane == 0) abort_now();
                break;
            }
            step0 += nsteps;
            if (misc[1]) break;
            // ---- end of panel: accumulator -> C (this warp's 32 rows) ----
            if (!ptx::mbar_wait(panel_done, p & 1u)) {
                if (lane == 0) abort_now();
                break;
            }
            tc_fence_after();
            const uint64_t r = (uint64_t)panel_idx * kSlabRows + tid;
            float *crow = a.C + r * a.ldc + n0;
#pragma unroll 1
            for (int ch = 0; ch < 4; ++ch) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + ch * 32, v);
                if (r < a.M) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        __stcs(reinterpret_cast<float4 *>(crow + ch * 32 + j * 4),
                               make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                                           __uint_as_float(v[4 * j + 3])));
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(drained);
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
    cudaError_t e = allow_dynamic_smem<spmm_slab_kernel>(kSmemBytes);
    if (e != cudaSuccess) return e;
    // B as a 2-D tensor (columns innermost); one gather4 brings 4 rows x 32 columns = a 4 x 128-byte atom
    CUtensorMap tmap;
    e = make_b_tensor_map(&tmap, a.B, a.N, a.K, a.ldb, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    if (e != cudaSuccess) return e;
    uint32_t blocks = (uint32_t)sm_count * kBlocksPerSm;
    if (blocks > a.num_panels) blocks = a.num_panels;
    spmm_slab_kernel<<<dim3(blocks, a.N / kN), kThreads, kSmemBytes, s>>>(tmap, a);
    return cudaGetLastError();
}

}  // namespace cutespmm
