// Slab kernel: the Blackwell-native tensor-core path.  A 128-row panel of A times the gathered rows
// of B, one tcgen05.mma (128 x 128 x 8, kind::tf32) per step of 8 active columns, accumulator in
// tensor memory (TMEM).
//
// Role in the reference: SpMM<NUM_WARPS,ILP_LEVEL> (kernel.cu:119-288) -- panels, active columns,
// bitmask-compressed A -- but with the data flow of the 5th-generation tensor core:
//   * four producer warps (taking turns, one step each) gather a step's eight rows of B (512 B each)
//     and its record with TMA bulk copies into a shared-memory landing stage, kStages deep,
//     mbarrier-tracked; the column lists and record offsets they need are themselves fetched by TMA
//     one segment ahead (issuing one bulk copy costs a thread on the order of a hundred cycles, so
//     a single issuing warp was the bottleneck);
//   * four builder warps transpose the eight rows into the MMA's canonical K-major layout (column
//     n's eight values as two 16-byte chunks at (n/8)*256 + (n%8)*16 + {0,128}; optionally rounding
//     to TF32 to nearest on the way); one of them, taking turns, expands the step's rows of A into
//     the same layout: it zeroes the rows written the previous time the stage was used and writes
//     the rows the record lists;
//   * one thread issues the MMA from shared-memory descriptors; B never passes through registers
//     as an MMA fragment, there is no per-lane fragment arithmetic, and the 128 x 128 fp32
//     accumulator lives in TMEM, not in registers;
//   * tcgen05.commit signals an mbarrier when the MMAs that read a stage are done, which frees the
//     stage; at the end of a panel the accumulator is read back with tcgen05.ld and stored to C.
// Every wait is bounded; a wait that runs out sets the plan's status word (3) and the block winds
// down: all threads still meet at the step barrier, leave the loops together, and TMEM is freed.
#include <cuda_runtime.h>

#include <cstdint>

#include "device_plan.hpp"
#include "plan.hpp"
#include "ptx.cuh"

namespace cutespmm {

namespace {

#ifndef SLAB_STAGES
#define SLAB_STAGES 4   // gathered rows of B + record in flight per block (hides the L2 / HBM gather latency)
#endif
#ifndef SLAB_TILES
#define SLAB_TILES 4    // operand tile pairs per block: one per builder warp
#endif
#ifndef SLAB_BLOCKS_PER_SM
#define SLAB_BLOCKS_PER_SM 3u
#endif
constexpr int kStages = SLAB_STAGES;
constexpr int kTiles = SLAB_TILES;
static_assert(kTiles == 4, "tile pair i & 3 belongs to builder warp i & 3");
// A landing stage must always be refilled by the same producer warp: a warp is in order on its own
// stages, so the one-bit phase parity of the stage's barriers can never be two phases stale.
static_assert(kStages % 4 == 0, "landing stage i % kStages must belong to producer warp i % 4");
constexpr int kConsumers = 128;               // 4 builder warps, one TMEM lane quadrant each
constexpr int kProducers = 4;                 // producer warps: warp 4 + j issues the copies of steps i with i % 4 == j
constexpr int kThreads = kConsumers + kProducers * 32 + 32;  // builders, producers, the MMA warp
constexpr int kN = 128;                       // columns of B / C per block
constexpr int kBStride = kN + 4;              // floats between staged rows of B

// shared memory: kTiles operand tile pairs, then kStages landing stages, then barriers
constexpr int kOffA = 0;                              // canonical A tile, 128 x 8 tf32
constexpr int kOffB = 4096;                           // canonical B tile, 128 (N) x 8 (K) tf32
constexpr int kOffDirty = 8192;                       // rows of the A tile that hold values: count (16 B), then row numbers
constexpr int kTileBytes = 8192 + 256;
constexpr int kOffRec = 8 * kBStride * 4;             // inside a landing stage: gathered rows first, then the step's record
constexpr int kStageBytes = (kOffRec + (int)kSlabRecMaxWords * 4 + 127) / 128 * 128;
constexpr int kStage0 = kTiles * kTileBytes;
#ifndef SLAB_META_SLOTS
#define SLAB_META_SLOTS 64
#endif
constexpr int kMetaSlots = SLAB_META_SLOTS;                          // step slots whose metadata one buffer holds
constexpr int kMetaBytes = kMetaSlots * 32 + (kMetaSlots + 4) * 4;  // columns, then record offsets (+ next, padded)
constexpr int kOffMeta = kStage0 + kStages * kStageBytes;  // two metadata buffers and their two barriers
constexpr int kOffBars = kOffMeta + 2 * kMetaBytes + 32;  // after the buffers: meta_full[2], meta_free[2]
// full[kStages], sfree[kStages], built[kTiles], mma_done[kTiles], panel_done, drained, then misc words
constexpr int kSmemBytes = kOffBars + (2 * kStages + 2 * kTiles + 2) * 8 + 16 + kTiles * 4;

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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

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
__global__ void __launch_bounds__(kThreads, SLAB_BLOCKS_PER_SM) spmm_slab_kernel(SlabArgs a)
{
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + kOffBars);   // TMA -> builders (1 arrival + bytes)
    uint64_t *sfree = full + kStages;        // builders -> producer: the landing stage has been consumed (4 arrivals)
    uint64_t *built = sfree + kStages;       // owning builder warp -> MMA warp: the tile pair is ready
    uint64_t *mma_done = built + kTiles;     // tcgen05.commit -> builders: the tile pair may be rewritten
    uint64_t *panel_done = mma_done + kTiles;  // tcgen05.commit -> builders: the accumulator is complete
    uint64_t *drained = panel_done + 1;      // builders -> MMA warp: the accumulator has been read (4 arrivals)
    volatile uint32_t *misc = reinterpret_cast<volatile uint32_t *>(drained + 1);  // [0] TMEM base, [1] abort flag, [2+s] step flags
    const uint32_t n0 = blockIdx.y * kN;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&sfree[s], 4);
        }
        for (int t = 0; t < kTiles; ++t) {
            ptx::mbar_init(&built[t], 1);
            ptx::mbar_init(&mma_done[t], 1);
        }
        ptx::mbar_init(panel_done, 1);
        ptx::mbar_init(drained, 4);
        for (int m = 0; m < 2; ++m) {
            ptx::mbar_init(reinterpret_cast<uint64_t *>(smem + kOffMeta + 2 * kMetaBytes) + m, 1);              // meta_full
            ptx::mbar_init(reinterpret_cast<uint64_t *>(smem + kOffMeta + 2 * kMetaBytes) + 2 + m, kProducers);  // meta_free
        }
        misc[1] = 0;
        ptx::fence_mbar_init();
    }
    // the A tiles start as zeros and hold no rows; afterwards the builder undoes exactly what was written
    for (int i = tid; i < kTiles * 256; i += kThreads)
        *reinterpret_cast<uint4 *>(smem + (i / 256) * kTileBytes + kOffA + (i % 256) * 16) = make_uint4(0, 0, 0, 0);
    if (tid < kTiles) *reinterpret_cast<volatile uint32_t *>(smem + tid * kTileBytes + kOffDirty) = 0;
    if (warp == 0) tmem_alloc(ptx::smem_u32(const_cast<uint32_t *>(&misc[0])), kN);  // 128 fp32 columns x 128 lanes
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = misc[0];
    const uint32_t my_panels = blockIdx.x < a.num_panels ? (a.num_panels - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    auto abort_now = [&]() {
        atomicExch(a.status, 3u);
        misc[1] = 1;
    };

    if (warp >= 4 && warp < 4 + kProducers) {
        // ================= producer warps: TMA gathers, kStages ahead =================
        const uint32_t pw = warp - 4;  // this warp issues the steps i with i % kProducers == pw
        // The column lists and record offsets of this block's panels are themselves fetched by TMA into a
        // double-buffered shared-memory area, one segment (<= kMetaSlots step slots) ahead of their use, so
        // the warp never waits on a global load while it issues: per step lanes 0-7 start the copies of the
        // eight gathered rows and lane 8 announces the byte count and starts the copy of the record.
        uint64_t *meta_full = reinterpret_cast<uint64_t *>(smem + kOffMeta + 2 * kMetaBytes), *meta_free = meta_full + 2;
        auto load_range = [&](uint32_t o, uint32_t &k0, uint32_t &k1) {
            k0 = k1 = 0;
            if (o < a.num_panels) {
                k0 = __ldg(a.panel_first + o);
                k1 = __ldg(a.panel_last + o);
            }
        };
        const float *Bn = a.B + n0;
        const uint32_t ldb32 = (uint32_t)a.ldb;
        // segment generator: walks this block's panels, cutting each into segments of <= kMetaSlots slots
        uint32_t g_ord = blockIdx.x, g_k, g_k1, r1_k0, r1_k1, r2_k0, r2_k1;
        load_range(g_ord, g_k, g_k1);
        load_range(g_ord + gridDim.x, r1_k0, r1_k1);
        load_range(g_ord + 2 * gridDim.x, r2_k0, r2_k1);
        uint32_t fetched = 0;  // segments whose metadata fetch has been started
        auto fetch_next = [&](uint32_t &seg_begin, uint32_t &seg_end) {  // returns false when there is no further segment
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
            if (g_k >= g_k1) {  // panel exhausted: move to this block's next panel (its range was loaded two panels ago)
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
                const uint32_t col = mcols[(k - cur_b) * 8 + (lane & 7)];
                const uint32_t o0 = moffs[k - cur_b], o1 = moffs[k - cur_b + 1];
                ok = ptx::mbar_wait(&sfree[s], ((issued / kStages) & 1u) ^ 1u);  // the landing stage has been consumed
                if (!ok) break;
                unsigned char *st = smem + kStage0 + s * kStageBytes;
                if (lane == 8) {
                    ptx::mbar_expect_tx(&full[s], 8u * kN * 4u + (o1 - o0) * 16u);
                    ptx::bulk_g2s(st + kOffRec, a.recs + (size_t)o0 * 4, (o1 - o0) * 16u, &full[s]);
                } else if (lane < 8) {
                    ptx::bulk_g2s(st + lane * kBStride * 4, Bn + (uint64_t)col * ldb32, kN * 4u, &full[s]);
                }
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&meta_free[m]);  // this warp is done with the segment's metadata
            if (!ok) {
                if (lane == 0) abort_now();
                break;
            }
            ++seg;
            cur_b = nxt_b; cur_e = nxt_e;
            have_cur = have_nxt;
        }
    } else if (warp == 4 + kProducers) {
        // ================= MMA warp: one thread issues every tcgen05.mma of the block =================
        if (lane == 0) {
            uint32_t step = 0;
            for (uint32_t p = 0; p < my_panels && !misc[1]; ++p) {
                // the previous panel's accumulator must have been read before it is overwritten
                if (p > 0 && !ptx::mbar_wait(drained, (p - 1) & 1u)) { abort_now(); break; }
                bool first = true;
                for (;;) {
                    const int s = step % kTiles;
                    const bool okm = ptx::mbar_wait(&built[s], (step / kTiles) & 1u);
                    if (!okm) { abort_now(); break; }
                    tc_fence_after();
                    unsigned char *st = smem + s * kTileBytes;
                    const uint32_t last = misc[2 + s];
                    tc_mma_tf32(tmem, smem_desc(ptx::smem_u32(st + kOffA), 128u, 256u), smem_desc(ptx::smem_u32(st + kOffB), 128u, 256u),
                                kIdesc, first ? 0u : 1u);
                    tc_commit(&mma_done[s]);
                    if (last) tc_commit(panel_done);
                    first = false;
                    ++step;
                    if (last) break;
                }
            }
        }
    } else {
        // ================= builder warps 0-3: operand tiles, then the accumulator read-back =================
        // Step i is built by warp i & 3 into tile pair i & 3 (its own), so four steps are under construction
        // at once; every warp still looks at every step's record header to follow the panel structure.
        uint32_t step = 0;
        for (uint32_t p = 0; p < my_panels && !misc[1]; ++p) {
            uint32_t panel_idx = 0;
            for (;;) {
                const int ls = step % kStages, t = step & 3;
                unsigned char *land = smem + kStage0 + ls * kStageBytes;  // gathered rows + record
                const bool ok1 = ptx::mbar_wait(&full[ls], (step / kStages) & 1u);  // rows of B and record have landed
                if (!ok1) {
                    if (lane == 0) abort_now();
                    break;
                }
                const uint32_t *rec = reinterpret_cast<const uint32_t *>(land + kOffRec);
                const uint32_t head = rec[0];
                const uint32_t last = (head >> 16) & 1u, cnt = head & 0xffffu;
                panel_idx = rec[1];
                if (warp == t) {
                    unsigned char *st = smem + t * kTileBytes;  // this warp's operand tiles
                    // the MMA that read these tiles four steps ago must be done
                    const bool ok2 = ptx::mbar_wait(&mma_done[t], ((step >> 2) & 1u) ^ 1u);
                    if (!ok2) {
                        if (lane == 0) abort_now();
                        break;
                    }
                    // ---- B: column n of the gathered rows -> one 32-byte row of the K-major operand ----
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int n = lane + 32 * q;
                        const float *col = reinterpret_cast<const float *>(land) + n;
                        float x[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            x[k] = col[k * kBStride];
                            if (ROUND_B) x[k] = __uint_as_float(ptx::f32_to_tf32_rna(x[k]));
                        }
                        float4 *d = reinterpret_cast<float4 *>(st + kOffB + (n >> 3) * 256 + (n & 7) * 16);
                        d[0] = make_float4(x[0], x[1], x[2], x[3]);
                        d[8] = make_float4(x[4], x[5], x[6], x[7]);  // + 128 bytes
                    }
                    // ---- A: clear the rows written the last time, write this step's ----
                    volatile uint32_t *dirty_cnt = reinterpret_cast<volatile uint32_t *>(st + kOffDirty);
                    unsigned char *dirty_rows = st + kOffDirty + 16;
                    const uint32_t old = *dirty_cnt;
                    for (uint32_t e = lane; e < old; e += 32) {
                        const uint32_t r = dirty_rows[e];
                        float4 *d = reinterpret_cast<float4 *>(st + kOffA + (r >> 3) * 256 + (r & 7) * 16);
                        d[0] = make_float4(0.f, 0.f, 0.f, 0.f);
                        d[8] = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    __syncwarp();
                    const uint32_t *entries = rec + kSlabRecHeaderWords;
                    const float *vals = reinterpret_cast<const float *>(entries + (cnt + 3) / 4 * 4);
                    for (uint32_t e = lane; e < cnt; e += 32) {
                        const uint32_t ent = entries[e];
                        const uint32_t r = ent & 0xffu, mask = (ent >> 8) & 0xffu;
                        const float *v0 = vals + (ent >> 16);
                        float v[8];
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const float x = ((mask >> c) & 1u) ? v0[__popc(mask & ((1u << c) - 1u))] : 0.f;
                            v[c] = __uint_as_float(ptx::f32_to_tf32_rna(x));
                        }
                        float4 *d = reinterpret_cast<float4 *>(st + kOffA + (r >> 3) * 256 + (r & 7) * 16);
                        d[0] = make_float4(v[0], v[1], v[2], v[3]);
                        d[8] = make_float4(v[4], v[5], v[6], v[7]);
                        dirty_rows[e] = (unsigned char)r;
                    }
                    if (lane == 0) {
                        *dirty_cnt = cnt;
                        misc[2 + t] = last;
                    }
                    ptx::fence_async_smem();  // the tensor core reads the tiles through the async proxy
                    __syncwarp();
                    if (lane == 0) {
                        ptx::mbar_arrive(&built[t]);
                        ptx::mbar_arrive(&sfree[ls]);
                    }
                } else {
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&sfree[ls]);  // this warp only needed the header
                }
                ++step;
                if (last) break;
            }
            if (misc[1]) break;
            // ---- end of panel: accumulator -> C (this warp's 32 rows) ----
            const bool ok3 = ptx::mbar_wait(panel_done, p & 1u);
            if (!ok3) {
                if (lane == 0) abort_now();
                break;
            }
            tc_fence_after();
            const uint64_t r = (uint64_t)panel_idx * kSlabRows + tid;
            float *crow = a.C + r * a.ldc + n0;
#pragma unroll 1
            for (int ch = 0; ch < 8; ++ch) {
                uint32_t v[16];
                tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + ch * 16, v);
                if (r < a.M) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        __stcs(reinterpret_cast<float4 *>(crow + ch * 16 + j * 4),
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
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(spmm_slab_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(spmm_slab_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    // three blocks per SM: 3 x 62 KB of shared memory, 3 x 128 of the 512 columns of tensor memory
    uint32_t blocks = (uint32_t)sm_count * SLAB_BLOCKS_PER_SM;
    if (blocks > a.num_panels) blocks = a.num_panels;
    const dim3 grid(blocks, a.N / kN);
    if (a.round_b) spmm_slab_kernel<true><<<grid, kThreads, kSmemBytes, s>>>(a);
    else spmm_slab_kernel<false><<<grid, kThreads, kSmemBytes, s>>>(a);
    return cudaGetLastError();
}

}  // namespace cutespmm
