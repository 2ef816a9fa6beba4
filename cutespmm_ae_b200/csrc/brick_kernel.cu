// Tensor-core brick kernel: the path for row panels whose 16x8 bricks are full enough that a dense
// contraction (zeros included) costs less than gathering a row of B per nonzero.
//
// It takes the place of SpMM<NUM_WARPS,ILP_LEVEL> + COMPUTE<ILP> (reference kernel.cu:16-288).
// What is kept: 16-row panels, active-column compaction, TF32 inputs rounded to nearest (cvt.rna,
// kernel.cu:28-35) with fp32 accumulation.  What is different:
//   * a brick's values are stored already in MMA fragment order, zeros included (544-byte records),
//     instead of a bitmap plus packed values expanded by popcounts (kernel.cu:20-27): the kernel is
//     bound by instruction latency, not by bytes, and the expansion was a sixth of its instructions;
//   * every warp is an autonomous pipeline over its own sequence of panels (panels are dealt
//     round-robin over the warps of the grid); it owns a ring of kStages shared-memory stages and
//     one mbarrier per stage.  The reference
//     drains a depth-2 cp.async pipeline and runs __syncthreads after every block of 16 columns
//     (kernel.cu:220-222); here no two warps ever wait for each other;
//   * the eight gathered rows of B of a brick arrive by two TMA gather4 loads (four rows of the slab
//     each, through a tensor map over B), the brick's record by a bulk copy; the
//     copies for brick k + kStages - 1 are issued before brick k is computed, across panel
//     boundaries, so the gather latency is hidden without occupancy;
//   * a brick is 16 x 8 and maps onto mma.m16n8k8 (the reference issues m16n8k4 on 16 x 4 bricks);
//     a warp covers the whole 128-column slab (16 accumulator tiles), so a brick is expanded once,
//     not once per warp of a block;
//   * B rows sit in shared memory with a stride of SLAB + 8 floats (the box of the tensor map is that
//     wide; its last 8 columns are padding, filled without touching memory when they lie beyond N),
//     which makes the B-fragment reads (lane (g,t) reads B[t][g], B[t+4][g]) hit 32 different banks.
//     (Reading four tiles' fragments with one 128-bit load was measured slower: the register pairs
//     the MMA wants then cost two moves per MMA.)
//   * the work list is cut by brick count (nnz balance), not by a per-GPU occupancy table.
#include <cuda_runtime.h>

#include <cstdint>

#include "device_plan.hpp"
#include "plan.hpp"
#include "ptx.cuh"
#include "tmap.hpp"

namespace cutespmm {

namespace {

constexpr int kStages = 3;
constexpr int kRecWords = kBrickRecWords;  // header + a full brick of values

template <int NT> struct StageLayout {
    static constexpr int kSlab = 8 * NT;         // columns of B / C a warp covers
    static constexpr int kStride = kSlab + 8;    // floats between consecutive B rows in shared memory
    static constexpr int kBBytes = 8 * kStride * 4;
    static constexpr int kHalfBytes = 4 * kStride * 4;  // what one gather4 load writes
    static constexpr int kStageBytes = kBBytes + kRecWords * 4;  // a warp's region: the B tiles of its stages, then their records
    // a warp's region: its stages, then its mbarriers; rounded so the next warp's stages stay 128-byte aligned
    static constexpr int kWarpBytes = (kStages * kStageBytes + kStages * 8 + 127) / 128 * 128;
    static_assert(kBBytes % 128 == 0 && kHalfBytes % 128 == 0 && (kRecWords * 4) % 16 == 0, "gather4 destinations must be 128-byte aligned");
    static_assert(kStride % 32 == 8, "the B-fragment reads are conflict-free only with this stride");
};

// ROUND_B: round the elements of B to tf32 to nearest (cvt.rna, what the reference does,
// kernel.cu:35) instead of letting the tensor core drop the low 13 mantissa bits.
// MULTI: the product is wider than one slab of columns (the single-slab kernel carries none of the slab bookkeeping).
template <int NT, bool ROUND_B, bool MULTI>
__global__ void __launch_bounds__(kBrickWarps * 32, 1) spmm_brick_kernel(const __grid_constant__ CUtensorMap tmap_b, BrickArgs a)
{
    using L = StageLayout<NT>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    // Panels are dealt round-robin over all warps of the grid: at any moment the grid works on one
    // contiguous window of the matrix, so a row of B that several panels share is fetched from HBM
    // once and found in L2 by the others.  Warp w of block b is number w * gridDim.x + b in that deal
    // (not b * warps + w): the last, part-filled round then lands on a few warps of every SM instead of
    // on all warps of the first SMs, and takes its share of a round's time instead of two thirds of one
    // (stencil512 0.0700 -> 0.0676 ms, elasticity40 0.0720 -> 0.0679 ms at N = 128).
    const uint32_t W = gridDim.x * kBrickWarps;
    uint32_t ord = warp * gridDim.x + blockIdx.x;  // this warp's current panel (ordinal among brick panels)
    if (ord >= a.num_panels) return;  // warps never synchronise with each other, so leaving early is safe
    // A product wider than one slab of L::kSlab columns walks every panel once per slab, slab after slab, before it moves
    // to its next panel: the panel's records and column lists are then found in L2 by the second walk, and one grid of
    // persistent blocks covers all slabs.
    const uint32_t slabs = MULTI ? a.N / L::kSlab : 1u;

    unsigned char *mine = smem_raw + (size_t)warp * L::kWarpBytes;
    uint64_t *full = reinterpret_cast<uint64_t *>(mine + kStages * L::kStageBytes);
    auto stage_b = [&](int s) { return reinterpret_cast<float *>(mine + s * L::kBBytes); };
    auto stage_rec = [&](int s) { return reinterpret_cast<uint32_t *>(mine + kStages * L::kBBytes + s * (kRecWords * 4)); };
    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) ptx::mbar_init(&full[s], 1);
        ptx::fence_mbar_init();
    }
    __syncwarp();

    // ---- producer state --------------------------------------------------------------------------
    // Metadata travels in groups of 4 brick slots: lane 2j+h (lanes 0..7) holds columns 4h..4h+3 of
    // slot j (records need none: slot k's record is at word k * kRecWords).  A panel starts on a group
    // boundary.  Loaded ahead of use: the next group of the current panel, the first group of the
    // warp's next panel, and the slot range of the panel after that.
    auto load_cols = [&](uint32_t g) {
        return lane < 8 ? __ldg(reinterpret_cast<const uint4 *>(a.cols + (size_t)g * 32) + lane) : make_uint4(0, 0, 0, 0);
    };
    auto load_range = [&](uint32_t o, uint32_t &k0, uint32_t &k1) {
        k0 = k1 = 0;
        if (o < a.num_panels) {
            k0 = __ldg(a.panel_first + o);
            k1 = __ldg(a.panel_last + o);
        }
    };
    uint32_t pk, pk_end;  // producer cursor: next slot to issue, end of its panel
    load_range(ord, pk, pk_end);
    uint32_t p_k0 = pk;   // first slot of the producer's panel (walked again for the next slab)
    uint32_t p_slab = 0, c_slab = 0;  // column slab of the producer cursor / of the brick being consumed
    uint32_t G = pk >> 2;
    uint4 mc_cur = load_cols(G), mc_nxt = load_cols(G + 1);
    uint32_t n_k0, n_k1, nn_k0, nn_k1;  // slot ranges of the next panel and the one after (k0 == k1: none)
    load_range(ord + W, n_k0, n_k1);
    load_range(ord + 2 * W, nn_k0, nn_k1);
    uint4 n_mc = load_cols(n_k0 >> 2);
    uint32_t p_ord = ord;            // panel ordinal of the producer cursor
    uint32_t issued = 0, done = 0;   // bricks issued / consumed by this warp so far
    int is = 0, ds = 0;              // ring positions of the next brick to issue / to consume
    uint32_t dpar = 0;               // mbarrier phase parity of stage ds

    auto producer_has_work = [&]() { return pk < pk_end; };
    auto issue_one = [&]() {  // start the copies of slot pk into stage issued % kStages, then advance the cursor
        const uint32_t k = pk;
        if ((k >> 2) != G) {
            ++G;
            mc_cur = mc_nxt;
            mc_nxt = load_cols(G + 1);
        }
        const int s = is;
        is = (is + 1 == kStages) ? 0 : is + 1;
        // lane 8 starts the copy of the record; lanes 2j and 2j+1, which hold the columns of slot j = k & 3,
        // start one gather4 load of four rows of B each straight from their registers
        const uint32_t j = k & 3;
        if (lane == 8) {
            ptx::mbar_expect_tx(&full[s], (uint32_t)L::kBBytes + kRecWords * 4u);
            ptx::bulk_g2s(stage_rec(s), a.recs + (size_t)k * kRecWords, kRecWords * 4u, &full[s]);
        }
        if ((uint32_t)(lane >> 1) == j)
            ptx::tma_gather4(reinterpret_cast<unsigned char *>(stage_b(s)) + (lane & 1) * L::kHalfBytes, &tmap_b, (int)(MULTI ? p_slab * L::kSlab : 0u), (int)mc_cur.x,
                             (int)mc_cur.y, (int)mc_cur.z, (int)mc_cur.w, &full[s]);
        ++issued;
        if (MULTI && pk + 1 == pk_end && p_slab + 1 < slabs) {  // panel finished for this slab: the same panel again, next slab
            ++p_slab;
            pk = p_k0;
            G = pk >> 2;
            mc_cur = load_cols(G);
            mc_nxt = load_cols(G + 1);
        } else if (++pk == pk_end) {  // panel finished: move the cursor to the warp's next panel
            p_slab = 0;
            p_ord += W;
            pk = n_k0;
            pk_end = n_k1;
            p_k0 = pk;
            G = pk >> 2;
            mc_cur = n_mc;
            n_k0 = nn_k0;
            n_k1 = nn_k1;
            if (pk < pk_end) {
                mc_nxt = load_cols(G + 1);
                n_mc = load_cols(n_k0 >> 2);
                load_range(p_ord + 2 * W, nn_k0, nn_k1);
            }
        }
    };

    // mma.m16n8k8 row-major A: lane (g,t) holds a0 = A[g][t], a1 = A[g+8][t], a2 = A[g][t+4], a3 = A[g+8][t+4]
    const int g = lane >> 2, t = lane & 3;

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

    for (int s0 = 1; s0 < kStages && producer_has_work(); ++s0) issue_one();  // fill the ring
    for (;;) {
        if (producer_has_work() && issued < done + kStages) issue_one();
        if (done == issued) break;  // nothing in flight and nothing left to issue
        const int s = ds;
        if (!ptx::mbar_wait(&full[s], dpar)) {
            if (lane == 0) atomicExch(a.status, 2u);  // the copies never landed: report, do not hang
            // give the copies still in flight a bounded chance to land before the shared memory is reused
            for (uint32_t j = done + 1; j < issued; ++j) ptx::mbar_wait(&full[j % kStages], (j / kStages) & 1u);
            return;
        }
        if (++ds == kStages) {
            ds = 0;
            dpar ^= 1u;
        }
        const uint32_t *rec = stage_rec(s);
        const uint2 info = *reinterpret_cast<const uint2 *>(rec + 4);
        const float4 a4 = *reinterpret_cast<const float4 *>(rec + kBrickRecHeaderWords + 4 * lane);  // this lane's fragment, zeros included
        uint32_t af[4];
        af[0] = ptx::f32_to_tf32_rna(a4.x);
        af[1] = ptx::f32_to_tf32_rna(a4.y);
        af[2] = ptx::f32_to_tf32_rna(a4.z);
        af[3] = ptx::f32_to_tf32_rna(a4.w);
        const float *b_lo = stage_b(s) + t * L::kStride + g, *b_hi = b_lo + 4 * L::kStride;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            uint32_t bf[2];
            bf[0] = ROUND_B ? ptx::f32_to_tf32_rna(b_lo[nt * 8]) : __float_as_uint(b_lo[nt * 8]);
            bf[1] = ROUND_B ? ptx::f32_to_tf32_rna(b_hi[nt * 8]) : __float_as_uint(b_hi[nt * 8]);
            ptx::mma_m16n8k8_tf32(acc[nt], af, bf);
        }
        if (info.x & 1u) {  // last brick of the panel: write its 16 x SLAB tile of C
            const uint64_t r_lo = (uint64_t)info.y * kPanelRows + g, r_hi = r_lo + 8;
            // a reordered plan writes every row to its place in the caller's C
            const uint64_t o_lo = a.row_map && r_lo < a.M ? __ldg(a.row_map + r_lo) : r_lo, o_hi = a.row_map && r_hi < a.M ? __ldg(a.row_map + r_hi) : r_hi;
            const uint32_t n0 = MULTI ? c_slab * L::kSlab : 0u;
            if (MULTI) c_slab = c_slab + 1 == slabs ? 0 : c_slab + 1;
            float *c_lo = a.C + o_lo * a.ldc + n0 + 2 * t, *c_hi = a.C + o_hi * a.ldc + n0 + 2 * t;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                if (r_lo < a.M) __stcs(reinterpret_cast<float2 *>(c_lo + nt * 8), make_float2(acc[nt][0], acc[nt][1]));
                if (r_hi < a.M) __stcs(reinterpret_cast<float2 *>(c_hi + nt * 8), make_float2(acc[nt][2], acc[nt][3]));
                acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
            }
        }
        ++done;
        __syncwarp();  // every lane is done with stage s before the next iteration refills it
    }
}

template <int NT, bool ROUND_B> cudaError_t launch_brick_t(const BrickArgs &a, int sm_count, cudaStream_t s)
{
    using L = StageLayout<NT>;
    constexpr int smem = kBrickWarps * L::kWarpBytes;
    const bool multi = a.N > (uint32_t)L::kSlab;
    cudaError_t e = multi ? allow_dynamic_smem<spmm_brick_kernel<NT, ROUND_B, true>>(smem) : allow_dynamic_smem<spmm_brick_kernel<NT, ROUND_B, false>>(smem);
    if (e != cudaSuccess) return e;
    uint32_t blocks = (a.num_panels + kBrickWarps - 1) / kBrickWarps;
    if (blocks > (uint32_t)sm_count) blocks = (uint32_t)sm_count;  // one resident block per SM, persistent
    // B as a 2-D tensor; the box is the slab plus the 8 columns of padding that give the shared-memory stride
    CUtensorMap tmap;
    e = make_b_tensor_map(&tmap, a.B, a.N, a.K, a.ldb, L::kStride, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (e != cudaSuccess) return e;
    if (multi) spmm_brick_kernel<NT, ROUND_B, true><<<blocks, kBrickWarps * 32, smem, s>>>(tmap, a);
    else spmm_brick_kernel<NT, ROUND_B, false><<<blocks, kBrickWarps * 32, smem, s>>>(tmap, a);
    return cudaGetLastError();
}

}  // namespace

bool brick_supports(uint32_t N, uint64_t ldb, uint64_t ldc, const void *B, const void *C)
{
    const uintptr_t pb = reinterpret_cast<uintptr_t>(B), pc = reinterpret_cast<uintptr_t>(C);
    return N % 32 == 0 && N > 0 && !((pb | pc) & 15) && !((ldb | ldc) & 3);
}

cudaError_t launch_brick(const BrickArgs &a, int sm_count, cudaStream_t s)
{
    if (a.num_bricks == 0 || a.num_panels == 0) return cudaSuccess;
    if (a.round_b) {
        if (a.N % 128 == 0) return launch_brick_t<16, true>(a, sm_count, s);
        if (a.N % 64 == 0) return launch_brick_t<8, true>(a, sm_count, s);
        return launch_brick_t<4, true>(a, sm_count, s);
    }
    if (a.N % 128 == 0) return launch_brick_t<16, false>(a, sm_count, s);
    if (a.N % 64 == 0) return launch_brick_t<8, false>(a, sm_count, s);
    return launch_brick_t<4, false>(a, sm_count, s);
}

}  // namespace cutespmm
