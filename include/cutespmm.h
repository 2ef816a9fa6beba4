/*
 * libcutespmm -- C ABI of the B200 (sm_100a) sparse x dense product
 *
 *        C[M x N] = A_sparse[M x K] * B_dense[K x N]
 *
 * fp32 storage, fp32 accumulation.  Row-major B and C with leading dimensions.
 * This is the boundary a host program binds instead of the reference project's
 * header-included classes; every entry point names the reference interface it
 * replaces (file:line inside aFatCa/cuTeSpMM_AE).
 *
 * Conventions
 *   - every function returns a cutespmm_status_t (0 = success, negative = error)
 *     and never exits or aborts the process (the reference's chkerr, inc.h:61-69,
 *     calls exit(-1));  cutespmm_last_error() gives the message of the calling
 *     thread's last failure;
 *   - host arrays are borrowed for the duration of the call only;
 *   - device pointers refer to the CUDA device that was current when the plan
 *     was created; all GPU work is ordered on the stream the caller passes
 *     (a cudaStream_t cast to void*, NULL = the legacy default stream the
 *     reference uses, spmm.cu:171-174);
 *   - cutespmm_spmm performs no allocation: the scratch it needs belongs to
 *     the plan.
 */
#ifndef CUTESPMM_H
#define CUTESPMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    CUTESPMM_OK = 0,
    CUTESPMM_EINVAL = -1,       /* bad argument: null pointer, index out of range, misaligned buffer */
    CUTESPMM_ENOMEM = -2,       /* host or device allocation failed */
    CUTESPMM_ECUDA = -3,        /* a CUDA runtime call or kernel launch failed (no device, ...) */
    CUTESPMM_EUNSUPPORTED = -4, /* valid request outside what this build handles */
    CUTESPMM_EIO = -5,          /* file could not be read or parsed */
    CUTESPMM_ETIMEOUT = -6,     /* a bounded device-side wait ran out (reported through the plan's status word) */
    CUTESPMM_ECOMM = -7         /* the communication library is missing or one of its calls failed */
} cutespmm_status_t;

/* Which kernel family executes a plan. */
typedef enum {
    CUTESPMM_PATH_AUTO = 0,  /* per-panel choice by brick density */
    CUTESPMM_PATH_ROWS = 1,  /* CUDA-core row-gather kernel for every row */
    CUTESPMM_PATH_BRICK = 2, /* tensor-core brick kernel (mma.sync, 16-row panels) for every panel */
    CUTESPMM_PATH_SLAB = 3   /* tensor-core slab kernel (tcgen05/TMEM, 128-row panels) for every panel; N must be a
                                multiple of 128, other N run on the row kernel */
} cutespmm_path_t;

/* Tensor-core path: A is always rounded to TF32 to nearest (cvt.rna, as the reference does,
 * kernel.cu:28-29).  By default the elements of B reach the tensor core as fp32 bit patterns whose low
 * 13 mantissa bits it ignores (truncation; measured relative Frobenius error about 4.5e-4 against the
 * fp32 CPU product).  With this flag B is rounded to nearest as well (kernel.cu:35; about 2.5e-4) at
 * the cost of one conversion per element of every gathered row.  Truncation is one-sided: on operands of
 * one sign the errors of a row do not cancel and the result comes out low by the mean truncation loss,
 * measured 3.6e-4 relative (brick and slab path alike; 8.5e-5 with this flag) -- still inside the 1e-3
 * the tensor-core paths state, with less margin than zero-mean data suggests.  Not available on CUTESPMM_PATH_SLAB, where
 * the copy engine places B in the tensor core's operand layout and no thread touches it. */
#define CUTESPMM_FLAG_ROUND_B_NEAREST 1u

/* Plan-time row reordering.  The reference's harness expects reordered inputs to come from outside (it parses the
 * names of reordered / split matrix files, gpu_kernels.cu:945-1047, and measures block affinity, :1049-1186) and
 * its CSR class carries the pairwise row similarity such a stage would use (inc/CSR.hpp:612-679).  Here the stage
 * is part of the plan: rows are processed in an order that puts rows with similar column sets into the same
 * 16-row panel -- rows sorted by their leading column indices, the cheap form of "most similar row next" -- so a
 * matrix whose rows arrive in a poor order still fills tensor-core bricks and shares rows of B inside a panel.  Only
 * the order of processing changes: B and C keep the caller's row order (every row of C is written to its own
 * place), and the panel views describe the reordered matrix.  Host builder only. */
typedef enum {
    CUTESPMM_REORDER_NONE = 0,
    CUTESPMM_REORDER_CLUSTER_ROWS = 1,  /* rows sorted by their leading column indices: one sort, restores a good order
                                           that was lost (shuffled input) */
    CUTESPMM_REORDER_SIMILAR_ROWS = 2   /* every 16-row panel grown greedily: the next row is the unplaced row that shares
                                           the most columns with the panel so far (the reference's row_simlarity /
                                           find_most_similar idea, inc/CSR.hpp:612-679, made linear-time through the
                                           column-to-rows index).  Panels become compact patches of the matrix graph, so
                                           they name fewer distinct rows of B than 16 consecutive rows do */
} cutespmm_reorder_t;

typedef struct {
    uint32_t struct_size; /* sizeof(cutespmm_options_t), for forward compatibility */
    uint32_t path;        /* cutespmm_path_t */
    uint32_t split_nnz;   /* rows longer than this are cut into chunks of this many nonzeros (at most 384) */
    uint32_t tile_nnz;    /* cost (nonzeros + 4 per row) a thread block takes per scheduling tile */
                          /* Both 0 (the default): 256 / 512 for large jobs; a job below about 2 M nonzeros gets tiles for
                             one resident wave, rows cut from max(128, cost/8192) nonzeros on and cut rows in pieces of
                             sqrt(length/2).  One of them 0: that one takes its large-job default. */
    float brick_density;  /* AUTO: panels whose 16x8 bricks are at least this full go to the brick kernel (0 = default) */
    uint32_t flags;       /* CUTESPMM_FLAG_* */
    uint32_t reorder;     /* cutespmm_reorder_t */
    uint32_t min_brick_panels; /* AUTO: with fewer dense panels than this, every panel goes to the row kernel (0 = default
                                  4440, two panels per warp of a full brick-kernel grid: below that most of its per-warp
                                  pipelines idle and a second launch for the other rows costs more than it saves) */
} cutespmm_options_t;

typedef struct {
    uint64_t M, K, nnz;
    uint64_t num_panels;      /* 16-row panels, ceil(M/16)                  (HRPB::numRowPanels, data.cu:60,87) */
    uint64_t num_blocks;      /* 16-column blocks of active columns          (blockedRowPtr[numRowPanels], data.cu:145) */
    uint64_t num_tiles;       /* scheduling tiles of the row kernel */
    uint64_t num_long_rows;   /* rows cut into chunks */
    uint64_t num_chunks;      /* chunks of long rows = rows of the partial-sum scratch */
    uint64_t brick_panels;    /* panels executed by the tensor-core kernel */
    uint64_t num_bricks;      /* non-empty 16x8 bricks in those panels */
    uint64_t device_bytes;    /* device memory the plan owns */
    uint64_t scratch_bytes_per_col; /* scratch bytes per column of B (times N gives the partial-sum scratch) */
} cutespmm_plan_info_t;

typedef struct cutespmm_plan cutespmm_plan_t;

const char *cutespmm_status_string(int status);
const char *cutespmm_last_error(void);
/* major*10000 + minor*100 + patch */
int cutespmm_version(void);

/* ---- preprocessing -------------------------------------------------------------------------
 * Replaces HRPB::HRPB / HRPB::DATASTRUCT (data.cu:80-335) and SPMM_TC::partition
 * (spmm.cu:691-822): builds the device-resident form of A and the nnz-balanced work list and
 * uploads both to the current CUDA device.  rowPtr has M+1 entries; cols/vals have rowPtr[M].
 * Column indices may be in any order inside a row (the reference silently loses nonzeros when
 * they are not ascending); duplicates are kept as separate terms.  Indices >= K, a decreasing
 * rowPtr, or rowPtr[M] >= 2^32 are rejected (EINVAL / EUNSUPPORTED).  opts may be NULL. */
int cutespmm_plan_create(cutespmm_plan_t **plan, uint64_t M, uint64_t K, const uint64_t *rowPtr,
                         const uint32_t *cols, const float *vals, const cutespmm_options_t *opts);

/* Same, with the 32-bit row pointers MTX_READER produces (IO.cu:7,32) and HRPB takes (data.cu:80). */
int cutespmm_plan_create_u32(cutespmm_plan_t **plan, uint32_t M, uint32_t K, const uint32_t *rowPtr,
                             const uint32_t *cols, const float *vals, const cutespmm_options_t *opts);

/* Host-only build of the same plan: no CUDA call is made and the plan cannot execute.  For
 * inspecting the work list and the packed format on a machine without a GPU. */
int cutespmm_plan_build_host(cutespmm_plan_t **plan, uint64_t M, uint64_t K, const uint64_t *rowPtr,
                             const uint32_t *cols, const float *vals, const cutespmm_options_t *opts);

/* A plan for a matrix that already lives on the device (rowPtr: M+1 x u32, cols: nnz x u32, vals: nnz x f32, all
 * device pointers): the nonzeros are packed by a kernel and never visit the host; only the row pointers do, because
 * the work lists are cut from them.  The reference preprocesses on the host only (data.cu:80-335) and its caller
 * uploads the result (data.cu:318-333); this is the entry point for a caller that has no host copy.  The plan runs
 * on the row kernel (opts->path auto or rows; brick and slab need the host builder's column analysis and are refused
 * with CUTESPMM_EUNSUPPORTED); rows need not be sorted.  The panel views (blocked_row_ptr, active_cols) are not
 * available for such a plan; plan_decode_csr reads the packed nonzeros back.  Work is queued on `stream`, which is
 * synchronised before the call returns (the column-range check is read back). */
int cutespmm_plan_create_device(cutespmm_plan_t **plan, uint64_t M, uint64_t K, const uint32_t *rowPtr_dev,
                                const uint32_t *cols_dev, const float *vals_dev, const cutespmm_options_t *opts,
                                void *stream);

/* Saves a plan to a file / loads it back (onto the current device, or host-only): preprocessing done once serves
 * later runs -- the reference preprocesses at every start (run.cu:17-20).  The file is specific to this library
 * version and byte order and carries a checksum; a damaged or foreign file is refused with CUTESPMM_EIO.  A loaded
 * plan behaves like the one that was saved (same kernels, bit-identical products). */
int cutespmm_plan_save(const cutespmm_plan_t *plan, const char *path);
int cutespmm_plan_load(cutespmm_plan_t **plan, const char *path, int host_only);

int cutespmm_plan_destroy(cutespmm_plan_t *plan);
int cutespmm_plan_info(const cutespmm_plan_t *plan, cutespmm_plan_info_t *info);

/* HRPB::blockedRowPtr (data.cu:65,145,176-185): prefix sum over 16-row panels of
 * ceil(distinct columns in the panel / 16).  out has num_panels+1 entries. */
int cutespmm_plan_blocked_row_ptr(const cutespmm_plan_t *plan, uint32_t *out);
/* HRPB::activeCols (data.cu:70,204-209): per panel its distinct columns ascending, zero-padded
 * to a multiple of 16.  out has num_blocks*16 entries. */
int cutespmm_plan_active_cols(const cutespmm_plan_t *plan, uint32_t *out);

/* Decodes the plan's packed form of A back to CSR (columns ascending inside a row, duplicates
 * merged in the brick part) -- the format round-trip check.  rowPtr: M+1, cols/vals: nnz. */
int cutespmm_plan_decode_csr(const cutespmm_plan_t *plan, uint64_t *rowPtr, uint32_t *cols, float *vals);

/* ---- execution -----------------------------------------------------------------------------
 * Replaces SPMM_TC::run (spmm.cu:823-839) and the kernel SpMM<NUM_WARPS,ILP_LEVEL>
 * (kernel.cu:119-288).  B: K x N device, row-major, leading dimension ldb >= N; C: M x N device,
 * ldc >= N.  Every row of C is written (rows without nonzeros become 0), so C needs no memset
 * (the reference relies on run.cu:43,49).  Any N >= 1.  The plan's device must be the current one
 * (CUTESPMM_EINVAL otherwise): a host that drives several GPUs calls cudaSetDevice before each plan. */
int cutespmm_spmm(const cutespmm_plan_t *plan, const float *B_dev, uint64_t ldb, float *C_dev,
                  uint64_t ldc, uint32_t N, void *stream);

/* Host-buffer call in the style of the reference driver loop (run.cu:38-53) and of its
 * float GPU_xxx(host pointers..., m, k, n, ...) wrappers (spmm.cu:860): copies B to the device,
 * runs the product, copies C back, ordered after the work already queued on `stream`, and waits
 * for it.  Large operands are pipelined in up to four column windows (copy-in, product and
 * copy-out on streams of the plan's own), so pinned host buffers let the two copy directions
 * overlap.  The device staging buffers belong to the plan and are (re)allocated only when N
 * grows.  kernel_ms (may be NULL) receives the device time of the products alone. */
int cutespmm_spmm_host(cutespmm_plan_t *plan, const float *B_host, uint64_t ldb, float *C_host,
                       uint64_t ldc, uint32_t N, void *stream, float *kernel_ms);

/* ---- SDDMM over the pattern of A ---------------------------------------------------------------
 * out[j] = (scale_by_values ? A_j : 1) * dot(X[row of j], Y[column of j]) for every stored nonzero j of the plan,
 * N columns wide.  The operator that accompanies SpMM in a graph layer (edge scores; the reference tree has it only
 * inside the TC-GNN baseline, TC-GNN_ATC23/TCGNN_conv/TCGNN.cpp:265 "forward_ef") and the gradient of C = A*B with
 * respect to the values of A (X = dC, Y = B).  X: M x N, Y: K x N, device, row-major.  out: nnz floats on the device,
 * in the plan's storage order: CSR order with the columns of a row ascending for a plan built on the host (the order
 * cutespmm_plan_decode_csr returns), the caller's own order for a plan built from device CSR.  fp32 throughout.
 * Not available for a plan with row reordering (CUTESPMM_EUNSUPPORTED). */
int cutespmm_sddmm(const cutespmm_plan_t *plan, const float *X_dev, uint64_t ldx, const float *Y_dev, uint64_t ldy, uint32_t N,
                   int scale_by_values, float *out_dev, void *stream);

/* New values for an unchanged pattern: vals_dev[j] becomes the value of nonzero j in the plan's storage order -- the
 * order cutespmm_sddmm writes its output in and cutespmm_plan_decode_csr returns -- so edge scores computed by
 * cutespmm_sddmm (and normalised by the caller) become the weights of the next product: the weighted / attention
 * aggregation of a graph layer (the reference tree carries it as the TC-GNN baseline's forward_AGNN,
 * TC-GNN_ATC23/TCGNN_conv/TCGNN.cpp:260-264).  One pass over the nonzeros on `stream`; products queued on the stream
 * afterwards see the new values.  For plans whose rows all run on the row kernel (path rows, or auto without dense
 * panels) and without row reordering; CUTESPMM_EUNSUPPORTED otherwise. */
int cutespmm_plan_set_values(cutespmm_plan_t *plan, const float *vals_dev, void *stream);

/* ---- product without any allocation ------------------------------------------------------------
 * No counterpart in the reference.  For callers that must not allocate device memory when they
 * call (all of HBM already belongs to the host framework's pool, a real-time loop that may not make
 * synchronising runtime calls, a fixed memory budget): they cannot create a plan, so they pass plain
 * CSR arrays that already live in device memory -- rowPtr (M+1 entries, rowPtr[M] = nnz), cols, vals
 * -- together with B and C, and get C = A * B computed in fp32 by the row kernel's method (a warp per
 * row, rows longer than CUTESPMM_NOALLOC_SPLIT_NNZ cut into chunks whose partial sums are added in a
 * fixed order).  The partial sums live in a CUTESPMM_NOALLOC_SCRATCH_BYTES array that is part of the
 * library image: every GPU that loads the library holds it until the process exits.  The call makes no
 * cudaMalloc/cudaFree and calls no allocating or synchronising routine: on the caller's stream it queues one
 * 16-byte cudaMemsetAsync (the counters its warps claim rows from, also part of the image) and up to three kernels.
 * Limits, checked before anything is launched (CUTESPMM_EUNSUPPORTED with a message otherwise):
 *   N <= CUTESPMM_NOALLOC_MAX_N   and   (2*ceil(nnz/SPLIT_NNZ) + 2) * roundup(N, 4) * 4 <= SCRATCH_BYTES
 *   (16.7 M nonzeros at N = 128).
 * All calls on a device share the scratch, which keeps the previous call's contents; nothing in it
 * needs clearing, but calls that overlap on the same GPU race on it -- keep them on one stream or
 * order them with events.  The first call on each device looks up the device addresses of the scratch and the
 * counters (cudaGetSymbolAddress) and the kernels' occupancy; make that first call outside any stream capture. */
#define CUTESPMM_NOALLOC_SCRATCH_BYTES (16u << 20)
#define CUTESPMM_NOALLOC_SPLIT_NNZ 1024u
#define CUTESPMM_NOALLOC_MAX_N 512u
int cutespmm_spmm_csr_noalloc(uint32_t M, uint32_t K, uint32_t nnz, const uint32_t *rowPtr_dev,
                              const uint32_t *cols_dev, const float *vals_dev, const float *B_dev, uint64_t ldb,
                              float *C_dev, uint64_t ldc, uint32_t N, void *stream);

/* Number of kernels one cutespmm_spmm call launches for this plan and N. */
int cutespmm_spmm_launch_count(const cutespmm_plan_t *plan, uint32_t N);

/* Which kernels those are: bit 0 the CUDA-core row kernel, bit 1 the tensor-core brick kernel, bit 2 the tcgen05 slab
 * kernel (16-byte aligned operands assumed).  A plan made with path auto runs products narrower than 64 columns on the
 * row kernel alone, whatever its panels look like: there a row kernel with several rows of A per warp is the faster. */
int cutespmm_spmm_kernels(const cutespmm_plan_t *plan, uint32_t N);

/* Status word the kernels of this plan write on a failed bounded wait (0 = none; 1 row kernel, 2 brick
 * kernel, 3 slab kernel).  Orders nothing: call after the stream has been synchronised.  A non-zero
 * word is cleared by the read, so it describes the launches since the previous read. */
int cutespmm_plan_device_status(const cutespmm_plan_t *plan, uint32_t *status);

/* ---- sharding ------------------------------------------------------------------------------
 * No counterpart in the reference (single GPU).  Cuts rows [0, M) into `nparts` contiguous
 * ranges of about equal cost (nonzeros + row_cost per row), every boundary a multiple of
 * `align_rows` (16 keeps row panels whole).  bounds has nparts+1 entries, bounds[0] = 0,
 * bounds[nparts] = M.  Each rank then builds a plan over its own rows and C stays row-sharded. */
int cutespmm_partition_rows(uint64_t M, const uint64_t *rowPtr, uint32_t nparts, uint32_t align_rows,
                            uint32_t row_cost, uint64_t *bounds);

/* ---- communicator and sharded execution ----------------------------------------------------
 * No counterpart in the reference (its driver, run.cu:8-72, runs one GPU).  Row panels are
 * independent, so a large matrix is cut by cutespmm_partition_rows, every rank (one GPU each: a
 * process, or a thread of one process) creates a plan over its own rows, and C stays row-sharded.
 * The one exchange of the path is B, which every rank needs in its own device memory; it travels
 * over NVLink through NCCL, which the library loads at run time (libnccl.so.2; no link dependency)
 * the first time a communicator is created.  No kernel of this library reads another GPU's memory.
 *
 * A communicator belongs to the CUDA device that was current when it was created; collective calls
 * on it must come from one thread at a time, in the same order on every rank. */
typedef struct cutespmm_comm cutespmm_comm_t;
#define CUTESPMM_COMM_ID_BYTES 128
/* Rank 0 obtains an id and hands it to the other ranks by any means (a file, MPI, a TCP store). */
int cutespmm_comm_unique_id(void *id_out /* CUTESPMM_COMM_ID_BYTES */);
/* One process per GPU: every rank calls this with the same id; collective. */
int cutespmm_comm_create(cutespmm_comm_t **comm, int nranks, int rank, const void *id);
/* One process, several GPUs: creates ndev communicators at once, comms[i] on devices[i] (NULL: 0..ndev-1). */
int cutespmm_comm_create_all(cutespmm_comm_t **comms, int ndev, const int *devices);
/* Wraps an ncclComm_t the caller already has (not destroyed by cutespmm_comm_destroy). */
int cutespmm_comm_adopt(cutespmm_comm_t **comm, void *nccl_comm, int nranks, int rank);
/* A communicator without a transport: collectives are recorded instead of executed.  For testing the
 * bookkeeping of the sharded calls on a machine without GPUs (see cutespmm_sharded_transfers). */
int cutespmm_comm_create_stub(cutespmm_comm_t **comm, int nranks, int rank);
/* The transfers a stub communicator was asked for since the last call of this function (same fields as
 * cutespmm_sharded_transfers); the record is emptied. */
int cutespmm_comm_stub_log(cutespmm_comm_t *comm, uint32_t max, int *roots, uint64_t *offsets, uint64_t *counts, uint32_t *n);
int cutespmm_comm_info(const cutespmm_comm_t *comm, int *nranks, int *rank);
int cutespmm_comm_destroy(cutespmm_comm_t *comm);

/* How B reaches every rank's memory before the product. */
typedef enum {
    CUTESPMM_B_RESIDENT = 0,    /* B_dev already holds all K rows on every rank: no exchange */
    CUTESPMM_B_FROM_ROOT = 1,   /* rank `root` holds B; one broadcast fills B_dev on the others */
    CUTESPMM_B_ROW_SHARDED = 2  /* rank r holds rows [b_bounds[r], b_bounds[r+1]) in place inside its K x N
                                   buffer B_dev (the C of a previous sharded product, a layer's output):
                                   one all-gather in place (equal slices) or one broadcast per slice */
} cutespmm_b_mode_t;

/* This rank's rows of C = A * B.  plan: built over this rank's rows; B_dev: K x N on this rank, rows
 * contiguous (ldb == N) unless the mode is RESIDENT; b_bounds: nranks+1 row bounds of B (ROW_SHARDED
 * only, else NULL); C_dev: this rank's rows of C.  The exchange and the product are queued on `stream`
 * and the call returns without waiting. */
int cutespmm_spmm_sharded(const cutespmm_plan_t *plan, cutespmm_comm_t *comm, int b_mode, int root, float *B_dev,
                          uint64_t ldb, const uint64_t *b_bounds, float *C_dev, uint64_t ldc, uint32_t N, void *stream);

/* The same from host buffers, in the style of cutespmm_spmm_host: rank r passes only its own slice of
 * B -- B_host_rows points at row b_bounds[r] of B, rows [b_bounds[r], b_bounds[r+1]) follow with leading
 * dimension ldb -- so every rank copies K/nranks rows over its own PCIe link, the slices are exchanged
 * over NVLink, and each rank copies its rows of C back to C_host.  Column windows pipeline copy-in,
 * exchange, product and copy-out.  comm == NULL (or one rank) with b_bounds == NULL is cutespmm_spmm_host.
 * Waits for completion.  kernel_ms / exchange_ms (may be NULL): device time of the products / exchanges. */
int cutespmm_spmm_sharded_host(cutespmm_plan_t *plan, cutespmm_comm_t *comm, const float *B_host_rows, uint64_t ldb,
                               const uint64_t *b_bounds, float *C_host, uint64_t ldc, uint32_t N, void *stream,
                               float *kernel_ms, float *exchange_ms);

/* Allocates now what cutespmm_spmm_host / cutespmm_spmm_sharded_host would allocate at their first call for N columns
 * (device staging for B and C, streams, events); `sharded` != 0 sizes it for a call with more than one rank.  A later
 * host-buffer call for the same or a smaller N then allocates nothing.
 * Needed by a process that drives several GPUs from several threads: a cudaMalloc -- and the first launch of a kernel
 * on a device, which loads its code -- synchronises with every device of the process, so it must not run on one thread
 * while another thread's collective kernel is already waiting for this thread to join (both would wait for ever).
 * Such a host reserves the staging and runs one local product per plan (cutespmm_spmm on resident data) before its
 * first collective; tests/cpp/sharded_driver.cpp does exactly that.  One process per GPU has no such coupling. */
int cutespmm_plan_reserve_host_staging(cutespmm_plan_t *plan, uint32_t N, int sharded);

/* The collectives a sharded call issues for one contiguous K x N block of B, in order: transfer i sends
 * count[i] floats starting at element offset[i] of the block from rank root[i] to every rank.  Returns the
 * number of transfers in *n (at most `max` are written).  Pure bookkeeping: works on a stub communicator. */
int cutespmm_sharded_transfers(const cutespmm_comm_t *comm, int b_mode, int root, uint64_t K, uint64_t N,
                               const uint64_t *b_bounds, uint32_t max, int *roots, uint64_t *offsets, uint64_t *counts,
                               uint32_t *n);

/* ---- MatrixMarket loader -------------------------------------------------------------------
 * Replaces MTX_READER (IO.cu:1-88).  pattern_only != 0 reproduces the reference exactly: every
 * value is 1.0 (IO.cu:68,81), M and K are padded up to multiples of 16 (IO.cu:30-31), a
 * "symmetric" header mirrors off-diagonal entries (IO.cu:16,42,77), entries keep file order
 * inside a row.  pattern_only == 0 keeps the file's values (SparseCoo behaviour,
 * inc/SparseCoo.hpp:91-157; 1.0 where the file has none). */
typedef struct cutespmm_mtx cutespmm_mtx_t;
int cutespmm_mtx_open(cutespmm_mtx_t **mtx, const char *path, int pattern_only);
int cutespmm_mtx_dims(const cutespmm_mtx_t *mtx, uint32_t *M, uint32_t *K, uint32_t *nnz);
/* Borrowed views valid until cutespmm_mtx_close (the fields MTX_READER exposes, IO.cu:4-9). */
int cutespmm_mtx_arrays(const cutespmm_mtx_t *mtx, const uint32_t **rowPtr, const uint32_t **cols,
                        const float **vals);
int cutespmm_mtx_close(cutespmm_mtx_t *mtx);

#ifdef __cplusplus
}
#endif
#endif /* CUTESPMM_H */
