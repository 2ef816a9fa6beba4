"""Parity of the CUDA path (called through the C ABI) with the CPU oracle, on a B200."""
import numpy as np
import pytest
import torch

import cutespmm_ae_b200 as cs
from cutespmm_ae_b200 import generators as g
from conftest import GOLDEN_CASES, REL_FRO_TOL, REL_FRO_TOL_FP32, load_golden

pytestmark = pytest.mark.gpu

PATHS = [cs.PATH_ROWS, cs.PATH_BRICK, cs.PATH_AUTO, cs.PATH_SLAB]
PATH_TOL = {cs.PATH_ROWS: REL_FRO_TOL_FP32, cs.PATH_BRICK: REL_FRO_TOL, cs.PATH_AUTO: REL_FRO_TOL, cs.PATH_SLAB: REL_FRO_TOL}


def run(plan, B_np, **kw):
    B = torch.from_numpy(np.ascontiguousarray(B_np)).cuda()
    C = torch.full((plan.M, B.shape[1]), float("nan"), device="cuda")  # every element must be overwritten
    plan.spmm(B, C, **kw)
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    return C.cpu().numpy()


@pytest.mark.parametrize("path", PATHS, ids=["rows", "brick", "auto", "slab"])
@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden_fixtures(oracle_mod, name, path):
    gd = load_golden(name)
    N = int(gd["N"])
    p = cs.Plan(int(gd["M"]), int(gd["K"]), gd["row_ptr"], gd["cols"], gd["vals"], path=path)
    C = run(p, gd["B"])
    assert oracle_mod.rel_fro(gd["C"], C) <= PATH_TOL[path]


@pytest.mark.parametrize("path", PATHS, ids=["rows", "brick", "auto", "slab"])
@pytest.mark.parametrize("workload,Ns", [("uniform4096", [32]), ("stencil512", [128]),
                                         ("elasticity40", [32, 64, 128, 256]), ("rmat20", [128])])
def test_named_workloads_match_oracle(oracle_mod, workload, Ns, path):
    if path == cs.PATH_SLAB and workload == "rmat20":
        pytest.skip("forcing a power-law graph through the dense 128-row path is covered at 2^11 nodes (test_slab_path_on_a_small_power_law_graph_and_rounding_modes); here it only costs time")
    w = g.WORKLOADS[workload]
    A = w["make"]()
    p = cs.Plan.from_csr(A, path=path)
    for N in Ns:
        B = g.dense_operand(A.K, N, w["b_seed"], w["b_dist"]).numpy()
        ref = oracle_mod.spmm_csr(A.row_ptr, A.cols, A.vals, B, A.M, A.K)
        C = run(p, B)
        err = oracle_mod.rel_fro(ref, C)
        assert err <= PATH_TOL[path], (workload, N, err)


@pytest.mark.parametrize("N", [1, 3, 4, 8, 12, 16, 20, 32, 33, 36, 48, 60, 64, 100, 128, 130, 200, 256, 384, 512, 516, 640, 1024])
def test_any_number_of_columns(oracle_mod, N):
    A = g.rmat(9, 8, seed=31, values="uniform")
    B = g.dense_operand(A.K, N, 32).numpy()
    p = cs.Plan.from_csr(A, path=cs.PATH_ROWS, split_nnz=32)
    assert p.info()["num_long_rows"] > 0
    ref = oracle_mod.spmm_csr(A.row_ptr, A.cols, A.vals, B, A.M, A.K)
    assert oracle_mod.rel_fro(ref, run(p, B)) <= REL_FRO_TOL_FP32


def test_slab_path_on_a_small_power_law_graph_and_rounding_modes(oracle_mod):
    A = g.rmat(11, 8, seed=33, values="uniform")  # wide 128-row panels, steps split at 256 values
    B = g.dense_operand(A.K, 256, 34).numpy()
    ref = oracle_mod.spmm_csr(A.row_ptr, A.cols, A.vals, B, A.M, A.K)
    e_slab = oracle_mod.rel_fro(ref, run(cs.Plan.from_csr(A, path=cs.PATH_SLAB), B))
    e_brick = oracle_mod.rel_fro(ref, run(cs.Plan.from_csr(A, path=cs.PATH_BRICK), B))
    e_round = oracle_mod.rel_fro(ref, run(cs.Plan.from_csr(A, path=cs.PATH_BRICK, round_b_nearest=True), B))
    assert e_round < e_brick <= REL_FRO_TOL and e_slab <= REL_FRO_TOL
    with pytest.raises(cs.CuteSpmmError) as e:  # B never passes a thread on the slab path, so it cannot be re-rounded
        cs.Plan.from_csr(A, path=cs.PATH_SLAB, round_b_nearest=True)
    assert e.value.status == -4


def test_same_sign_operands_keep_the_stated_bound_on_the_tensor_core_paths(oracle_mod):
    """All-positive A and B: the truncation of B to TF32 on the brick and slab paths is one-sided (every product comes
    out low, by up to 2^-10 of its value and 2^-11.5 on average over mantissas), so the errors of a row do not cancel.
    The stated bound (relative Frobenius 1e-3) must hold there too; rounding B to nearest removes the bias."""
    A0 = g.WORKLOADS["elasticity40"]["make"]()
    vals = A0.vals.abs() + 0.25
    B = (g.dense_operand(A0.K, 128, 52).abs() + 0.25).numpy()
    ref = oracle_mod.spmm_csr(A0.row_ptr, A0.cols, vals, B, A0.M, A0.K)
    rp, cols = A0.row_ptr.numpy(), A0.cols.numpy()
    errs = {}
    for name, kw in (("brick", dict(path=cs.PATH_BRICK)), ("slab", dict(path=cs.PATH_SLAB)),
                     ("brick_nearest", dict(path=cs.PATH_BRICK, round_b_nearest=True))):
        errs[name] = oracle_mod.rel_fro(ref, run(cs.Plan(A0.M, A0.K, rp, cols, vals.numpy(), **kw), B))
    print("same-sign operands, relative Frobenius error:", errs)
    assert errs["brick"] <= REL_FRO_TOL and errs["slab"] <= REL_FRO_TOL
    assert 2e-4 <= errs["brick"] <= 6e-4          # the bias itself: about 2^-11.5 = 3.5e-4
    assert errs["brick_nearest"] <= 0.5 * errs["brick"]


@pytest.mark.parametrize("kind", ["rows_with_long_rows", "brick"])
def test_product_captured_in_a_cuda_graph_and_replayed(oracle_mod, kind):
    """cutespmm_spmm allocates nothing and synchronises nothing, so an iterative caller can capture it in a CUDA graph:
    the replays must give the product of whatever B holds at replay time (the long rows' arrival counters are back at
    zero after every launch)."""
    if kind == "brick":
        A = g.stencil9(64, 64)
        plan = cs.Plan.from_csr(A, path=cs.PATH_BRICK)
        tol = REL_FRO_TOL
    else:
        A = g.rmat(11, 8, seed=71, values="uniform")
        plan = cs.Plan.from_csr(A, path=cs.PATH_ROWS)
        assert plan.info()["num_long_rows"] > 0
        tol = REL_FRO_TOL_FP32
    N = 128
    B = g.dense_operand(A.K, N, 72).cuda()
    C = torch.full((A.M, N), float("nan"), device="cuda")
    plan.spmm(B, C)  # first launch outside the capture (kernel attributes, module load)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        plan.spmm(B, C)
    for seed in (73, 74, 75):
        B.copy_(g.dense_operand(A.K, N, seed).cuda())
        C.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        ref = oracle_mod.spmm_csr(A.row_ptr, A.cols, A.vals, B.cpu().numpy(), A.M, A.K)
        assert oracle_mod.rel_fro(ref, C.cpu().numpy()) <= tol
    assert plan.device_status() == 0


def test_strided_and_misaligned_operands(oracle_mod):
    A = g.uniform_random(300, 200, 5, seed=41)  # M not a multiple of 16
    p = cs.Plan.from_csr(A, path=cs.PATH_ROWS)
    N = 96
    big = g.dense_operand(A.K, N + 7, 42).cuda()
    Bv = big[:, 3 : 3 + N]  # 12-byte offset: not 16-byte aligned, ld = N + 7
    Cbig = torch.full((A.M, N + 5), float("nan"), device="cuda")
    Cv = Cbig[:, 1 : 1 + N]
    p.spmm(Bv, Cv)
    torch.cuda.synchronize()
    ref = oracle_mod.spmm_csr(A.row_ptr, A.cols, A.vals, Bv.cpu().contiguous().numpy(), A.M, A.K)
    assert oracle_mod.rel_fro(ref, Cv.cpu().contiguous().numpy()) <= REL_FRO_TOL_FP32
    assert torch.isnan(Cbig[:, 0]).all() and torch.isnan(Cbig[:, 1 + N :]).all()  # nothing outside the window


def test_empty_rows_panels_and_matrix(oracle_mod):
    # rows 0..63 empty, a dense row, then empties
    M, K, N = 160, 64, 64
    rp = np.zeros(M + 1, np.uint64)
    rp[70:] = 64
    rp[100:] = 65
    cols = np.concatenate([np.arange(64), [5]]).astype(np.uint32)
    vals = np.linspace(-1, 1, 65).astype(np.float32)
    B = g.dense_operand(K, N, 51).numpy()
    ref = oracle_mod.spmm_csr(rp, cols, vals, B, M, K)
    for path in (cs.PATH_ROWS, cs.PATH_AUTO, cs.PATH_BRICK, cs.PATH_SLAB):
        C = run(cs.Plan(M, K, rp, cols, vals, path=path), B)
        assert oracle_mod.rel_fro(ref, C) <= REL_FRO_TOL
        assert not C[:69].any() and not C[100:].any()
    zero = cs.Plan(48, 16, np.zeros(49, np.uint64), np.zeros(0, np.uint32), np.zeros(0, np.float32))
    assert not run(zero, np.ones((16, 32), np.float32)).any()


def test_unsorted_and_duplicate_columns(oracle_mod):
    gd = load_golden("uniform_256_unsorted")
    p = cs.Plan(int(gd["M"]), int(gd["K"]), gd["row_ptr"], gd["cols"], gd["vals"], path=cs.PATH_ROWS)
    assert oracle_mod.rel_fro(gd["C"], run(p, gd["B"])) <= REL_FRO_TOL_FP32
    # duplicates add up, as in spmm_coo
    rp = np.array([0, 3, 3, 4], np.uint64)
    cols = np.array([2, 2, 0, 1], np.uint32)
    vals = np.array([1.0, 2.0, 4.0, 8.0], np.float32)
    B = g.dense_operand(3, 32, 61).numpy()
    ref = oracle_mod.spmm_csr(rp, cols, vals, B, 3, 3)
    for path in (cs.PATH_ROWS, cs.PATH_BRICK, cs.PATH_SLAB):
        assert oracle_mod.rel_fro(ref, run(cs.Plan(3, 3, rp, cols, vals, path=path), B)) <= REL_FRO_TOL


def test_hub_rows_are_deterministic(oracle_mod):
    A = g.rmat(14, 8, seed=71, values="uniform")
    p = cs.Plan.from_csr(A, path=cs.PATH_ROWS, split_nnz=128)
    assert p.info()["num_chunks"] > 100
    B = g.dense_operand(A.K, 128, 72).numpy()
    c1, c2 = run(p, B), run(p, B)
    assert np.array_equal(c1.view(np.uint32), c2.view(np.uint32))  # no atomics: bit-stable run to run
    ref = oracle_mod.spmm_csr(A.row_ptr, A.cols, A.vals, B, A.M, A.K)
    assert oracle_mod.rel_fro(ref, c1) <= REL_FRO_TOL_FP32


def test_host_buffer_call(oracle_mod):
    gd = load_golden("elasticity_4")
    p = cs.Plan(int(gd["M"]), int(gd["K"]), gd["row_ptr"], gd["cols"], gd["vals"])
    Bh = torch.from_numpy(gd["B"]).pin_memory()
    C, ms = p.spmm_host(Bh)
    assert ms > 0.0
    assert oracle_mod.rel_fro(gd["C"], C.numpy()) <= REL_FRO_TOL
    C2, _ = p.spmm_host(gd["B"][:, :17].copy())  # narrower N reuses the staging buffers
    assert oracle_mod.rel_fro(gd["C"][:, :17].copy(), C2.numpy()) <= REL_FRO_TOL


@pytest.mark.parametrize("N", [16, 32, 64, 128, 512])
def test_small_job_sizing_cuts_long_rows_finer_and_sums_them_in_the_kernel(oracle_mod, N):
    """A small matrix (a latency-bound job) with a few rows of thousands of nonzeros among short ones: with the sizes
    left to the library the long rows are cut into pieces of about sqrt(length / 2) nonzeros, rows of more than 128
    nonzeros are cut too, and one launch computes everything -- the pieces of a row are added in the kernel by whoever finishes last.
    Repeated launches must give the same bits (the arrival counters return to zero; the sum order is fixed)."""
    rng = np.random.default_rng(5)
    M, K = 3001, 2500
    lens = rng.integers(0, 9, M)
    lens[[7, 1500, 2999]] = [2400, 700, 128]  # 69 / 22 pieces; 128 stays whole
    lens[100:140] = 140                       # just over the cut length: 5 pieces each
    rp = np.zeros(M + 1, np.int64); np.cumsum(lens, out=rp[1:])
    cols = np.concatenate([np.sort(rng.choice(K, int(l), replace=False)) for l in lens]).astype(np.int32)
    vals = rng.standard_normal(cols.size).astype(np.float32)
    p = cs.Plan(M, K, rp, cols, vals, path=cs.PATH_ROWS)
    info = p.info()
    assert info["num_long_rows"] == 42 and info["num_chunks"] == 69 + 22 + 40 * 5
    assert p.launch_count(N) == 1
    B = g.dense_operand(K, N, 77).numpy()
    ref = oracle_mod.spmm_csr(rp, cols, vals, B, M, K)
    C1 = run(p, B)
    assert oracle_mod.rel_fro(ref, C1) <= REL_FRO_TOL_FP32
    for _ in range(3):
        assert np.array_equal(C1, run(p, B))
    # the same matrix with the sizes given: rows up to 256 nonzeros stay whole
    q = cs.Plan(M, K, rp, cols, vals, path=cs.PATH_ROWS, split_nnz=256, tile_nnz=512)
    assert q.info()["num_long_rows"] == 2
    assert oracle_mod.rel_fro(ref, run(q, B)) <= REL_FRO_TOL_FP32


@pytest.mark.parametrize("N,pad,pinned", [(128, 0, True), (256, 0, True), (200, 12, True), (160, 0, False), (40, 8, True)])
def test_host_call_pipelined_in_column_windows(oracle_mod, N, pad, pinned):
    """Operands of 8 MB and more go through the host call in up to four column windows (copy-in,
    product, copy-out overlapped); the result must be the one-piece product for every window
    shape: full windows, a narrow last window, padded leading dimensions, pageable memory."""
    A = g.stencil9(192)  # M = K = 36864: 36864 x 128 x 4 B = 18.9 MB at N = 128 (two windows), 5.9 MB at N = 40 (one piece)
    p = cs.Plan.from_csr(A)
    Bfull = torch.randn(A.K, N + pad)
    Cfull = torch.full((A.M, N + pad), float("nan"))
    if pinned:
        Bfull, Cfull = Bfull.pin_memory(), Cfull.pin_memory()
    Bh, Ch = Bfull[:, :N], Cfull[:, :N]
    _, ms = p.spmm_host(Bh, Ch)
    assert ms > 0.0
    ref = p.spmm(Bh.cuda().contiguous()).cpu()  # device-resident call, one piece (may take another kernel: compare at tolerance)
    assert oracle_mod.rel_fro(ref.numpy(), Ch.contiguous().numpy()) <= REL_FRO_TOL
    if pad:
        assert torch.isnan(Cfull[:, N:]).all()  # nothing written beyond column N
    want = oracle_mod.spmm_csr(A.row_ptr, A.cols, A.vals, Bh.contiguous().numpy(), A.M, A.K)
    assert oracle_mod.rel_fro(want, Ch.contiguous().numpy()) <= REL_FRO_TOL


def test_execution_errors_are_status_codes():
    gd = load_golden("stencil_16x16")
    p = cs.Plan(int(gd["M"]), int(gd["K"]), gd["row_ptr"], gd["cols"], gd["vals"])
    B = torch.zeros(int(gd["K"]), 16, device="cuda")
    assert cs.lib.cutespmm_spmm(p._h, B.data_ptr(), 8, B.data_ptr(), 16, 16, None) == -1  # ldb < N
    assert cs.lib.cutespmm_spmm(p._h, None, 16, B.data_ptr(), 16, 16, None) == -1
    assert cs.lib.cutespmm_spmm(p._h, B.data_ptr() + 2, 16, B.data_ptr(), 16, 16, None) == -1  # misaligned


def test_full_size_properties_without_cpu_product(oracle_mod):
    """At the size where the CPU product takes too long: linearity in B and the column-sum identity
    1^T (A B) = (A^T 1)^T B, both checked on the device in fp64, and a sample of rows (2^16 random rows plus every
    row with more than 4096 nonzeros) against the CPU oracle.  The plan is built from the device-resident CSR."""
    A = g.rmat(22, 8, seed=1005, values="uniform", device="cuda")
    N = 128
    p = cs.Plan.from_device_csr(A.M, A.K, A.row_ptr.to(torch.int32), A.cols.to(torch.int32), A.vals)
    B1 = g.dense_operand(A.K, N, 81, device="cuda")
    B2 = g.dense_operand(A.K, N, 82, device="cuda")
    C1, C2, C12 = p.spmm(B1), p.spmm(B2), p.spmm(B1 + B2)
    torch.cuda.synchronize()
    num = (C12.double() - C1.double() - C2.double()).norm()
    assert float(num / C12.double().norm()) < 1e-5
    colsum = torch.zeros(A.K, dtype=torch.float64, device="cuda")
    colsum.index_add_(0, A.cols.long(), A.vals.double())
    expect = colsum @ B1.double()
    got = C1.double().sum(0)
    assert float((got - expect).norm() / expect.norm()) < 1e-5
    deg = (A.row_ptr[1:] - A.row_ptr[:-1]).cpu()
    gen = torch.Generator().manual_seed(7)
    which = torch.unique(torch.cat([torch.randint(0, A.M, (1 << 16,), generator=gen), torch.nonzero(deg > 4096).flatten()]))
    want = oracle_mod.spmm_csr_rows(A.row_ptr.cpu(), A.cols.cpu(), A.vals.cpu(), B1.cpu().numpy(), which.numpy())
    assert oracle_mod.rel_fro(want, C1[which.cuda()].cpu().numpy()) <= REL_FRO_TOL_FP32


def test_largest_configuration_at_its_own_size(oracle_mod):
    """The R-MAT graph with 2^24 nodes at N = 128 on one GPU: B and C hold 2^31 elements each, so every element offset
    above 2^31 - 1 needs the kernels' 64-bit address arithmetic (the reference computes these offsets in 32 bits,
    kernel.cu:149,267,281).  Checked: 2^16 random rows plus every row with more than 4096 nonzeros against the CPU
    oracle, and the column-sum identity 1^T (A B) = (A^T 1)^T B in fp64 as the whole-matrix checksum.  The plan is
    built from the device-resident CSR."""
    free, _ = torch.cuda.mem_get_info()
    if free < 60 << 30:
        pytest.skip("needs about 60 GB of free device memory")
    w = g.WORKLOADS["rmat24"]
    A = w["make"](device="cuda")
    N = w["N"]
    assert A.M == 1 << 24 and A.M * N == 1 << 31
    p = cs.Plan.from_device_csr(A.M, A.K, A.row_ptr.to(torch.int32), A.cols.to(torch.int32), A.vals)
    B = g.dense_operand(A.K, N, w["b_seed"], w["b_dist"], device="cuda")
    C = torch.full((A.M, N), float("nan"), device="cuda")
    p.spmm(B, C)
    torch.cuda.synchronize()
    assert p.device_status() == 0
    # whole-matrix checksum, fp64, in row chunks (no 17 GB temporaries)
    colsum = torch.zeros(A.K, dtype=torch.float64, device="cuda")
    colsum.index_add_(0, A.cols.long(), A.vals.double())
    expect = torch.zeros(N, dtype=torch.float64, device="cuda")
    got = torch.zeros(N, dtype=torch.float64, device="cuda")
    step = 1 << 20
    for r in range(0, A.K, step):
        expect += colsum[r : r + step] @ B[r : r + step].double()
        got += C[r : r + step].sum(0, dtype=torch.float64)
    assert float((got - expect).norm() / expect.norm()) < 1e-5
    # sampled rows against the oracle: random rows over the whole range (high rows: offsets beyond 2^31) + every hub row
    deg = A.row_ptr[1:] - A.row_ptr[:-1]
    gen = torch.Generator().manual_seed(11)
    hubs = torch.nonzero(deg > 4096).flatten().cpu()
    assert hubs.numel() > 100
    rand = torch.unique(torch.cat([torch.randint(0, A.M, (1 << 16,), generator=gen), torch.tensor([A.M - 1])]))
    assert int(rand.max()) * N + N - 1 > 2**31 - 2**20  # the top of the offset range is sampled
    Bh = B.cpu().numpy()
    rp, cols, vals = A.row_ptr.cpu(), A.cols.cpu(), A.vals.cpu()
    for which, tol in ((rand[deg[rand.cuda()].cpu() <= 4096], REL_FRO_TOL_FP32), (hubs, 10 * REL_FRO_TOL_FP32)):
        # hub rows hold up to 3.7e5 nonzeros: the oracle adds them one after the other in fp32, the kernel in chunks of 256,
        # and the two orders differ by the rounding noise of the longer chain -- hence the wider bound for them
        got_rows = C[which.cuda()].cpu().numpy()
        want = oracle_mod.spmm_csr_rows(rp, cols, vals, Bh, which.numpy())
        assert not np.isnan(got_rows).any()
        assert oracle_mod.rel_fro(want, got_rows) <= tol, (which.numel(), tol)


@pytest.mark.parametrize("how", ["cluster", "similar"])
@pytest.mark.parametrize("path", [cs.PATH_ROWS, cs.PATH_BRICK, cs.PATH_AUTO], ids=["rows", "brick", "auto"])
def test_row_clustering_keeps_the_callers_row_order(oracle_mod, path, how):
    """A plan with CUTESPMM_REORDER_CLUSTER_ROWS processes the rows in another order but writes every row of C to its
    own place: the product of a row-shuffled stencil and of a power-law graph (hub rows cut into chunks: the in-launch sum
    writes mapped rows too) must equal the oracle's on the caller's matrix."""
    from test_host import _shuffle_rows

    S, _ = _shuffle_rows(g.stencil9(160))
    for A, N in ((S, 128), (S, 96), (g.rmat(13, 8, seed=5, values="uniform"), 64)):
        p = cs.Plan.from_csr(A, path=path, reorder=how, split_nnz=64)
        B = g.dense_operand(A.K, N, 77).numpy()
        ref = oracle_mod.spmm_csr(A.row_ptr, A.cols, A.vals, B, A.M, A.K)
        assert oracle_mod.rel_fro(ref, run(p, B)) <= PATH_TOL[path], (A.name, N)
    if path == cs.PATH_AUTO:  # the point of the option: the shuffled stencil is back on the tensor-core kernel
        assert cs.Plan.from_csr(S, reorder=how).info()["num_bricks"] > 0 and cs.Plan.from_csr(S).info()["num_bricks"] == 0


@pytest.mark.parametrize("N,pad,path", [(128, 0, cs.PATH_AUTO), (200, 8, cs.PATH_AUTO), (64, 0, cs.PATH_ROWS), (256, 0, cs.PATH_BRICK)])
def test_host_call_in_blocks_of_rows_on_banded_matrices(oracle_mod, N, pad, path):
    """On one GPU, operands of many megabytes and a matrix whose rows name an advancing range of columns, the host call
    uploads B in row order, multiplies block of rows by block of rows and returns each block's rows of C while B is
    still arriving.  Every block boundary, both work lists (N = 200 is not a width the brick kernel takes) and padded
    leading dimensions must give the oracle's product; a matrix that does not qualify (a graph whose every block of
    rows names all of B) takes the column-window path and must be right as well."""
    A = g.stencil9(384)  # M = K = 147456: 75 MB at N = 128 -> 9 blocks of rows
    p = cs.Plan.from_csr(A, path=path, split_nnz=256)
    Bfull = g.dense_operand(A.K, N + pad, 91).pin_memory()
    Cfull = torch.full((A.M, N + pad), float("nan")).pin_memory()
    Bh, Ch = Bfull[:, :N], Cfull[:, :N]
    for _ in range(2):  # the second call reuses the cut and the staging
        Ch.fill_(float("nan"))
        _, ms = p.spmm_host(Bh, Ch)
        assert ms > 0.0
        want = oracle_mod.spmm_csr(A.row_ptr, A.cols, A.vals, Bh.contiguous().numpy(), A.M, A.K)
        assert oracle_mod.rel_fro(want, Ch.contiguous().numpy()) <= PATH_TOL[path]
    if pad:
        assert torch.isnan(Cfull[:, N:]).all()
    G = g.rmat(16, 16, seed=93, values="uniform")  # hub rows (chunks + fix-up) and no band: column windows
    pg = cs.Plan.from_csr(G)
    Bg = g.dense_operand(G.K, 128, 94).pin_memory()
    Cg, _ = pg.spmm_host(Bg)
    want = oracle_mod.spmm_csr(G.row_ptr, G.cols, G.vals, Bg.numpy(), G.M, G.K)
    assert oracle_mod.rel_fro(want, Cg.numpy()) <= REL_FRO_TOL_FP32 * 5
    # a banded matrix with long rows inside the band: the chunk and fix-up lists are cut by blocks too
    rows, K2 = 1 << 16, 1 << 16
    lens = np.full(rows, 6, dtype=np.int64)
    lens[::997] = 700
    rp = np.zeros(rows + 1, dtype=np.int64)
    np.cumsum(lens, out=rp[1:])
    r_of = np.repeat(np.arange(rows), lens)
    cols = np.clip(r_of + (np.arange(rp[-1]) - rp[r_of]) - 3, 0, K2 - 1)
    vals = np.linspace(-1.0, 1.0, rp[-1]).astype(np.float32)
    pb = cs.Plan(rows, K2, rp, cols.astype(np.uint32), vals)
    assert pb.info()["num_long_rows"] > 0
    Bb = g.dense_operand(K2, 128, 95).pin_memory()
    Cb, _ = pb.spmm_host(Bb)
    want = oracle_mod.spmm_csr(rp.astype(np.uint64), cols.astype(np.uint32), vals, Bb.numpy(), rows, K2)
    assert oracle_mod.rel_fro(want, Cb.numpy()) <= REL_FRO_TOL
