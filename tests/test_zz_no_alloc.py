"""cutespmm_spmm_csr_noalloc -- the entry point for callers that may not allocate device memory at
call time (their framework owns all of HBM, or they run where allocating calls are forbidden).  It
keeps its partial sums in a scratch array built into the library, so this test checks what such a
caller relies on: the result equals the plan-based entry point's and the CPU oracle's on two calls
in a row (the second call meets the scratch as the first left it), requests beyond the built-in
scratch are refused with an error instead of being attempted, and input that would index outside
the caller's buffers is stopped before or inside the call.  Collected last on purpose (file name)."""
import numpy as np
import pytest
import torch

import cutespmm_ae_b200 as cs
from cutespmm_ae_b200 import generators as g
from conftest import REL_FRO_TOL_FP32

pytestmark = pytest.mark.gpu


def _rel_fro(ref, got):
    return float((got.double() - ref.double()).norm() / ref.double().norm())


def test_noalloc_matches_plan_entry_point_twice_in_a_row(oracle_mod):
    A = g.rmat(15, 8, seed=91, values="uniform")  # hub rows well above the 1024-nonzero chunk length
    assert int((A.row_ptr[1:] - A.row_ptr[:-1]).max()) > 2 * 1024
    plan = cs.Plan.from_csr(A, path=cs.PATH_ROWS)  # the existing entry point, fp32 row kernel
    rp, cols, vals = A.row_ptr.to(torch.int32).cuda(), A.cols.cuda(), A.vals.cuda()
    for call, (N, seed) in enumerate(((128, 92), (200, 93))):  # second call: other width, other B, same scratch
        B = g.dense_operand(A.K, N, seed, device="cuda")
        ref = plan.spmm(B)
        C = torch.full((A.M, N), float("nan"), device="cuda")  # caller-provided output, fully overwritten
        cs.spmm_csr_noalloc(A.M, A.K, rp, cols, vals, B, C)
        torch.cuda.synchronize()
        assert _rel_fro(ref, C) <= REL_FRO_TOL_FP32, f"call {call}"
        # and against the independent checker, not only against another kernel of this library
        want = oracle_mod.spmm_csr(A.row_ptr, A.cols, A.vals, B.cpu().numpy(), A.M, A.K)
        assert oracle_mod.rel_fro(want, C.cpu().numpy()) <= REL_FRO_TOL_FP32, f"call {call} vs oracle"


def test_noalloc_small_and_empty_rows():
    M, K, N = 40, 30, 33
    rp = np.zeros(M + 1, np.int32)
    rp[5:] = 3
    rp[20:] = 4
    cols = torch.tensor([1, 7, 29, 0], dtype=torch.int32, device="cuda")
    vals = torch.tensor([1.0, -2.0, 0.5, 3.0], device="cuda")
    B = g.dense_operand(K, N, 94, device="cuda")
    C = torch.full((M, N), float("nan"), device="cuda")
    cs.spmm_csr_noalloc(M, K, torch.from_numpy(rp).cuda(), cols, vals, B, C)
    torch.cuda.synchronize()
    exp = torch.zeros((M, N), device="cuda")
    exp[4] = B[1] - 2.0 * B[7] + 0.5 * B[29]
    exp[19] = 3.0 * B[0]
    assert torch.allclose(C, exp, rtol=1e-6, atol=1e-6)


def test_noalloc_rejects_what_the_builtin_scratch_cannot_hold():
    d = torch.zeros(8, dtype=torch.int32, device="cuda")
    f = torch.zeros(8, device="cuda")
    # N above the maximum
    st = cs.lib.cutespmm_spmm_csr_noalloc(1, 1, 1, d.data_ptr(), d.data_ptr(), f.data_ptr(), f.data_ptr(), 513,
                                          f.data_ptr(), 513, 513, None)
    assert st == -4 and b"MAX_N" in cs.lib.cutespmm_last_error()
    # more nonzeros than (scratch / N) allows: refused before any pointer is touched
    st = cs.lib.cutespmm_spmm_csr_noalloc(1 << 20, 1 << 20, 1 << 30, d.data_ptr(), d.data_ptr(), f.data_ptr(),
                                          f.data_ptr(), 128, f.data_ptr(), 128, 128, None)
    assert st == -4 and b"scratch" in cs.lib.cutespmm_last_error()
    assert cs.lib.cutespmm_spmm_csr_noalloc(4, 4, 0, None, None, None, None, 8, f.data_ptr(), 8, 8, None) == -1


def test_noalloc_wrapper_refuses_mis_shaped_operands():
    A = g.uniform_random(64, 48, 4, seed=95)
    rp, cols, vals = A.row_ptr.to(torch.int32).cuda(), A.cols.cuda(), A.vals.cuda()
    B = g.dense_operand(A.K, 32, 96, device="cuda")
    good = torch.empty((A.M, 32), device="cuda")
    for kw in (dict(Cout=torch.empty((A.M - 1, 32), device="cuda")),   # too few rows: the kernel would write past the end
               dict(Cout=torch.empty((A.M, 31), device="cuda")),       # too narrow
               dict(B=g.dense_operand(A.K - 1, 32, 96, device="cuda")),  # B shorter than A is wide
               dict(row_ptr=rp[:-1])):
        args = dict(row_ptr=rp, cols=cols, vals=vals, B=B, Cout=good)
        args.update(kw)
        with pytest.raises(ValueError):
            cs.spmm_csr_noalloc(A.M, A.K, args["row_ptr"], args["cols"], args["vals"], args["B"], args["Cout"])


def test_noalloc_survives_row_pointers_and_columns_beyond_the_arrays(oracle_mod):
    """A row pointer array whose last entries exceed the `nnz` the caller states, and a column index that is not below
    K, must not make the kernels index outside the scratch, the CSR arrays or B: positions are clamped to nnz and the
    out-of-range column contributes nothing."""
    A = g.rmat(12, 16, seed=97, values="uniform")  # rows longer than 1024 nonzeros: the chunk and fix-up kernels run
    assert int((A.row_ptr[1:] - A.row_ptr[:-1]).max()) > 1024
    N = 64
    B = g.dense_operand(A.K, N, 98, device="cuda")
    cols = A.cols.clone()
    cols[7] = A.K + 5  # not a row of B
    vals_ok = A.vals.clone()
    vals_ok[7] = 0.0   # what "contributes nothing" means for the checker
    want = oracle_mod.spmm_csr(A.row_ptr, A.cols, vals_ok, B.cpu().numpy(), A.M, A.K)
    C = torch.full((A.M, N), float("nan"), device="cuda")
    cs.spmm_csr_noalloc(A.M, A.K, A.row_ptr.to(torch.int32).cuda(), cols.cuda(), A.vals.cuda(), B, C)
    torch.cuda.synchronize()
    assert oracle_mod.rel_fro(want, C.cpu().numpy()) <= REL_FRO_TOL_FP32
    # row pointers that run past the stated nnz: rows are cut off at nnz, nothing beyond the arrays is touched
    rp_bad = A.row_ptr.clone()
    rp_bad[-40:] += 5000
    nnz_kept = A.nnz
    rp_clamped = rp_bad.clamp(max=nnz_kept)
    want2 = oracle_mod.spmm_csr(rp_clamped, A.cols, A.vals, B.cpu().numpy(), A.M, A.K)
    C2 = torch.full((A.M, N), float("nan"), device="cuda")
    cs.spmm_csr_noalloc(A.M, A.K, rp_bad.to(torch.int32).cuda(), A.cols.cuda(), A.vals.cuda(), B, C2)
    torch.cuda.synchronize()
    assert oracle_mod.rel_fro(want2, C2.cpu().numpy()) <= REL_FRO_TOL_FP32
