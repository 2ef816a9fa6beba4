"""cutespmm_plan_create_device: a plan built from CSR arrays that live on the GPU must give the row kernel's
result bit for bit (same work lists, same kernel), decode to the arrays it was given, and refuse what the
device builder does not do."""
import numpy as np
import pytest
import torch

import cutespmm_ae_b200 as cs
from cutespmm_ae_b200 import generators as g

pytestmark = pytest.mark.gpu


def _dev(A):
    return (A.row_ptr.to(torch.int32).cuda().contiguous(), A.cols.to(torch.int32).cuda().contiguous(), A.vals.to(torch.float32).cuda().contiguous())


@pytest.mark.parametrize("make,N", [(lambda: g.rmat(14, 8, seed=31, values="uniform"), 128), (lambda: g.stencil9(96), 64),
                                     (lambda: g.uniform_random(1000, 777, 5, seed=4), 20)])
def test_device_built_plan_equals_host_built_rows_plan(oracle_mod, make, N):
    A = make()
    rp, cols, vals = _dev(A)
    pd = cs.Plan.from_device_csr(A.M, A.K, rp, cols, vals)
    ph = cs.Plan.from_csr(A, path=cs.PATH_ROWS)
    id_, ih = pd.info(), ph.info()
    for k in ("M", "K", "nnz", "num_tiles", "num_long_rows", "num_chunks"):
        assert id_[k] == ih[k]
    assert id_["brick_panels"] == 0
    B = g.dense_operand(A.K, N, 17, device="cuda")
    Cd, Ch = pd.spmm(B), ph.spmm(B)
    torch.cuda.synchronize()
    assert torch.equal(Cd, Ch)
    ref = oracle_mod.spmm_csr(A.row_ptr, A.cols, A.vals, B.cpu().numpy(), A.M, A.K)
    assert oracle_mod.rel_fro(ref, Cd.cpu().numpy()) <= 2e-6
    drp, dcols, dvals = pd.decode_csr()
    assert np.array_equal(drp, A.row_ptr.numpy().astype(np.uint64))
    assert np.array_equal(dcols, A.cols.numpy().astype(np.uint32)) and np.array_equal(dvals, A.vals.numpy())
    assert pd.device_status() == 0


def test_device_builder_handles_unsorted_rows_hub_rows_and_empty_matrices(oracle_mod):
    A = g.rmat(12, 16, seed=9, values="uniform")  # hub rows longer than the split length: chunks + fix-up
    perm = torch.arange(A.nnz)
    rp = A.row_ptr.numpy()
    for r in range(0, A.M, 7):  # reverse the nonzeros of every seventh row: rows need not be sorted
        perm[rp[r]:rp[r + 1]] = torch.arange(rp[r + 1] - 1, rp[r] - 1, -1)
    cols, vals = A.cols[perm], A.vals[perm]
    pd = cs.Plan.from_device_csr(A.M, A.K, A.row_ptr.to(torch.int32).cuda(), cols.to(torch.int32).cuda(), vals.cuda())
    assert pd.info()["num_long_rows"] > 0
    B = g.dense_operand(A.K, 32, 5, device="cuda")
    C = pd.spmm(B).cpu().numpy()
    ref = oracle_mod.spmm_csr(A.row_ptr, cols, vals, B.cpu().numpy(), A.M, A.K)
    assert oracle_mod.rel_fro(ref, C) <= 2e-6
    empty = cs.Plan.from_device_csr(64, 32, torch.zeros(65, dtype=torch.int32, device="cuda"), torch.zeros(0, dtype=torch.int32, device="cuda"),
                                    torch.zeros(0, device="cuda"))
    assert torch.count_nonzero(empty.spmm(torch.ones(32, 8, device="cuda"))) == 0


def test_device_builder_refusals():
    A = g.stencil9(16)
    rp, cols, vals = _dev(A)
    with pytest.raises(cs.CuteSpmmError) as e:
        cs.Plan.from_device_csr(A.M, A.K, rp, cols, vals, path=cs.PATH_BRICK)
    assert e.value.status == -4
    bad_cols = cols.clone()
    bad_cols[5] = A.K  # out of range
    with pytest.raises(cs.CuteSpmmError) as e:
        cs.Plan.from_device_csr(A.M, A.K, rp, bad_cols, vals)
    assert e.value.status == -1
    bad_rp = rp.clone()
    bad_rp[3] = bad_rp[4] + 1  # decreasing
    with pytest.raises(cs.CuteSpmmError) as e:
        cs.Plan.from_device_csr(A.M, A.K, bad_rp, cols, vals)
    assert e.value.status == -1
    p = cs.Plan.from_device_csr(A.M, A.K, rp, cols, vals)
    with pytest.raises(cs.CuteSpmmError) as e:
        p.blocked_row_ptr()
    assert e.value.status == -4
