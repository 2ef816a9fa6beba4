"""cutespmm_sddmm against the CPU oracle: one dot product of feature rows per stored nonzero, in the plan's
storage order; every plan flavour, any N, strided operands, hub rows, and its use as the gradient of the product
with respect to the values of A."""
import numpy as np
import pytest
import torch

import cutespmm_ae_b200 as cs
from cutespmm_ae_b200 import generators as g

pytestmark = pytest.mark.gpu
TOL = 2e-6  # fp32 dot products, another summation order than the oracle's


def rel(ref, got):
    ref, got = ref.astype(np.float64), got.astype(np.float64)
    return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))


@pytest.mark.parametrize("N", [128, 64, 100, 200, 7, 512])
@pytest.mark.parametrize("scale", [False, True])
def test_sddmm_matches_oracle_for_any_width(oracle_mod, N, scale):
    A = g.rmat(11, 8, seed=51, values="uniform")  # hub rows: the chunked part of the work list
    p = cs.Plan.from_csr(A, split_nnz=64)
    assert p.info()["num_long_rows"] > 0
    X = g.dense_operand(A.M, N, 52, device="cuda")
    Y = g.dense_operand(A.K, N, 53, device="cuda")
    out = torch.full((A.nnz,), float("nan"), device="cuda")
    p.sddmm(X, Y, out, scale_by_values=scale)
    torch.cuda.synchronize()
    want = oracle_mod.sddmm_csr(A.row_ptr, A.cols, A.vals if scale else None, X.cpu().numpy(), Y.cpu().numpy())
    assert rel(want, out.cpu().numpy()) <= TOL


@pytest.mark.parametrize("make,path", [(lambda: g.stencil9(64), cs.PATH_AUTO), (lambda: g.elasticity3d(8, 3, 4), cs.PATH_BRICK),
                                        (lambda: g.uniform_random(300, 200, 5, seed=41), cs.PATH_ROWS)])
def test_sddmm_on_every_plan_flavour_and_strided_operands(oracle_mod, make, path):
    A = make()
    N = 96
    Xbig, Ybig = g.dense_operand(A.M, N + 5, 54).cuda(), g.dense_operand(A.K, N + 3, 55).cuda()
    X, Y = Xbig[:, 1 : 1 + N], Ybig[:, 3 : 3 + N]  # not 16-byte aligned, padded leading dimensions
    want = oracle_mod.sddmm_csr(A.row_ptr, A.cols, A.vals, X.cpu().contiguous().numpy(), Y.cpu().contiguous().numpy())
    host = cs.Plan.from_csr(A, path=path)
    dev = cs.Plan.from_device_csr(A.M, A.K, A.row_ptr.to(torch.int32).cuda(), A.cols.cuda(), A.vals.cuda(), path=path)
    for plan in (host, dev):
        out = plan.sddmm(X, Y, scale_by_values=True)
        torch.cuda.synchronize()
        assert rel(want, out.cpu().numpy()) <= TOL


def test_sddmm_is_the_gradient_of_the_product_with_respect_to_the_values(oracle_mod):
    """C = A B  =>  dL/dA_j = <dL/dC[row of j], B[column of j]>: check against a finite difference of the oracle."""
    A = g.uniform_random(64, 48, 4, seed=61)
    N = 32
    B = g.dense_operand(A.K, N, 62)
    G = g.dense_operand(A.M, N, 63)  # dL/dC for L = sum(G * C)
    p = cs.Plan.from_csr(A)
    grad = p.sddmm(G.cuda(), B.cuda()).cpu().numpy()
    rows = np.repeat(np.arange(A.M), np.diff(A.row_ptr.numpy()))
    expect = (G.numpy()[rows].astype(np.float64) * B.numpy()[A.cols.numpy()].astype(np.float64)).sum(1)
    assert rel(expect, grad) <= TOL
    j = 17  # one entry by finite difference through the oracle's product
    vals = A.vals.numpy().astype(np.float32).copy()
    loss = lambda v: float((G.numpy().astype(np.float64) * oracle_mod.spmm_csr(A.row_ptr, A.cols, v, B.numpy(), A.M, A.K)).sum())  # noqa: E731
    vp, vm = vals.copy(), vals.copy()
    vp[j] += 0.25
    vm[j] -= 0.25
    assert abs((loss(vp) - loss(vm)) / 0.5 - grad[j]) <= 1e-3 * max(1.0, abs(grad[j]))


def test_sddmm_refusals_and_empty_cases():
    A = g.stencil9(16)
    p = cs.Plan.from_csr(A, reorder="cluster", path=cs.PATH_ROWS)
    X = torch.zeros(A.M, 8, device="cuda")
    if p.info()["nnz"]:
        S, _ = __import__("test_host")._shuffle_rows(A)
        ps = cs.Plan.from_csr(S, reorder="cluster")
        with pytest.raises(cs.CuteSpmmError) as e:
            ps.sddmm(X, X)
        assert e.value.status == -4
    with pytest.raises(ValueError):
        cs.Plan.from_csr(A).sddmm(X, torch.zeros(A.K, 9, device="cuda"))
    empty = cs.Plan(32, 16, np.zeros(33, np.uint64), np.zeros(0, np.uint32), np.zeros(0, np.float32))
    assert empty.sddmm(torch.zeros(32, 8, device="cuda"), torch.zeros(16, 8, device="cuda")).numel() == 0


@pytest.mark.parametrize("builder", ["host", "device"])
def test_set_values_makes_edge_scores_the_weights_of_the_next_product(oracle_mod, builder, tmp_path):
    """The attention step of a graph layer: scores = sddmm(X, Y), any elementwise normalisation, set_values(scores), then
    the product aggregates with those weights.  The pattern and the work lists stay; decode and save see the new values."""
    A = g.rmat(11, 8, seed=81, values="uniform")  # hub rows: chunks whose pieces are summed in the launch
    if builder == "host":
        p = cs.Plan.from_csr(A, path=cs.PATH_ROWS)
    else:
        p = cs.Plan.from_device_csr(A.M, A.K, A.row_ptr.to(torch.int32).cuda(), A.cols.to(torch.int32).cuda(), A.vals.cuda(), path=cs.PATH_ROWS)
    assert p.info()["num_long_rows"] > 0
    X, Y = g.dense_operand(A.M, 64, 82, device="cuda"), g.dense_operand(A.K, 64, 83, device="cuda")
    w = torch.tanh(p.sddmm(X, Y) / 8.0)
    p.set_values(w)
    rp, cc, vv = p.decode_csr()  # the plan's storage order, with the new values
    assert np.array_equal(vv, w.cpu().numpy())
    B = g.dense_operand(A.K, 128, 84)
    C = torch.full((A.M, 128), float("nan"), device="cuda")
    p.spmm(B.cuda(), C)
    torch.cuda.synchronize()
    ref = oracle_mod.spmm_csr(rp, cc, vv, B.numpy(), A.M, A.K)
    assert oracle_mod.rel_fro(ref, C.cpu().numpy()) <= TOL
    # a second replacement, and the saved plan carries what the device holds
    p.set_values(-w)
    f = tmp_path / "weighted.plan"
    p.save(f)
    q = cs.Plan.load(f)
    C2 = torch.empty_like(C)
    q.spmm(B.cuda(), C2)
    torch.cuda.synchronize()
    assert oracle_mod.rel_fro(-ref, C2.cpu().numpy()) <= TOL
    assert np.array_equal(q.decode_csr()[2], -vv)


def test_set_values_is_refused_where_the_values_live_in_tensor_core_records_or_rows_are_reordered():
    S = g.stencil9(64)
    for kw in (dict(path=cs.PATH_BRICK), dict(path=cs.PATH_ROWS, reorder="cluster")):
        p = cs.Plan.from_csr(S, **kw)
        with pytest.raises(cs.CuteSpmmError) as e:
            p.set_values(torch.ones(S.nnz, device="cuda"))
        assert e.value.status == -4
    p = cs.Plan.from_csr(S, path=cs.PATH_ROWS)
    with pytest.raises(ValueError):
        p.set_values(torch.ones(S.nnz + 1, device="cuda"))
