"""torch.library wrapper over the C ABI (cutespmm_ae_b200/torch_ops.py): forward equals the plan's product,
the gradient with respect to B is A^T dC (transposed plan), the registered fake kernels give shapes without running
anything, and torch's own operator checker accepts the registration."""
import numpy as np
import pytest
import torch

import cutespmm_ae_b200 as cs
from cutespmm_ae_b200 import generators as g
from cutespmm_ae_b200 import torch_ops


def test_transpose_csr_matches_dense_transpose():
    A = g.uniform_random(37, 23, 4, seed=3)
    rp, cols, vals = torch_ops.transpose_csr(A.M, A.K, A.row_ptr.numpy(), A.cols.numpy(), A.vals.numpy())
    dense = np.zeros((A.M, A.K), np.float32)
    rows = np.repeat(np.arange(A.M), np.diff(A.row_ptr.numpy()))
    dense[rows, A.cols.numpy()] = A.vals.numpy()
    dt = np.zeros((A.K, A.M), np.float32)
    trows = np.repeat(np.arange(A.K), np.diff(rp.astype(np.int64)))
    dt[trows, cols] = vals
    assert np.array_equal(dt, dense.T)


def test_ops_are_registered_and_fake_kernels_give_shapes():
    A = g.stencil9(16)
    op = torch_ops.SparseOperator(cs.Plan.from_csr(A, host_only=True))
    assert hasattr(torch.ops.cutespmm, "spmm") and hasattr(torch.ops.cutespmm, "sddmm")
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        B = torch.empty(A.K, 24)
        assert tuple(torch.ops.cutespmm.spmm(op.id, B).shape) == (A.M, 24)
        assert tuple(torch.ops.cutespmm.spmm_transposed(op.id, torch.empty(A.M, 8)).shape) == (A.K, 8)
        assert tuple(torch.ops.cutespmm.sddmm(op.id, torch.empty(A.M, 8), torch.empty(A.K, 8), False).shape) == (A.nnz,)
    with pytest.raises(RuntimeError):
        torch.ops.cutespmm.spmm(10**9, torch.empty(3, 3))
    op.close()


@pytest.mark.gpu
def test_forward_backward_and_opcheck(oracle_mod):
    A = g.rmat(10, 8, seed=9, values="uniform")
    # the transposed plan (backward pass) is built with the same options: the fp32 row kernel on both sides
    op = torch_ops.SparseOperator(cs.Plan.from_csr(A, path=cs.PATH_ROWS), plan_kwargs=dict(path=cs.PATH_ROWS))
    B = g.dense_operand(A.K, 64, 10, device="cuda").requires_grad_(True)
    C = op(B)
    ref = oracle_mod.spmm_csr(A.row_ptr, A.cols, A.vals, B.detach().cpu().numpy(), A.M, A.K)
    assert oracle_mod.rel_fro(ref, C.detach().cpu().numpy()) <= 2e-6
    G = g.dense_operand(A.M, 64, 11, device="cuda")
    (C * G).sum().backward()
    t_rp, t_cols, t_vals = torch_ops.transpose_csr(A.M, A.K, A.row_ptr.numpy(), A.cols.numpy(), A.vals.numpy())
    want = oracle_mod.spmm_csr(t_rp, t_cols, t_vals, G.cpu().numpy(), A.K, A.M)  # A^T G
    assert oracle_mod.rel_fro(want, B.grad.cpu().numpy()) <= 2e-6
    scores = op.sddmm(G, B.detach())
    want_s = oracle_mod.sddmm_csr(A.row_ptr, A.cols, None, G.cpu().numpy(), B.detach().cpu().numpy())
    assert np.linalg.norm(scores.cpu().numpy() - want_s) <= 2e-6 * np.linalg.norm(want_s)
    torch.library.opcheck(torch.ops.cutespmm.spmm.default, (op.id, B.detach().clone().requires_grad_(True)),
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))
    op.close()


@pytest.mark.gpu
def test_attention_weights_flow_through_forward_and_backward(oracle_mod):
    """scores = sddmm -> weights -> set_values: the forward product and the gradient with respect to B (through the plan
    of A^T, rebuilt after the values changed) both use the new weights."""
    A = g.rmat(10, 8, seed=19, values="uniform")
    op = torch_ops.SparseOperator(cs.Plan.from_csr(A, path=cs.PATH_ROWS), plan_kwargs=dict(path=cs.PATH_ROWS))
    B = g.dense_operand(A.K, 64, 20, device="cuda").requires_grad_(True)
    G = g.dense_operand(A.M, 64, 21, device="cuda")
    (op(B) * G).sum().backward()  # builds the plan of A^T from the old values
    B.grad = None
    w = torch.sigmoid(op.sddmm(G, B.detach()))
    op.set_values(w)
    rp, cc, vv = op.plan.decode_csr()
    C = op(B)
    assert oracle_mod.rel_fro(oracle_mod.spmm_csr(rp, cc, vv, B.detach().cpu().numpy(), A.M, A.K), C.detach().cpu().numpy()) <= 2e-6
    (C * G).sum().backward()
    t_rp, t_cols, t_vals = torch_ops.transpose_csr(A.M, A.K, rp, cc, vv)
    want = oracle_mod.spmm_csr(t_rp, t_cols, t_vals, G.cpu().numpy(), A.K, A.M)
    assert oracle_mod.rel_fro(want, B.grad.cpu().numpy()) <= 2e-6
    op.close()


@pytest.mark.gpu
def test_weighted_product_is_differentiable_in_the_weights_and_in_b():
    """op.weighted(w, B) against a dense torch product built from the same pattern: forward, dC/dw (SDDMM) and dC/dB
    (the transposed plan with permuted weights), twice with different weights (the plans are reused)."""
    A = g.uniform_random(300, 200, 7, seed=31)
    op = torch_ops.SparseOperator(cs.Plan.from_csr(A, path=cs.PATH_ROWS), plan_kwargs=dict(path=cs.PATH_ROWS))
    rp, cc, _ = op.plan.decode_csr()
    rows = torch.from_numpy(np.repeat(np.arange(A.M), np.diff(rp.astype(np.int64)))).cuda()
    cols = torch.from_numpy(cc.astype(np.int64)).cuda()
    for seed in (32, 33):
        w = g.dense_operand(A.nnz, 1, seed, device="cuda").flatten().requires_grad_(True)
        B = g.dense_operand(A.K, 48, seed + 10, device="cuda").requires_grad_(True)
        G = g.dense_operand(A.M, 48, seed + 20, device="cuda")
        (op.weighted(w, B) * G).sum().backward()
        w2, B2 = w.detach().clone().requires_grad_(True), B.detach().clone().requires_grad_(True)
        dense = torch.zeros(A.M, A.K, device="cuda").index_put((rows, cols), w2)
        C_ref = dense @ B2
        (C_ref * G).sum().backward()
        C = op.weighted(w.detach(), B.detach())
        assert torch.allclose(C, C_ref.detach(), rtol=1e-4, atol=1e-4)
        assert torch.allclose(w.grad, w2.grad, rtol=1e-4, atol=1e-4)
        assert torch.allclose(B.grad, B2.grad, rtol=1e-4, atol=1e-4)
    torch.library.opcheck(torch.ops.cutespmm.spmm_weighted.default,
                          (op.id, w.detach().clone().requires_grad_(True), B.detach().clone().requires_grad_(True)),
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))
    op.close()
