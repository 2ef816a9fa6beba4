"""PyTorch operator over the C ABI: `torch.ops.cutespmm.spmm(plan_id, B)` and `torch.ops.cutespmm.sddmm(...)`.

The reference tree ships its graph-layer operators as a pybind extension of the TC-GNN baseline
(TC-GNN_ATC23/TCGNN_conv/TCGNN.cpp:260-271: forward / backward are the same SpMM on the symmetric
adjacency, forward_ef is SDDMM).  Here the same two operators are `torch.library` custom ops on top of
libcutespmm, so they work under autograd, `torch.compile` (through the registered fake kernels) and on
any stream:

    op = SparseOperator(plan)          # registers the plan, gives it an integer id
    C = op(B)                          # C = A @ B, differentiable with respect to B
    scores = op.sddmm(X, Y)            # one dot product per stored nonzero
    C = op.weighted(w, B)              # C = (pattern of A with values w) @ B, differentiable with respect to w and B

The gradient of C = A @ B with respect to B is A^T @ dC: the transposed plan is built on first use
(from the plan's own decoded CSR) and cached.  In `op(B)` A is constant data of the plan, so no gradient flows
to its values.  `op.weighted(w, B)` is the attention form (TCGNN.cpp:260-264, forward_AGNN): w -- one weight per
stored nonzero in the plan's storage order, typically normalised `op.sddmm` scores -- replaces the plan's values
(Plan.set_values) before the product; its gradients are dB = A_w^T @ dC (the transposed plan receives w through a
permutation computed once) and dw = sddmm(dC, B).
"""
from __future__ import annotations

import itertools
import weakref

import numpy as np
import torch

from . import Plan

__all__ = ["SparseOperator", "register_plan", "unregister_plan", "transpose_csr"]

_plans: dict[int, "SparseOperator"] = {}
_ids = itertools.count(1)


def transpose_csr(M: int, K: int, row_ptr, cols, vals):
    """CSR of A^T (K x M) from CSR of A (M x K); entries of a row of A^T ordered by their row in A."""
    rp = np.asarray(row_ptr, dtype=np.int64)
    cols = np.asarray(cols, dtype=np.int64)
    rows = np.repeat(np.arange(M, dtype=np.int64), np.diff(rp))
    order = np.argsort(cols, kind="stable")
    t_rp = np.zeros(K + 1, dtype=np.uint64)
    np.cumsum(np.bincount(cols, minlength=K), out=t_rp[1:])
    return t_rp, rows[order].astype(np.uint32), np.asarray(vals, dtype=np.float32)[order]


class SparseOperator:
    """A plan registered for use from torch ops.  Keeps the plan (and, once a backward pass has run, the plan of
    A^T) alive until `close()` or garbage collection."""

    def __init__(self, plan: Plan, *, plan_kwargs: dict | None = None):
        self.plan = plan
        self.M, self.K, self.nnz = plan.M, plan.K, plan.nnz
        self._plan_kwargs = plan_kwargs or {}
        self._transposed: Plan | None = None
        self._t_perm: torch.Tensor | None = None  # storage position in A of every stored position of A^T
        self.id = next(_ids)
        _plans[self.id] = self
        weakref.finalize(self, _plans.pop, self.id, None)

    def transposed(self) -> Plan:
        if self._transposed is None:
            rp, cols, vals = self.plan.decode_csr()
            t_rp, t_cols, t_vals = transpose_csr(self.M, self.K, rp, cols, vals)
            self._transposed = Plan(self.K, self.M, t_rp, t_cols, t_vals, **self._plan_kwargs)
        return self._transposed

    def __call__(self, B: torch.Tensor) -> torch.Tensor:
        return torch.ops.cutespmm.spmm(self.id, B)

    def sddmm(self, X: torch.Tensor, Y: torch.Tensor, scale_by_values: bool = False) -> torch.Tensor:
        return torch.ops.cutespmm.sddmm(self.id, X, Y, scale_by_values)

    def weighted(self, w: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
        return torch.ops.cutespmm.spmm_weighted(self.id, w, B)

    def _transposed_with(self, w: torch.Tensor) -> Plan:
        """The plan of A^T carrying the weights w (given in this plan's storage order)."""
        if self._t_perm is None:
            rp, cols, _ = self.plan.decode_csr()
            self._t_perm = torch.from_numpy(np.argsort(np.asarray(cols, dtype=np.int64), kind="stable")).to(w.device)
        t = self.transposed()
        t.set_values(w.detach().contiguous()[self._t_perm])
        return t

    def set_values(self, vals: torch.Tensor) -> None:
        """New values for the same pattern (Plan.set_values), e.g. normalised `sddmm` scores as attention weights.  The
        plan of A^T, if a backward pass has built one, is dropped and rebuilt from the new values on next use."""
        self.plan.set_values(vals)
        if self._transposed is not None:
            self._transposed.close()
            self._transposed = None

    def close(self) -> None:
        _plans.pop(self.id, None)
        for p in (self.plan, self._transposed):
            if p is not None:
                p.close()


def register_plan(plan: Plan, **kw) -> int:
    """Registers `plan` and returns the id the ops take; the registry holds the only strong reference."""
    op = SparseOperator(plan, **kw)
    _keep[op.id] = op
    return op.id


def unregister_plan(plan_id: int) -> None:
    op = _keep.pop(plan_id, None) or _plans.get(plan_id)
    if op is not None:
        op.close()


_keep: dict[int, SparseOperator] = {}


def _get(plan_id: int) -> SparseOperator:
    try:
        return _plans[plan_id]
    except KeyError:
        raise RuntimeError(f"cutespmm: no plan registered under id {plan_id}") from None


@torch.library.custom_op("cutespmm::spmm", mutates_args=())
def _spmm(plan_id: int, B: torch.Tensor) -> torch.Tensor:
    op = _get(plan_id)
    Bc = B if B.stride(-1) == 1 else B.contiguous()
    return op.plan.spmm(Bc)


@_spmm.register_fake
def _(plan_id: int, B: torch.Tensor) -> torch.Tensor:
    return B.new_empty((_get(plan_id).M, B.shape[1]))


@torch.library.custom_op("cutespmm::spmm_transposed", mutates_args=())
def _spmm_t(plan_id: int, G: torch.Tensor) -> torch.Tensor:
    op = _get(plan_id)
    Gc = G if G.stride(-1) == 1 else G.contiguous()
    return op.transposed().spmm(Gc)


@_spmm_t.register_fake
def _(plan_id: int, G: torch.Tensor) -> torch.Tensor:
    return G.new_empty((_get(plan_id).K, G.shape[1]))


def _spmm_backward(ctx, grad_C):
    return None, torch.ops.cutespmm.spmm_transposed(ctx.plan_id, grad_C)


def _spmm_setup(ctx, inputs, output):
    ctx.plan_id = inputs[0]


_spmm.register_autograd(_spmm_backward, setup_context=_spmm_setup)
_spmm_t.register_autograd(lambda ctx, g: (None, torch.ops.cutespmm.spmm(ctx.plan_id, g)), setup_context=_spmm_setup)


@torch.library.custom_op("cutespmm::spmm_weighted", mutates_args=())
def _spmm_w(plan_id: int, w: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    op = _get(plan_id)
    op.plan.set_values(w.detach().contiguous())
    Bc = B if B.stride(-1) == 1 else B.contiguous()
    return op.plan.spmm(Bc)


@_spmm_w.register_fake
def _(plan_id: int, w: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    return B.new_empty((_get(plan_id).M, B.shape[1]))


@torch.library.custom_op("cutespmm::spmm_weighted_transposed", mutates_args=())
def _spmm_wt(plan_id: int, w: torch.Tensor, G: torch.Tensor) -> torch.Tensor:
    op = _get(plan_id)
    Gc = G if G.stride(-1) == 1 else G.contiguous()
    return op._transposed_with(w).spmm(Gc)


@_spmm_wt.register_fake
def _(plan_id: int, w: torch.Tensor, G: torch.Tensor) -> torch.Tensor:
    return G.new_empty((_get(plan_id).K, G.shape[1]))


def _spmm_w_setup(ctx, inputs, output):
    ctx.plan_id = inputs[0]
    ctx.save_for_backward(inputs[1], inputs[2])


def _spmm_w_backward(ctx, grad_C):
    w, B = ctx.saved_tensors
    grad_w = torch.ops.cutespmm.sddmm(ctx.plan_id, grad_C, B, False) if ctx.needs_input_grad[1] else None
    grad_B = torch.ops.cutespmm.spmm_weighted_transposed(ctx.plan_id, w, grad_C) if ctx.needs_input_grad[2] else None
    return None, grad_w, grad_B


_spmm_w.register_autograd(_spmm_w_backward, setup_context=_spmm_w_setup)


@torch.library.custom_op("cutespmm::sddmm", mutates_args=())
def _sddmm(plan_id: int, X: torch.Tensor, Y: torch.Tensor, scale_by_values: bool) -> torch.Tensor:
    op = _get(plan_id)
    Xc = X if X.stride(-1) == 1 else X.contiguous()
    Yc = Y if Y.stride(-1) == 1 else Y.contiguous()
    return op.plan.sddmm(Xc, Yc, scale_by_values=scale_by_values)


@_sddmm.register_fake
def _(plan_id: int, X: torch.Tensor, Y: torch.Tensor, scale_by_values: bool) -> torch.Tensor:
    return X.new_empty((_get(plan_id).nnz,))
