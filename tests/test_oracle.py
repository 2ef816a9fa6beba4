"""The CPU oracle against the golden vectors the reference's own routines produced, and -- where
the reference build is present -- against those routines directly."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN_CASES, load_golden


def _coo_rows(rp):
    return np.repeat(np.arange(rp.size - 1, dtype=np.uint32), np.diff(rp.astype(np.int64)))


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_oracle_matches_reference_golden_bit_for_bit(oracle_mod, name):
    gd = load_golden(name)
    M, K = int(gd["M"]), int(gd["K"])
    c_coo = oracle_mod.spmm_coo(_coo_rows(gd["row_ptr"]), gd["cols"], gd["vals"], gd["B"], M, K)
    c_csr = oracle_mod.spmm_csr(gd["row_ptr"], gd["cols"], gd["vals"], gd["B"], M, K)
    assert np.array_equal(c_coo.view(np.uint32), gd["C"].view(np.uint32))
    assert np.array_equal(c_csr.view(np.uint32), gd["C"].view(np.uint32))


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_max_rel_err_matches_reference_golden(oracle_mod, name):
    gd = load_golden(name)
    assert oracle_mod.max_rel_err(gd["C"], gd["C_perturbed"]) == float(gd["max_rel_err"])
    assert oracle_mod.max_rel_err(gd["C"], gd["C"]) == 0.0


def test_rows_subset_equals_full(oracle_mod):
    gd = load_golden("rmat_s8")
    which = np.array([0, 3, 17, 255, 128], dtype=np.uint64)
    sub = oracle_mod.spmm_csr_rows(gd["row_ptr"], gd["cols"], gd["vals"], gd["B"], which)
    assert np.array_equal(sub, gd["C"][which.astype(np.int64)])


def test_rel_fro(oracle_mod):
    a = np.ones((4, 4), np.float32)
    b = a.copy()
    b[0, 0] = 2.0
    assert oracle_mod.rel_fro(a, a) == 0.0
    assert abs(oracle_mod.rel_fro(a, b) - 0.25) < 1e-12


def test_oracle_against_reference_build_if_present(oracle_mod):
    """Runs the reference's spmm_coo (compiled from its own sources) on a fresh random case."""
    if not oracle_mod.ref_available():
        pytest.skip("oracle/_ref not built on this machine (needs the reference tree)")
    from cutespmm_ae_b200 import generators as g

    R = oracle_mod.Ref()
    A = g.uniform_random(512, 384, 6, seed=99)
    B = g.dense_operand(A.K, 24, 98).numpy()
    rows = _coo_rows(A.row_ptr.numpy())
    ref = R.spmm_coo(rows, A.cols, A.vals, B, A.M, A.K)
    mine = oracle_mod.spmm_csr(A.row_ptr, A.cols, A.vals, B, A.M, A.K)
    assert np.array_equal(ref.view(np.uint32), mine.view(np.uint32))
    pert = mine * np.float32(1.001)
    assert R.max_rel_err(ref, pert) == oracle_mod.max_rel_err(mine, pert)
