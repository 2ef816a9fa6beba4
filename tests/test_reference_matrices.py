"""Regression sweep over the MatrixMarket files the reference project ships (its ae_matrices/ folder), on the
CPU: the loader, the plan's packed format and the reference-compatible views on real sparsity patterns.

Opt-in by presence: runs only where a checkout of the reference project is found (oracle.reference_root():
$CUTESPMM_REF, or a directory named "reference" beside this repository) and its host routines have been compiled into oracle/_ref; skipped everywhere else.  Nothing of those files
is stored in this repository.
"""
from pathlib import Path

import numpy as np
import pytest

import cutespmm_ae_b200 as cs


def _matrix_files():
    import oracle

    root = oracle.reference_root()
    if root and (root / "ae_matrices").is_dir():
        return sorted((root / "ae_matrices").glob("*/*.mtx"))
    return []


FILES = _matrix_files()
pytestmark = pytest.mark.skipif(not FILES, reason="the reference's ae_matrices/ folder is not mounted on this machine")


@pytest.fixture(scope="module")
def ref(oracle_mod):
    if not oracle_mod.ref_available():
        pytest.skip("oracle/_ref not built on this machine (needs the reference tree)")
    return oracle_mod.Ref()


def _sorted_unique(rp, cols):
    """True when every row's columns are strictly ascending (what HRPB needs, data.cu:80-93)."""
    d = np.diff(cols.astype(np.int64))
    starts = rp[1:-1].astype(np.int64)
    inside = np.ones(max(cols.size - 1, 0), dtype=bool)
    inside[starts[(starts > 0) & (starts < cols.size)] - 1] = False  # differences across a row boundary do not count
    return bool(np.all(d[inside] > 0))


@pytest.mark.parametrize("path", FILES, ids=[p.stem for p in FILES])
def test_loader_plan_and_views_on_reference_matrix(path, ref, oracle_mod):
    # a1: the loader against MTX_READER (IO.cu:10-87): padded dimensions, file order inside a row, all values 1.0
    M, K, nnz, rp, cols, vals = ref.mtx_read(path)
    r = cs.MtxReader(path)
    assert (r.M, r.K, r.nnz) == (M, K, nnz)
    assert np.array_equal(r.rowPtr, rp) and np.array_equal(r.cols, cols) and np.array_equal(r.vals, vals)

    # a2/a3: the plan's packed form decodes to the same matrix (as a linear map: rows may be unsorted in the
    # file and repeat an entry, so compare products with a small dense operand instead of the arrays)
    rp64 = rp.astype(np.uint64)
    rng = np.random.default_rng(int(nnz) % 9973)
    vals = rng.uniform(0.5, 1.5, size=nnz).astype(np.float32)  # distinct values, so that a misplaced one shows
    for p_path in (cs.PATH_AUTO, cs.PATH_ROWS):
        plan = cs.Plan(M, K, rp64, cols, vals, path=p_path, host_only=True)
        drp, dcols, dvals = plan.decode_csr()
        B = rng.standard_normal((K, 4)).astype(np.float32)
        want = oracle_mod.spmm_csr(rp64, cols, vals, B, M, K)
        got = oracle_mod.spmm_csr(drp, dcols, dvals, B, M, K)
        assert oracle_mod.rel_fro(want, got) <= 1e-6
        info = plan.info()
        assert info["nnz"] == nnz and info["M"] == M and info["K"] == K

    # b: blockedRowPtr / activeCols against the reference's own preprocessing, where its precondition holds
    if nnz and _sorted_unique(rp, cols):
        plan = cs.Plan(M, K, rp64, cols, vals, host_only=True)
        brp, ac, _ = ref.hrpb(M, K, rp, cols, vals)
        assert np.array_equal(plan.blocked_row_ptr(), brp)
        assert np.array_equal(plan.active_cols(), ac)
