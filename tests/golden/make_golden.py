"""Generates the golden fixtures in this directory from the REFERENCE project's own host routines.

    python tests/golden/make_golden.py          (needs oracle/_ref, i.e. `make -C oracle ref`)

For every case the inputs are stored next to what the reference computed from them:
  * C = spmm_coo(...)                      (reference inc.h:71-83)
  * check_gemm_correctness_coo(C, C')      (reference inc.h:84-110) for a perturbed C'
  * HRPB blockedRowPtr / activeCols        (reference data.cu:80-335), where the input meets its
    preconditions (M, K multiples of 16, ascending unique columns)
  * MTX_READER output                      (reference IO.cu:10-87) for the .mtx files written here
The fixtures are small on purpose (tens of KB each); the tests read only these files, never the
reference tree.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import oracle  # noqa: E402
from cutespmm_ae_b200 import generators as g  # noqa: E402

OUT = Path(__file__).resolve().parent


def coo_rows(A):
    return torch.repeat_interleave(torch.arange(A.M), A.row_ptr[1:] - A.row_ptr[:-1]).numpy().astype(np.uint32)


def save_case(R, name, A, N, b_seed, dist="normal", hrpb=True, shuffle_rows=False):
    rp = A.row_ptr.numpy().astype(np.uint64)
    cols = A.cols.numpy().astype(np.uint32).copy()
    vals = A.vals.numpy().astype(np.float32).copy()
    if shuffle_rows:  # unsorted columns inside rows (the order MTX_READER may produce)
        rng = np.random.default_rng(7)
        for r in range(A.M):
            j0, j1 = int(rp[r]), int(rp[r + 1])
            perm = rng.permutation(j1 - j0)
            cols[j0:j1] = cols[j0:j1][perm]
            vals[j0:j1] = vals[j0:j1][perm]
    B = g.dense_operand(A.K, N, b_seed, dist).numpy()
    rows = coo_rows(A)
    C = R.spmm_coo(rows, cols, vals, B, A.M, A.K)
    Cp = (C.astype(np.float64) * (1.0 + 1e-3 * np.sin(np.arange(C.size).reshape(C.shape)))).astype(np.float32)
    err = R.max_rel_err(C, Cp)
    d = dict(M=A.M, K=A.K, N=N, row_ptr=rp, cols=cols, vals=vals, B=B, C=C, C_perturbed=Cp, max_rel_err=np.float32(err))
    if hrpb:
        brp, ac, words = R.hrpb(A.M, A.K, rp.astype(np.uint32), cols, vals)
        d.update(blocked_row_ptr=brp, active_cols=ac, hrpb_stream_words=np.uint64(words))
    np.savez_compressed(OUT / f"{name}.npz", **d)
    print(name, "nnz", cols.size, "N", N, "max_rel_err", err)


def ragged(M=48, K=64, seed=5):
    """Empty rows, a full row, single-entry rows; M and K multiples of 16 so HRPB accepts it."""
    rng = np.random.default_rng(seed)
    rows = []
    for r in range(M):
        if r % 5 == 0:
            c = np.array([], dtype=np.int64)
        elif r == 7:
            c = np.arange(K)
        elif r % 3 == 0:
            c = np.array([rng.integers(K)])
        else:
            c = np.sort(rng.choice(K, size=rng.integers(1, 12), replace=False))
        rows.append(c)
    rp = np.zeros(M + 1, dtype=np.int64)
    rp[1:] = np.cumsum([len(c) for c in rows])
    cols = np.concatenate(rows).astype(np.int32)
    vals = rng.standard_normal(cols.size).astype(np.float32)
    return g.CsrMatrix(M, K, torch.from_numpy(rp), torch.from_numpy(cols), torch.from_numpy(vals), "ragged")


MTX_GENERAL = """%%MatrixMarket matrix coordinate real general
% a comment line
5 7 9
1 1 2.5
3 2 -1.0
3 7 4.0
2 2 1.5
5 1 3.0
3 1 0.5
1 7 -2.0
4 4 9.0
2 6 1.25
"""
MTX_SYMMETRIC = """%%MatrixMarket matrix coordinate pattern symmetric
20 20 8
1 1
5 2
7 7
20 1
13 4
6 5
19 18
20 20
"""


MTX_VALUES_UNSORTED = """%%MatrixMarket matrix coordinate real general
6 6 10
6 1 0.5
2 3 -1.25
1 1 4
2 1 3.5
4 4 7
2 2 -2
6 6 1e-3
5 2 2.5
1 6 9
3 3 -0.125
"""


def main():
    if not oracle.ref_available():
        raise SystemExit("oracle/_ref is not built: run `make -C oracle ref REF=<reference tree>`")
    R = oracle.Ref()
    save_case(R, "uniform_256", g.uniform_random(256, 256, 8, seed=11), 32, 21, "uniform_pm1")
    save_case(R, "stencil_16x16", g.stencil9(16, 16, seed=12), 16, 22)
    save_case(R, "elasticity_4", g.elasticity3d(4, 3, seed=13), 64, 23)  # M = 192
    save_case(R, "rmat_s8", g.rmat(8, 8, seed=14, values="uniform"), 8, 24)
    save_case(R, "ragged_48x64", ragged(), 40, 25)
    save_case(R, "uniform_256_unsorted", g.uniform_random(256, 256, 8, seed=11), 32, 21, "uniform_pm1", hrpb=False,
              shuffle_rows=True)
    for name, text in (("general_5x7", MTX_GENERAL), ("symmetric_20", MTX_SYMMETRIC)):
        path = OUT / f"{name}.mtx"
        path.write_text(text)
        M, K, nnz, rp, cols, vals = R.mtx_read(path)
        np.savez_compressed(OUT / f"mtx_{name}.npz", M=M, K=K, nnz=nnz, row_ptr=rp, cols=cols, vals=vals)
        print(name, M, K, nnz)
    # SparseCoo -> CSR_Matrix of the reference (inc/SparseCoo.hpp:91-157, inc/CSR.hpp:162-187)
    for name, text in (("general_5x7", None), ("symmetric_20", None), ("values_unsorted_6x6", MTX_VALUES_UNSORTED)):
        path = OUT / f"{name}.mtx"
        if text is not None:
            path.write_text(text)
        m, n, nnz, rp, cols, vals = R.csr_from_mtx(path)
        np.savez_compressed(OUT / f"loader_{name}.npz", nrows=m, ncols=n, nnz=nnz, row_ptr=rp, cols=cols, vals=vals)
        print("loader", name, m, n, nnz)


if __name__ == "__main__":
    main()
