"""Runs the reference project's own GPU path (oracle/_ref/libcutespmm_ref_gpu.so, built by oracle/Makefile from the
reference sources) on one of the synthetic workloads, in a process of its own, and prints one JSON line:

    python oracle/ref_gpu_run.py --workload stencil512 --N 128
    python oracle/ref_gpu_run.py --mtx some/matrix.mtx --N 128      (pattern of a MatrixMarket file, values 1.0, as run.cu reads it)

A separate process on purpose: the reference's host code ends the process on any CUDA error (chkerr, inc.h:61-69) and
indexes its occupancy table without checking the key, so a failure there must not take a benchmark run with it.
The result is checked against the CPU oracle before any time is reported.  MEASUREMENT INFRASTRUCTURE ONLY.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))


def sorted_pattern_from_mtx(g, path):
    """The file's pattern as the reference's own reader delivers it (IO.cu:10-87: values 1.0, dimensions padded to
    multiples of 16, symmetric files mirrored), with every row's columns sorted and duplicates dropped -- the order its
    preprocessing needs (data.cu:80-93)."""
    import numpy as np
    import torch

    import oracle

    M, K, nnz, rp, cols, vals = oracle.Ref().mtx_read(path)
    rows = np.repeat(np.arange(M, dtype=np.int64), np.diff(rp.astype(np.int64)))
    keys = np.unique(rows * K + cols.astype(np.int64))
    r, c = keys // K, (keys % K).astype(np.int32)
    row_ptr = np.zeros(M + 1, dtype=np.int64)
    np.cumsum(np.bincount(r, minlength=M), out=row_ptr[1:])
    return g.CsrMatrix(M, K, torch.from_numpy(row_ptr), torch.from_numpy(c), torch.ones(c.size, dtype=torch.float32), Path(path).stem)


def run_one(oracle, g, A, N, b_seed, b_dist, iters):
    """One (matrix, N): the JSON-able result of the reference's GPU path, checked against the CPU oracle."""
    if N not in (16, 32, 64, 128, 256, 512) or A.M % 16 or A.K % 16:
        return {"unavailable": "shape outside what the reference's launcher takes"}
    if (A.M // 16) * (A.K // 16) > (1 << 31):
        return {"unavailable": "the reference's preprocessing allocates (M/16)*(K/16) offsets (data.cu:91): too large for this matrix"}
    B = g.dense_operand(A.K, N, b_seed, b_dist).numpy()
    C, prep, cold, warm, flushed = oracle.ref_gpu_spmm(A.M, A.K, A.row_ptr, A.cols, A.vals, B, iters=iters)
    err = oracle.rel_fro(oracle.spmm_csr(A.row_ptr, A.cols, A.vals, B, A.M, A.K), C)
    if not err <= 1e-3:
        return {"unavailable": f"its result differs from the CPU oracle (relative Frobenius error {err:.3e}): not timed"}
    gf = lambda ms: round(2.0 * A.nnz * N / (ms * 1e-3) / 1e9, 1)  # noqa: E731
    return {"kernel": "SpMM<NUM_WARPS,ILP_LEVEL> (kernel.cu:119-288), TM=16 TN=4 Machine=0, built for sm_100a", "rel_fro": err,
            "ms_l2_flushed": round(flushed, 5), "gflops_l2_flushed": gf(flushed), "ms_l2_not_flushed": round(warm, 5),
            "gflops_l2_not_flushed": gf(warm), "ms_first_launch": round(cold, 5), "preprocessing_ms": round(prep, 1),
            "launches": 2 * iters + 1,
            "note": "each launch alone between CUDA events; C zeroed before every launch (not timed), as run.cu:43,49 does; "
                    "ms_l2_flushed follows this benchmark's own protocol (256 MiB write before each launch)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="", choices=["", "uniform4096", "stencil512", "elasticity40"])
    ap.add_argument("--mtx", default="", help="MatrixMarket file(s) instead of a named workload, comma-separated: one JSON line per (file, N)")
    ap.add_argument("--N", required=True, help="feature size(s), comma-separated")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    import oracle

    spec = importlib.util.spec_from_file_location("cutespmm_generators", HERE.parent / "cutespmm_ae_b200" / "generators.py")
    g = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = g
    spec.loader.exec_module(g)
    Ns = [int(x) for x in a.N.split(",")]
    if a.mtx:
        for f in a.mtx.split(","):
            A = sorted_pattern_from_mtx(g, f)
            for N in Ns:
                out = run_one(oracle, g, A, N, 4242, "normal", a.iters)
                out.update(matrix=Path(f).stem, N=N)
                print(json.dumps(out), flush=True)
        return
    w = g.WORKLOADS[a.workload]
    A = w["make"]()
    for N in Ns:
        out = run_one(oracle, g, A, N, w["b_seed"], w["b_dist"], a.iters)
        out.update(matrix=a.workload, N=N)
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
