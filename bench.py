#!/usr/bin/env python
"""Benchmark driver for the SpMM path:  C[M x N] = A_sparse[M x K] * B_dense[K x N].

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one product over one synthetic workload (seeded generators standing in for the
SuiteSparse matrices the reference measures on).  Metric: GFLOP/s = 2 * nnz * N / t, the formula of
the reference's report script (present_gflops.py:30-35).  One JSON line is printed by rank 0.

Default workload: the large power-law graph (R-MAT, 2^24 nodes, N = 128), strong scaling: the matrix
stays the same for every GPU count, its row panels are cut into nnz-balanced contiguous ranges, one per
rank (cutespmm_partition_rows), every rank builds a plan for its own rows, C stays row-sharded.

  value     device time of the product alone, B resident in every GPU's HBM, CUDA events per step on
            the launching stream, L2 flushed between steps, max over ranks;
  from_root / row_sharded (N > 1)
            the same step including the exchange of B through the library's communicator
            (cutespmm_spmm_sharded): broadcast from rank 0, or in-place all-gather of row slices;
  e2e       the same product through the host-buffer entry point (cutespmm_spmm_sharded_host):
            every rank uploads its slice of B from pinned host memory over its own PCIe link, the
            slices are exchanged over NVLink, C rows return to the host; all inside the timed region;
  roofline  algorithmic bytes (8*nnz + 4*(M+1) + 4*N*rows of B named + 4*M*N per rank) / device time
            against the measured HBM copy bandwidth of this machine class;
  parity    every rank checks a sample of its own rows of C against the CPU oracle;
  cpu_baseline  the CPU oracle (row-parallel port of the reference's spmm_coo) on the host cores;
  per_config (1 GPU) the same kernel-only figures for the other four configurations and for the
            block-structured matrix at N = 32, 64, 256.

`--impl reference` times the reference project's own CPU implementation of the product (its
spmm_coo compiled from the reference sources into oracle/_ref when available, else the oracle port)
on a bounded sample of the same workload, with the OpenMP thread count set explicitly.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

if "reference" in sys.argv:  # the CPU arm states its own thread count; a launcher may have exported OMP_NUM_THREADS=1
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_HBM_GBS = 6650.0
WORKLOADS = ["uniform4096", "stencil512", "elasticity40", "rmat20", "rmat22", "rmat24"]
# the other configurations reported beside the default one on a single GPU: (workload, N)
PER_CONFIG = [("uniform4096", 32), ("stencil512", 128), ("elasticity40", 32), ("elasticity40", 64), ("elasticity40", 128),
              ("elasticity40", 256), ("rmat20", 128)]


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="rmat24", choices=WORKLOADS)
    ap.add_argument("--N", type=int, default=0, help="columns of B (0 = the workload's own)")
    ap.add_argument("--path", default="auto", choices=["auto", "rows", "brick", "slab"])
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"])
    ap.add_argument("--no-flush", action="store_true", help="do not flush L2 between steps")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-per-config", action="store_true", help="skip the per_config block (1 GPU)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg")
    ap.add_argument("--sddmm", action="store_true", help="1 GPU: also time cutespmm_sddmm over the workload's plan (block \"sddmm\")")
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the host-buffer leg (0 = chosen by operand size)")
    ap.add_argument("--matrices", default="", help="a folder of MatrixMarket files: print the per-matrix table instead of the benchmark line")
    ap.add_argument("--no-reference-gpu", action="store_true", help="--matrices: skip the reference's own kernel")
    ap.add_argument("--reorder", default="none", choices=["none", "cluster", "similar"], help="plan-time reordering option")
    return ap.parse_args()


def load_generators():
    """The generators module by file path: importing the package would load libcutespmm.so, which the CPU reference
    arm must not have in its process."""
    spec = importlib.util.spec_from_file_location("cutespmm_generators", ROOT / "cutespmm_ae_b200" / "generators.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


# ----------------------------------------------------------------------------------------------
def make_matrix(g, workload: str, scale_factor: int, device):
    """The workload's A on `device`; scale_factor > 1 grows it for weak scaling.  Returns (A, N, seed of B, distribution of B)."""
    s = scale_factor
    if workload == "uniform4096":
        return g.uniform_random(4096 * s, 4096 * s, 16, 1001, device), 32, 2001, "uniform_pm1"
    if workload == "stencil512":
        return g.stencil9(512, 512 * s, 1002, device), 128, 2002, "normal"
    if workload == "elasticity40":
        n = round(40 * s ** (1.0 / 3.0))
        return g.elasticity3d(n, 3, 1003, device), 128, 2003, "normal"
    if workload.startswith("rmat"):
        scale = int(workload[4:]) + int(np.log2(s))
        vals = "rownorm" if workload == "rmat20" else "uniform"
        seed = {"rmat20": 1004, "rmat24": 1005}.get(workload, 1006)
        return g.rmat(scale, 8, seed=seed, values=vals, device=device), 128, seed + 1000, "normal"
    raise ValueError(workload)


def strided_rows(A, target_nnz: int):
    """A representative bounded sample of A's rows: every `stride`-th row, so that about target_nnz nonzeros are kept
    and the degree distribution (hub rows included) and the column distribution stay those of the whole matrix.
    Returns (sub-CSR on the CPU with the column space of A, stride)."""
    g = sys.modules.get("cutespmm_generators") or sys.modules.get("cutespmm_ae_b200.generators")
    stride = max(1, int(A.nnz // max(target_nnz, 1)))
    if stride == 1:
        return A.cpu(), 1
    rows = torch.arange(stride // 2, A.M, stride, device=A.row_ptr.device)
    lo, hi = A.row_ptr[rows], A.row_ptr[rows + 1]
    lens = hi - lo
    rp = torch.zeros(rows.numel() + 1, dtype=torch.int64, device=lens.device)
    torch.cumsum(lens, 0, out=rp[1:])
    total = int(rp[-1])
    idx = torch.repeat_interleave(lo - rp[:-1], lens, output_size=total) + torch.arange(total, device=lens.device)
    return g.CsrMatrix(rows.numel(), A.K, rp.cpu(), A.cols[idx].cpu(), A.vals[idx].cpu(), A.name + f"[::{stride}]"), stride


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def measured_hbm_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except (KeyError, ValueError):
            pass
    return FALLBACK_HBM_GBS, "fallback 6650 GB/s (no MEASURED_PEAKS.json)"


def dram_traffic_for(workload: str, N: int, path: str, world: int):
    """Per-launch DRAM bytes of the dominant kernel from the committed ncu capture of exactly this workload, N and path
    on one GPU; None where there is no such capture (never another shape's figure)."""
    if world != 1:
        return None
    f = ROOT / "profiles" / "dram_traffic.json"
    if not f.exists():
        return None
    try:
        table = json.loads(f.read_text())
    except ValueError:
        return None
    return table.get(f"{workload}:N{N}:{path}")


def bytes_model(nnz, M, N, b_rows):
    return 8 * nnz + 4 * (M + 1) + 4 * N * b_rows + 4 * M * N


# ----------------------------------------------------------------------------------------------
def cpu_baseline(A_dev, N, B_host_fn, budget_s=10.0):
    """Times the oracle port (row-parallel OpenMP over all host cores) on the workload or, when one pass would exceed
    the budget, on a strided sample of its rows."""
    import oracle

    cores = os.cpu_count() or 1
    threads = oracle.set_threads(cores)

    def arrays(sub):
        return sub.row_ptr.numpy().astype(np.uint64), sub.cols.numpy().astype(np.uint32), sub.vals.numpy()

    B = B_host_fn()
    sub, stride = strided_rows(A_dev, min(A_dev.nnz, 2_000_000))
    rp, cols, vals = arrays(sub)
    oracle.spmm_csr(rp, cols, vals, B, sub.M, sub.K)  # warm-up (page faults, thread pool)
    t0 = time.perf_counter()
    oracle.spmm_csr(rp, cols, vals, B, sub.M, sub.K)
    rate = sub.nnz / max(time.perf_counter() - t0, 1e-6)  # nonzeros per second
    if stride > 1:  # size the sample so that one pass takes about budget/4 seconds
        sub, stride = strided_rows(A_dev, int(min(A_dev.nnz, max(2_000_000, rate * budget_s / 4))))
        rp, cols, vals = arrays(sub)
    reps, t_total = 0, 0.0
    while reps < 3 or (t_total < 2.0 and reps < 20):
        t0 = time.perf_counter()
        oracle.spmm_csr(rp, cols, vals, B, sub.M, sub.K)
        t_total += time.perf_counter() - t0
        reps += 1
        if t_total > budget_s:
            break
    gflops = 2.0 * sub.nnz * N * reps / t_total / 1e9
    sample = "whole workload" if stride == 1 else f"every {stride}th row: {sub.M} of {A_dev.M} rows, {sub.nnz} nonzeros"
    return {"value": round(gflops, 3), "unit": "GFLOP/s", "cores": threads, "kind": "port",
            "sample": f"{sample}, {reps} passes, OpenMP static over rows, {threads} threads"}


def run_reference(args):
    """--impl reference: the reference's CPU product on a bounded sample, rank 0 only.  Neither the package nor its
    shared library is imported here."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle

    g = load_generators()
    dev = torch.device("cuda", 0) if torch.cuda.is_available() and args.workload in ("rmat22", "rmat24") else torch.device("cpu")
    A, N, b_seed, b_dist = make_matrix(g, args.workload, 1, dev)  # inputs only: the timed routine below is CPU code
    N = args.N or N
    cores = os.cpu_count() or 1
    use_ref = oracle.ref_available()
    # bounded sample: the reference's spmm_coo opens an OpenMP region per nonzero (inc.h:78-81), a cost per nonzero that
    # does not depend on N, so the sample is sized in nonzeros.
    target_nnz = 1 << 16 if use_ref else min(A.nnz, 1 << 21)
    sub, stride = strided_rows(A, target_nnz)
    M_full, K, nnz_full = A.M, A.K, A.nnz
    del A
    if dev.type == "cuda":
        torch.cuda.empty_cache()
    # only the rows of B the sample names are needed: build them from the counter-based generator, renumber the columns
    uniq, inv = torch.unique(sub.cols.long(), return_inverse=True)
    B = torch.empty((uniq.numel(), N), dtype=torch.float32)
    for u0 in range(0, uniq.numel(), 1 << 16):  # element (k, n) of B is a function of (seed, k*N + n), as in generators.dense_operand
        u = uniq[u0 : u0 + (1 << 16)]
        flat = (u[:, None] * N + torch.arange(N)[None, :]).reshape(-1)
        vals_b = g.normal01(flat, b_seed, 3) if b_dist == "normal" else 2.0 * g.uniform01(flat, b_seed, 3) - 1.0
        B[u0 : u0 + u.numel()] = vals_b.to(torch.float32).view(u.numel(), N)
    B = B.numpy()
    rp = sub.row_ptr.numpy().astype(np.uint64)
    cols, vals = inv.numpy().astype(np.uint32), sub.vals.numpy()
    coo_rows = np.repeat(np.arange(sub.M, dtype=np.uint32), np.diff(rp.astype(np.int64)))
    Ksub = int(uniq.numel())
    if use_ref:
        R = oracle.Ref()
        fn = lambda: R.spmm_coo(coo_rows, cols, vals, B, sub.M, Ksub)  # noqa: E731
        set_threads, kind = R.set_threads, "reference"
    else:
        fn = lambda: oracle.spmm_csr(rp, cols, vals, B, sub.M, Ksub)  # noqa: E731
        set_threads, kind = oracle.set_threads, "port"

    def timed(threads):
        n = set_threads(threads)
        for _ in range(max(1, min(args.warmup, 3))):
            fn()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            fn()
        return n, (time.perf_counter() - t0) / args.steps

    # The routine forks a parallel region per nonzero, so more threads can make it slower: time it with every host
    # thread and with one, and report the faster as the value (both are stated).
    n_all, dt_all = timed(cores)
    n_one, dt_one = timed(1) if kind == "reference" and cores > 1 else (n_all, dt_all)
    dt, n_used = (dt_all, n_all) if dt_all <= dt_one else (dt_one, n_one)
    gf = lambda t: 2.0 * sub.nnz * N / t / 1e9  # noqa: E731
    line = {
        "impl": "reference", "metric": "spmm_gflops", "value": round(gf(dt), 4), "unit": "GFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "M": M_full, "K": K, "nnz": nnz_full, "N": N},
        "cpu_baseline": {"value": round(gf(dt), 4), "unit": "GFLOP/s", "cores": n_used, "kind": kind,
                         "sample": (f"every {stride}th row ({sub.M} rows, {sub.nnz} nonzeros) per step; "
                                    + ("spmm_coo compiled from the reference sources (inc.h:71-83)" if use_ref
                                       else "oracle port, OpenMP static over rows")
                                    + f"; OMP threads {n_all}: {gf(dt_all):.4f} GFLOP/s, OMP threads {n_one}: {gf(dt_one):.4f} GFLOP/s")},
        "e2e": {"value": round(gf(dt), 4), "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
def build_plan(cs, A_dev, path_name: str, reorder: str, flags: dict | None = None):
    """A plan over the rows of A_dev (CSR on the GPU), built from the device arrays where the device builder takes the
    request and by the host builder otherwise.  Returns (plan, milliseconds, builder name)."""
    path = {"auto": cs.PATH_AUTO, "rows": cs.PATH_ROWS, "brick": cs.PATH_BRICK, "slab": cs.PATH_SLAB}[path_name]
    kw = dict(flags or {})
    if reorder != "none":
        kw["reorder"] = reorder
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    plan = None
    if A_dev.nnz and not kw and A_dev.nnz < 2**32 and path_name != "slab":
        try:
            plan = cs.Plan.from_device_csr(A_dev.M, A_dev.K, A_dev.row_ptr.to(torch.int32), A_dev.cols.to(torch.int32).contiguous(),
                                           A_dev.vals.contiguous(), path=path)
            how = "device"
        except cs.CuteSpmmError as e:
            if e.status != -4:  # anything but "the device builder does not take this request"
                raise
    if plan is None:
        plan = cs.Plan.from_csr(A_dev.cpu(), path=path, **kw)
        how = "host"
    torch.cuda.synchronize()
    return plan, (time.perf_counter() - t0) * 1e3, how


def time_steps(step, steps, warmup, flush, dist, dev):
    """W warm-up steps, then `steps` steps each between its own CUDA events (L2 flushed before each), max over ranks.
    Returns (ms per step, median, min)."""
    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    torch.cuda.synchronize()
    for a, b in evs:
        if flush is not None:
            flush.fill_(1)
        a.record()
        step()
        b.record()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    per = np.array([a.elapsed_time(b) for a, b in evs])
    t = torch.tensor([per.sum(), np.median(per), per.min()], device=dev, dtype=torch.float64)
    if dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total, med, mn = (float(x) for x in t)
    return total / steps, med, mn


def parity_sample(A_dev, B, C, n_random=1 << 13, n_longest=8, seed=7):
    """Rows of C checked against the CPU oracle: a random sample of this rank's rows plus its longest ones.  Only the
    rows of B those rows name travel to the host.  Returns (relative Frobenius error, rows checked)."""
    import oracle

    if A_dev.M == 0 or A_dev.nnz == 0:
        return 0.0, 0
    dev = A_dev.row_ptr.device
    deg = A_dev.row_ptr[1:] - A_dev.row_ptr[:-1]
    gen = torch.Generator().manual_seed(seed)
    which = torch.cat([torch.randint(0, A_dev.M, (min(n_random, A_dev.M),), generator=gen).to(dev),
                       torch.topk(deg, min(n_longest, A_dev.M)).indices])
    which = torch.unique(which)
    lo, lens = A_dev.row_ptr[which], deg[which]
    rp = torch.zeros(which.numel() + 1, dtype=torch.int64, device=dev)
    torch.cumsum(lens, 0, out=rp[1:])
    total = int(rp[-1])
    idx = torch.repeat_interleave(lo - rp[:-1], lens, output_size=total) + torch.arange(total, device=dev)
    uniq, inv = torch.unique(A_dev.cols[idx].long(), return_inverse=True)
    want = oracle.spmm_csr(rp.cpu().numpy().astype(np.uint64), inv.cpu().numpy().astype(np.uint32), A_dev.vals[idx].cpu().numpy(),
                           B[uniq].cpu().numpy(), which.numel(), uniq.numel())
    return oracle.rel_fro(want, C[which].cpu().numpy()), int(which.numel())


def measure_config(cs, g, workload, N, path_name, steps, dev, flush, peak, reference_gpu=True):
    """Kernel-only figures of one single-GPU configuration (the per_config block)."""
    A, N0, b_seed, b_dist = make_matrix(g, workload, 1, dev)
    N = N or N0
    plan, plan_ms, how = build_plan(cs, A, path_name, "none")
    B = g.dense_operand(A.K, N, b_seed, b_dist, device=dev)
    C = torch.empty((A.M, N), dtype=torch.float32, device=dev)
    ms, med, mn = time_steps(lambda: plan.spmm(B, C), steps, 3, flush, None, dev)
    err, rows = parity_sample(A, B, C, n_random=1 << 11)
    Bh = torch.empty((A.K, N), dtype=torch.float32).pin_memory()
    Bh.copy_(B)
    Ch = torch.empty((A.M, N), dtype=torch.float32).pin_memory()
    plan.spmm_host(Bh, Ch)
    t0 = time.perf_counter()
    for _ in range(3):
        plan.spmm_host(Bh, Ch)
    e2e_ms = (time.perf_counter() - t0) / 3 * 1e3
    balg = bytes_model(A.nnz, A.M, N, A.K)
    ach = balg / (ms * 1e-3) / 1e9
    info = plan.info()
    out = {"workload": workload, "N": N, "nnz": A.nnz, "path": plan.kernels(N), "ms_per_step": round(ms, 5),
           "ms_min": round(mn, 5), "gflops": round(2.0 * A.nnz * N / (ms * 1e-3) / 1e9, 1),
           "roofline": {"bound": "hbm", "achieved": round(ach, 1), "peak": peak, "unit": "GB/s", "frac": round(ach / peak, 4),
                        "traffic": dram_traffic_for(workload, N, path_name, 1)},
           "e2e_ms_per_step": round(e2e_ms, 3), "e2e_gflops": round(2.0 * A.nnz * N / (e2e_ms * 1e-3) / 1e9, 1),
           "plan_create_ms": round(plan_ms, 1), "plan_builder": how, "rel_fro_sample": err, "rows_checked": rows}
    if (workload, N) in (("stencil512", 128), ("rmat20", 128)):  # the operator next to the product in a graph layer
        del Bh, Ch
        out["sddmm"] = measure_sddmm(plan, A, B, steps, dev, flush, peak)
    plan.close()
    # the reference's own kernel on the same GPU, for context (its preprocessing cannot hold the two R-MAT configurations)
    if reference_gpu and workload in ("uniform4096", "stencil512", "elasticity40"):
        del B, C
        torch.cuda.empty_cache()
        out["reference_gpu"] = reference_gpu_block(workload, N)
    return out


def measure_sddmm(plan, A, Y, steps, dev, flush, peak, n_random=1 << 11, seed=11):
    """cutespmm_sddmm over the same plan and dense operand (Y = B, X = a second dense matrix): device time per call, the
    algorithmic bytes it stands for (A as CSR once, X once, the rows of Y the pattern names once, one float out per
    nonzero) and a sample of rows checked against the CPU oracle."""
    import oracle
    from cutespmm_ae_b200 import generators as g

    N = Y.shape[1]
    X = g.dense_operand(A.M, N, 9099, "normal", device=dev)
    out = torch.empty(A.nnz, dtype=torch.float32, device=dev)
    ms, _, mn = time_steps(lambda: plan.sddmm(X, Y, out, scale_by_values=True), steps, 3, flush, None, dev)
    gen = torch.Generator().manual_seed(seed)
    which = torch.unique(torch.randint(0, A.M, (min(n_random, A.M),), generator=gen).to(dev))
    deg = A.row_ptr[1:] - A.row_ptr[:-1]
    lo, lens = A.row_ptr[which], deg[which]
    rp = torch.zeros(which.numel() + 1, dtype=torch.int64, device=dev)
    torch.cumsum(lens, 0, out=rp[1:])
    total = int(rp[-1])
    idx = torch.repeat_interleave(lo - rp[:-1], lens, output_size=total) + torch.arange(total, device=dev)
    uniq, inv = torch.unique(A.cols[idx].long(), return_inverse=True)
    want = oracle.sddmm_csr(rp.cpu().numpy().astype(np.uint64), inv.cpu().numpy().astype(np.uint32), A.vals[idx].cpu().numpy(),
                            X[which].cpu().numpy(), Y[uniq].cpu().numpy())
    got = out[idx].cpu().numpy()
    err = float(np.linalg.norm(want.astype(np.float64) - got) / max(np.linalg.norm(want.astype(np.float64)), 1e-30))
    balg = 8 * A.nnz + 4 * (A.M + 1) + 4 * N * A.M + 4 * N * min(A.K, A.nnz) + 4 * A.nnz
    ach = balg / (ms * 1e-3) / 1e9
    return {"ms_per_step": round(ms, 5), "ms_min": round(mn, 5), "gflops": round(2.0 * A.nnz * N / (ms * 1e-3) / 1e9, 1),
            "roofline": {"bound": "hbm", "achieved": round(ach, 1), "peak": peak, "unit": "GB/s", "frac": round(ach / peak, 4), "traffic": None},
            "rel_err_sample": err, "nonzeros_checked": total, "gpu_launches_per_call": 1}


def reference_gpu_blocks(workload, Ns, mtx_files=None, timeout=600):
    """The reference project's GPU path (its HRPB preprocessing, work list and kernel SpMM<NUM_WARPS, ILP_LEVEL>,
    kernel.cu:119-288) built for sm_100a into oracle/_ref by oracle/Makefile, run by oracle/ref_gpu_run.py in a process
    of its own (the reference's host code exits on errors): results checked against the CPU oracle first, then timed.
    Returns {(matrix name, N): block}; a (matrix, N) the process did not reach is missing."""
    if not (ROOT / "oracle" / "_ref" / "libcutespmm_ref_gpu.so").exists():
        return {None: {"unavailable": "oracle/_ref/libcutespmm_ref_gpu.so is not built (needs a checkout of the reference next to this repository)"}}
    what = ["--mtx", ",".join(str(f) for f in mtx_files)] if mtx_files else ["--workload", workload]
    try:
        res = subprocess.run([sys.executable, str(ROOT / "oracle" / "ref_gpu_run.py"), *what, "--N", ",".join(str(n) for n in Ns)],
                             capture_output=True, text=True, timeout=timeout)
        out, code, err = res.stdout, res.returncode, res.stderr
    except subprocess.TimeoutExpired as e:
        out, code, err = (e.stdout or b"").decode() if isinstance(e.stdout, bytes) else (e.stdout or ""), -1, f"did not finish within {timeout} s"
    blocks = {}
    for ln in out.splitlines():
        if ln.startswith("{"):
            d = json.loads(ln)
            blocks[(d.pop("matrix"), d.pop("N"))] = d
    if code != 0:
        tail = (err or "").strip().splitlines()[-1:] or [""]
        blocks[None] = {"unavailable": f"the reference's GPU path ended with code {code}: {tail[0][:200]}"}
    return blocks


def reference_gpu_block(workload, N):
    blocks = reference_gpu_blocks(workload, [N], timeout=240)
    return blocks.get((workload, N)) or blocks.get(None) or {"unavailable": "no result"}


def run_ours(args):
    import cutespmm_ae_b200 as cs
    from cutespmm_ae_b200 import generators as g

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: libcutespmm has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    if args.gpus != world and rank == 0:
        print(f"note: --gpus {args.gpus} but WORLD_SIZE={world}; using {world}", file=sys.stderr)

    grow = world if args.scaling == "weak" else 1
    A, N, b_seed, b_dist = make_matrix(g, args.workload, grow, dev)
    N = args.N or N
    M, K, nnz = A.M, A.K, A.nnz
    name = A.name

    # nnz-balanced contiguous row ranges, one per rank; each rank plans its own rows only
    bounds = cs.partition_rows(A.row_ptr.cpu(), world, align_rows=16, row_cost=2) if world > 1 else np.array([0, M], dtype=np.uint64)
    r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
    mine = A.row_slice(r0, r1) if world > 1 else A
    if world > 1:  # keep this rank's rows only
        mine = g.CsrMatrix(mine.M, mine.K, mine.row_ptr.clone(), mine.cols.clone(), mine.vals.clone(), mine.name)
    del A
    torch.cuda.empty_cache()
    plan, plan_ms, plan_how = build_plan(cs, mine, args.path, args.reorder)
    info = plan.info()
    comm = cs.Comm.from_torch() if world > 1 else None

    # B: every rank generates the same B from the counter-based generator (the steady state of an iterative use);
    # the exchange legs below move it again through the library's communicator
    B = g.dense_operand(K, N, b_seed, b_dist, device=dev)
    C = torch.empty((mine.M, N), dtype=torch.float32, device=dev)
    flush = None if args.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    peak, peak_src = measured_hbm_peak()
    sampler = ClockSampler(local).start() if rank == 0 else None
    wall0 = time.perf_counter()
    ms_per_step, med_ms, min_ms = time_steps(lambda: plan.spmm(B, C), args.steps, args.warmup, flush, dist, dev)
    wall = time.perf_counter() - wall0
    clocks = sampler.stop() if sampler else None
    status = plan.device_status()
    if status != 0:
        raise SystemExit(f"device status word is {status}: a bounded wait ran out")
    sddmm_block = measure_sddmm(plan, mine, B, min(args.steps, 20), dev, flush, peak) if (args.sddmm and world == 1) else None
    # the same steps back to back without the flush (whatever the previous step left in L2 stays): reported beside the
    # flushed figure, never instead of it
    warm_ms = None
    if flush is not None:
        n_w = min(args.steps, 20)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_w):
            plan.spmm(B, C)
        e1.record()
        torch.cuda.synchronize()
        t_w = torch.tensor([e0.elapsed_time(e1) / n_w], device=dev)
        if dist:
            dist.all_reduce(t_w, op=dist.ReduceOp.MAX)
        warm_ms = float(t_w.item())

    # parity: every rank checks a sample of its own rows against the CPU oracle
    err, rows_checked = parity_sample(mine, B, C)
    t_p = torch.tensor([err, float(rows_checked)], device=dev, dtype=torch.float64)
    if dist:
        errs = [torch.zeros_like(t_p) for _ in range(world)]
        dist.all_gather(errs, t_p)
    else:
        errs = [t_p]
    parity = {"rel_fro_max": max(float(e[0]) for e in errs), "rows_checked": int(sum(float(e[1]) for e in errs)),
              "rel_fro_by_rank": [float(f"{float(e[0]):.3e}") for e in errs], "tolerance": 1e-3,
              "checker": "CPU oracle (oracle/spmm_oracle.c) on a random sample of each rank's rows plus its longest rows"}
    if not parity["rel_fro_max"] <= 1e-3:
        raise SystemExit(f"parity failed: {parity}")

    # the exchange legs: B from rank 0 (broadcast) and B row-sharded (in-place all-gather), each followed by the product
    exchange = {}
    if dist:
        n_p = min(args.steps, 5)
        Cx = torch.empty_like(C)
        even = np.minimum(np.arange(world + 1, dtype=np.uint64) * np.uint64(-(-K // world)), np.uint64(K))
        legs = {"from_root": lambda: plan.spmm_sharded(comm, B, Cx, b_mode=cs.B_FROM_ROOT, root=0),
                "row_sharded": lambda: plan.spmm_sharded(comm, B, Cx, b_mode=cs.B_ROW_SHARDED, b_bounds=even)}
        for leg, fn in legs.items():
            Cx.fill_(float("nan"))
            fn()  # warm-up
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n_p):
                fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / n_p], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if not torch.equal(Cx, C):
                raise SystemExit(f"{leg}: the product behind the exchange differs from the resident-B product")
            exchange[leg] = {"ms_per_step": round(float(t.item()), 3), "value": round(2.0 * nnz * N / (float(t.item()) * 1e-3) / 1e9, 2),
                             "unit": "GFLOP/s", "exchanged_bytes_per_rank": K * N * 4}
        del Cx
        # the broadcast alone, for reference
        dist.broadcast(B, 0)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dist.broadcast(B, 0)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        exchange["bcast_ms"] = round(float(t.item()), 3)

    # end to end through the host-buffer entry point: every rank uploads only its slice of B from pinned host memory,
    # the slices meet over NVLink, every rank's rows of C return to its host buffer
    e2e = None
    Bh_full = None
    if not args.no_e2e:
        even = np.minimum(np.arange(world + 1, dtype=np.uint64) * np.uint64(-(-K // world)), np.uint64(K))
        k0, k1 = int(even[rank]), int(even[rank + 1])
        Bh = torch.empty((k1 - k0, N), dtype=torch.float32).pin_memory()
        Bh.copy_(B[k0:k1])
        if world == 1:
            Bh_full = Bh
        Ch = torch.empty((mine.M, N), dtype=torch.float32).pin_memory()
        op_bytes = (K + M) * N * 4
        e2e_steps = args.e2e_steps or (3 if op_bytes > (4 << 30) else min(args.steps, 10))
        plan.spmm_sharded_host(comm, Bh, even, Ch)
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        t0 = time.perf_counter()
        kms = xms = 0.0
        for _ in range(e2e_steps):
            _, k_, x_ = plan.spmm_sharded_host(comm, Bh, even, Ch)  # returns after this rank's stream has been synchronised
            kms, xms = kms + k_, xms + x_
        if dist:
            dist.barrier()  # the step is over when the slowest rank has its rows
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        t_e = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
        if dist:
            dist.all_reduce(t_e, op=dist.ReduceOp.MAX)
        e2e_s = float(t_e.item())
        got = Ch[: min(mine.M, 4096)].to(dev).double()
        if mine.M and not float((got - C[: got.shape[0]].double()).norm()) <= 1e-5 * float(got.norm()) + 1e-30:
            raise SystemExit("the host-buffer product differs from the device-resident one")
        check = float(Ch.double().abs().sum())  # the device->host result is consumed
        e2e = {"value": round(2.0 * nnz * N / e2e_s / 1e9, 2), "unit": "GFLOP/s", "h2d_bytes_per_step": K * N * 4,
               "d2h_bytes_per_step": M * N * 4, "ms_per_step": round(e2e_s * 1e3, 3), "steps": e2e_steps,
               "kernel_ms": round(kms / e2e_steps, 3), "exchange_ms": round(xms / e2e_steps, 3), "checksum": check,
               "copies": f"each of {world} rank(s) uploads K/{world} rows of B and downloads its own rows of C"}
        if world > 1:
            del Bh, Ch

    flops = 2.0 * nnz * N
    gflops = flops / (ms_per_step * 1e-3) / 1e9
    # roofline of the dominant kernel, per rank (all ranks run the same kernel on shards of equal cost): a shard reads
    # only the rows of B its columns name
    distinct_cols = int(torch.unique(mine.cols).numel()) if world > 1 else K
    bytes_alg = bytes_model(mine.nnz, mine.M, N, min(K, distinct_cols))
    achieved = bytes_alg / (ms_per_step * 1e-3) / 1e9
    gather_bytes = 8 * mine.nnz + 4 * (mine.M + 1) + 4 * N * mine.nnz + 4 * mine.M * N
    line = {
        "metric": "spmm_gflops", "value": round(gflops, 2), "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "M": M, "K": K, "nnz": nnz, "N": N, "path": args.path, "kernels": plan.kernels(N), "reorder": args.reorder,
                   "matrix": name, "rows_per_rank": [int(bounds[i + 1] - bounds[i]) for i in range(world)],
                   "l2": "not flushed" if args.no_flush else "flushed between steps (256 MiB write)",
                   "operands_bytes": bytes_alg, "parallelism": f"row panels over {world} GPU(s), B resident in every GPU, C row-sharded"},
        "ms_median": round(med_ms, 5), "ms_min": round(min_ms, 5), "ms_per_step_l2_not_flushed": None if warm_ms is None else round(warm_ms, 5),
        "wall_ms_per_step": round(wall * 1e3 / (args.steps + max(args.warmup, 3)), 4),
        "plan_create_ms": round(plan_ms, 1), "plan_builder": plan_how,
        "plan": {k: info[k] for k in ("num_tiles", "num_long_rows", "num_chunks", "brick_panels", "num_bricks", "device_bytes")},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                     "traffic": dram_traffic_for(args.workload, N, args.path, world), "peak_source": peak_src,
                     "bytes_model": "8*nnz + 4*(M+1) + 4*N*min(K, distinct columns) + 4*M*N per launch and rank (A as CSR once, the rows of B it names once, C once)",
                     "frac_of_8TBs_nominal": round(achieved / 8000.0, 4),
                     # secondary model for matrices whose B cannot live in L2: every nonzero fetches its row of B (no reuse)
                     "gather_model_bytes": gather_bytes, "gather_model_GBs": round(gather_bytes / (ms_per_step * 1e-3) / 1e9, 1)},
        "parity": parity,
        "gpu_launches": args.steps * plan.launch_count(N),
        "clocks": clocks,
    }
    if e2e is not None:
        line["e2e"] = e2e
    if exchange:
        line["bcast_ms"] = exchange.pop("bcast_ms")
        line["bcast_bytes"] = K * N * 4
        line.update(exchange)
    if rank == 0 and not args.no_cpu:
        def b_host():
            return Bh_full.numpy() if Bh_full is not None else B.cpu().numpy()
        line["cpu_baseline"] = cpu_baseline(mine, N, b_host)
        if world > 1:
            line["cpu_baseline"]["sample"] += f"; rows of rank 0's shard ({mine.M} rows)"
    if dist:
        dist.barrier()
    if sddmm_block is not None:
        line["sddmm"] = sddmm_block
    if world == 1 and not args.no_per_config:
        del C, Bh_full
        plan.close()
        del B
        torch.cuda.empty_cache()
        per = []
        for wl, n in PER_CONFIG:
            if wl == args.workload and n == N:
                continue
            per.append(measure_config(cs, g, wl, n, "auto", min(args.steps, 20), dev, flush, peak))
            torch.cuda.empty_cache()
        line["per_config"] = per
    if rank == 0:
        print(json.dumps(line), flush=True)
    if comm is not None:
        comm.close()
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def run_matrices(args):
    """--matrices DIR: the table the reference's report script prints (present_gflops.py:36-42: matrix, N, GFLOP/s of its
    kernel and of a baseline) over the MatrixMarket files under DIR, N in {32, 128, 512} (run.cu:16).  Every file is
    read the way run.cu reads it (pattern only, values 1.0, padded to multiples of 16; rows then sorted); the product is
    checked on sampled rows against the CPU oracle; beside this library's figure stands the reference's own kernel on
    the same GPU, L2 flushed before every launch for both, where oracle/_ref holds it."""
    import cutespmm_ae_b200 as cs
    from cutespmm_ae_b200 import generators as g

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: libcutespmm has no CPU path")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    files = sorted(Path(args.matrices).glob("**/*.mtx"))
    if not files:
        raise SystemExit(f"no .mtx files under {args.matrices}")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ref_blocks = {None: {"unavailable": "skipped (--no-reference-gpu)"}} if args.no_reference_gpu else \
        reference_gpu_blocks("", (32, 128, 512), mtx_files=files, timeout=1200)  # one process for all files
    print("matrix, rows, nnz, N(feature size), path, GFLOPS, relFro (sampled rows), reference kernel GFLOPS (same GPU), ratio")
    table = []
    for f in files:
        r = cs.MtxReader(f, pattern_only=True)
        rows = np.repeat(np.arange(r.M, dtype=np.int64), np.diff(r.rowPtr.astype(np.int64)))
        keys = np.unique(rows * r.K + r.cols.astype(np.int64))  # rows sorted, duplicates dropped (what HRPB needs, data.cu:80-93)
        rr, cc = keys // r.K, (keys % r.K).astype(np.int32)
        rp = np.zeros(r.M + 1, dtype=np.int64)
        np.cumsum(np.bincount(rr, minlength=r.M), out=rp[1:])
        A = g.CsrMatrix(r.M, r.K, torch.from_numpy(rp).to(dev), torch.from_numpy(cc).to(dev), torch.ones(cc.size, dtype=torch.float32, device=dev), f.stem)
        plan, _, _ = build_plan(cs, A, args.path, args.reorder)
        info = plan.info()
        for N in (32, 128, 512):
            B = g.dense_operand(A.K, N, 4242, "normal", device=dev)
            C = torch.empty((A.M, N), dtype=torch.float32, device=dev)
            ms, _, _ = time_steps(lambda: plan.spmm(B, C), 10, 3, flush, None, dev)
            err, _ = parity_sample(A, B, C, n_random=1 << 10)
            gf = 2.0 * A.nnz * N / (ms * 1e-3) / 1e9
            ref = ref_blocks.get((f.stem, N)) or ref_blocks.get(None) or {"unavailable": "not reached"}
            ref_gf = ref.get("gflops_l2_flushed")
            kind = plan.kernels(N)
            row = {"matrix": f.stem, "rows": A.M, "nnz": A.nnz, "N": N, "path": kind, "gflops": round(gf, 1), "rel_fro": err,
                   "reference_gpu_gflops": ref_gf, "ratio": None if not ref_gf else round(gf / ref_gf, 2),
                   "reference_note": ref.get("unavailable")}
            table.append(row)
            print(f"{f.stem}, {A.M}, {A.nnz}, {N}, {kind}, {gf:.1f}, {err:.2e}, {ref_gf if ref_gf else 'n/a'}, {row['ratio'] if row['ratio'] else 'n/a'}", flush=True)
            if not err <= 1e-3:
                raise SystemExit(f"parity failed on {f}: {err}")
            del B, C
        plan.close()
        del A
        torch.cuda.empty_cache()
    ratios = [t["ratio"] for t in table if t["ratio"]]
    print(json.dumps({"metric": "spmm_gflops_table", "matrices": len(files), "rows": table,
                      "geomean_ratio_vs_reference_kernel": round(float(np.exp(np.mean(np.log(ratios)))), 3) if ratios else None}), flush=True)


def main():
    args = parse_args()
    if args.matrices:
        run_matrices(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
