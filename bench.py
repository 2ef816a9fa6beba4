#!/usr/bin/env python
"""Benchmark driver for the SpMM path:  C[M x N] = A_sparse[M x K] * B_dense[K x N].

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one product over one synthetic workload (seeded generators standing in for the
SuiteSparse matrices the reference measures on).  Metric: GFLOP/s = 2 * nnz * N / t, the formula of
the reference's report script (present_gflops.py:30-35).  One JSON line is printed by rank 0.

  value     device time of the product alone, operands resident in HBM, CUDA events per step on the
            launching stream, L2 flushed between steps, max over ranks;
  e2e       the same product through the host-buffer entry point (cutespmm_spmm_host): pinned host
            B in, host C out, copies inside the timed region;
  roofline  algorithmic bytes (8*nnz + 4*(M+1) + 4*K*N + 4*M*N) / device time against the measured
            HBM copy bandwidth of this machine class;
  cpu_baseline  the CPU oracle (row-parallel port of the reference's spmm_coo) on the host cores.

With more than one GPU (torchrun, one rank per GPU) the default is weak scaling: the matrix family
grows with the rank count, rows are cut into nnz-balanced contiguous ranges (cutespmm_partition_rows),
every rank builds a plan for its own rows, B is replicated into every GPU's HBM with one NCCL
broadcast (timed separately, `bcast_ms`), C stays row-sharded.  `--scaling strong` keeps the matrix
fixed instead.

`--impl reference` times the reference project's own CPU implementation of the product (its
spmm_coo compiled from the reference sources into oracle/_ref when available, else the oracle port)
on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="stencil512",
                    choices=["uniform4096", "stencil512", "elasticity40", "rmat20", "rmat22", "rmat24"])
    ap.add_argument("--N", type=int, default=0, help="columns of B (0 = the workload's own)")
    ap.add_argument("--path", default="auto", choices=["auto", "rows", "brick", "slab"])
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--no-flush", action="store_true", help="do not flush L2 between steps")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the host-buffer leg (0 = min(steps, 10))")
    return ap.parse_args()


# ----------------------------------------------------------------------------------------------
def make_matrix(workload: str, scale_factor: int, device):
    """The workload's A on `device`; scale_factor > 1 grows it for weak scaling."""
    from cutespmm_ae_b200 import generators as g

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


def dram_traffic_for(workload: str, path: str):
    """Per-launch DRAM bytes of the dominant kernel from the committed ncu capture, if there is one."""
    f = ROOT / "profiles" / "dram_traffic.json"
    if f.exists():
        try:
            return json.loads(f.read_text()).get(f"{workload}:{path}")
        except ValueError:
            return None
    return None


# ----------------------------------------------------------------------------------------------
def cpu_baseline(A_cpu, N, b_seed, b_dist, budget_s=12.0, max_rows=None):
    """Times the oracle port (row-parallel OpenMP over all host cores) on the workload or, when one
    pass would exceed the budget, on its leading rows."""
    import oracle
    from cutespmm_ae_b200 import generators as g

    cores = os.cpu_count() or 1
    M = A_cpu.M
    B = g.dense_operand(A_cpu.K, N, b_seed, b_dist).numpy()

    def slice_rows(target_nnz):
        rows = int(torch.searchsorted(A_cpu.row_ptr, torch.tensor(int(target_nnz))).item())
        rows = max(16, min(M, rows))
        if max_rows:
            rows = min(rows, max_rows)
        sub = A_cpu.row_slice(0, rows) if rows < M else A_cpu
        return sub, (sub.row_ptr.numpy().astype(np.uint64), sub.cols.numpy().astype(np.uint32), sub.vals.numpy())

    # probe on about 2 M nonzeros, then size the sample so that one pass takes about budget/4 seconds
    sub, (rp, cols, vals) = slice_rows(min(A_cpu.nnz, 2_000_000))
    oracle.spmm_csr(rp, cols, vals, B, sub.M, sub.K)  # warm-up (page faults, thread pool)
    t0 = time.perf_counter()
    oracle.spmm_csr(rp, cols, vals, B, sub.M, sub.K)
    rate = sub.nnz / max(time.perf_counter() - t0, 1e-6)  # nonzeros per second
    if sub.nnz < A_cpu.nnz:
        sub, (rp, cols, vals) = slice_rows(min(A_cpu.nnz, rate * budget_s / 4))
    rows = sub.M
    reps, t_total = 0, 0.0
    while reps < 3 or (t_total < 2.0 and reps < 20):
        t0 = time.perf_counter()
        oracle.spmm_csr(rp, cols, vals, B, sub.M, sub.K)
        t_total += time.perf_counter() - t0
        reps += 1
        if t_total > budget_s:
            break
    gflops = 2.0 * sub.nnz * N * reps / t_total / 1e9
    sample = "whole workload" if rows == M else f"leading {rows} of {M} rows ({sub.nnz} nonzeros)"
    return {"value": round(gflops, 3), "unit": "GFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{sample}, {reps} passes, OpenMP static over rows"}


def run_reference(args):
    """--impl reference: the reference's CPU product on a bounded sample, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    from cutespmm_ae_b200 import generators as g

    A, N, b_seed, b_dist = make_matrix(args.workload, 1, "cpu")
    N = args.N or N
    cores = os.cpu_count() or 1
    use_ref = oracle.ref_available()
    # bounded sample: the reference's spmm_coo opens an OpenMP region per nonzero (inc.h:78-81), a
    # cost per nonzero that does not depend on N, so the sample is sized in nonzeros.
    target_nnz = 1 << 16 if use_ref else min(A.nnz, 1 << 24)
    rows = int(torch.searchsorted(A.row_ptr, torch.tensor(target_nnz)).item())
    rows = max(16, min(A.M, rows))
    sub = A.row_slice(0, rows)
    B = g.dense_operand(A.K, N, b_seed, b_dist).numpy()
    rp = sub.row_ptr.numpy().astype(np.uint64)
    cols, vals = sub.cols.numpy().astype(np.uint32), sub.vals.numpy()
    coo_rows = np.repeat(np.arange(rows, dtype=np.uint32), np.diff(rp.astype(np.int64)))
    if use_ref:
        R = oracle.Ref()
        fn = lambda: R.spmm_coo(coo_rows, cols, vals, B, sub.M, sub.K)  # noqa: E731
        kind = "reference"
    else:
        fn = lambda: oracle.spmm_csr(rp, cols, vals, B, sub.M, sub.K)  # noqa: E731
        kind = "port"
    for _ in range(max(1, min(args.warmup, 2))):
        fn()
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / steps
    gflops = 2.0 * sub.nnz * N / dt / 1e9
    line = {
        "impl": "reference", "metric": "spmm_gflops", "value": round(gflops, 4), "unit": "GFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "M": A.M, "K": A.K, "nnz": A.nnz, "N": N},
        "cpu_baseline": {"value": round(gflops, 4), "unit": "GFLOP/s", "cores": cores, "kind": kind,
                         "sample": f"leading {rows} rows ({sub.nnz} nonzeros) per step; "
                                   + ("spmm_coo compiled from the reference sources (inc.h:71-83), OpenMP as written there"
                                      if use_ref else "oracle port, OpenMP static over rows")},
        "e2e": {"value": round(gflops, 4), "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
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
    A, N, b_seed, b_dist = make_matrix(args.workload, grow, dev)
    N = args.N or N
    M, K, nnz = A.M, A.K, A.nnz

    # nnz-balanced contiguous row ranges, one per rank; each rank plans its own rows only
    from cutespmm_ae_b200.sharded import ShardedSpmm

    path = {"auto": cs.PATH_AUTO, "rows": cs.PATH_ROWS, "brick": cs.PATH_BRICK, "slab": cs.PATH_SLAB}[args.path]
    t0 = time.perf_counter()
    shard = ShardedSpmm(A, path=path)
    plan_ms = (time.perf_counter() - t0) * 1e3
    del A
    plan, mine, bounds = shard.plan, shard.rows, shard.bounds
    info = plan.info()
    # a shard that runs on the row kernel only can also be planned from device-resident CSR: time that builder too
    plan_dev_ms = None
    if info["num_bricks"] == 0 and args.path in ("auto", "rows") and mine.nnz:
        d_rp, d_c, d_v = (mine.row_ptr.to(torch.int32).to(dev), mine.cols.to(torch.int32).to(dev), mine.vals.to(torch.float32).to(dev))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        pd = cs.Plan.from_device_csr(mine.M, mine.K, d_rp, d_c, d_v)
        plan_dev_ms = (time.perf_counter() - t0) * 1e3
        pd.close()
        del pd, d_rp, d_c, d_v

    # B: produced on rank 0, replicated into every GPU's own HBM by one NCCL broadcast
    bcast_ms = None
    if world > 1:
        B = g.dense_operand(K, N, b_seed, b_dist, device=dev) if rank == 0 else torch.empty((K, N), dtype=torch.float32, device=dev)
        dist.broadcast(B, 0)  # warm-up of the communicator
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dist.broadcast(B, 0)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        bcast_ms = float(t.item())
    else:
        B = g.dense_operand(K, N, b_seed, b_dist, device=dev)
    C = torch.empty((mine.M, N), dtype=torch.float32, device=dev)
    flush = None if args.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        plan.spmm(B, C)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    sampler = ClockSampler(local).start() if rank == 0 else None
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    torch.cuda.synchronize()
    wall0 = time.perf_counter()
    for a, b in evs:
        if flush is not None:
            flush.fill_(1)
        a.record()
        step()
        b.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall0
    if dist:
        dist.barrier()
    clocks = sampler.stop() if sampler else None
    per_step = np.array([a.elapsed_time(b) for a, b in evs])
    t_local = torch.tensor([per_step.sum(), np.median(per_step), per_step.min()], device=dev, dtype=torch.float64)
    if dist:
        dist.all_reduce(t_local, op=dist.ReduceOp.MAX)
    total_ms, med_ms, min_ms = (float(x) for x in t_local)
    ms_per_step = total_ms / args.steps
    if plan.device_status() != 0:
        raise SystemExit(f"device status word is {plan.device_status()}: a bounded wait ran out")
    # the same steps back to back without the flush (whatever the previous step left in L2 stays): reported beside the
    # flushed figure, never instead of it
    warm_ms = None
    if flush is not None:
        n_w = min(args.steps, 20)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_w):
            step()
        e1.record()
        torch.cuda.synchronize()
        t_w = torch.tensor([e0.elapsed_time(e1) / n_w], device=dev)
        if dist:
            dist.all_reduce(t_w, op=dist.ReduceOp.MAX)
        warm_ms = float(t_w.item())

    # B on rank 0 only: broadcast (whole, or in two column windows with each product queued behind its window), then the product
    from_root = None
    if dist:
        n_p = min(args.steps, 5)
        Cp = torch.empty_like(C)
        by_windows = {}
        for nwin in (1, 2):
            kw = dict(root=0, Cout=Cp, max_windows=nwin, min_cols=64, device=dev)
            shard.spmm_from_root(B if rank == 0 else None, N, **kw)  # warm-up
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n_p):
                shard.spmm_from_root(B if rank == 0 else None, N, **kw)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / n_p], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            by_windows[nwin] = float(t.item())
            if not torch.allclose(Cp, C, rtol=1e-3, atol=1e-3):
                raise SystemExit("the product behind the broadcast differs from the resident-B product")
        best = min(by_windows, key=by_windows.get)
        from_root = {"ms_per_step": round(by_windows[best], 3), "windows": best, "unit": "GFLOP/s",
                     "ms_by_windows": {str(k): round(v, 3) for k, v in by_windows.items()}}
        shard._recv.clear()
        del Cp

    # end to end through the host-buffer entry point: pinned host B in, host C out, every step
    e2e_steps = args.e2e_steps or min(args.steps, 10)
    Bh = torch.empty((K, N), dtype=torch.float32).pin_memory()
    Bh.copy_(B)
    Ch = torch.empty((mine.M, N), dtype=torch.float32).pin_memory()
    plan.spmm_host(Bh, Ch)
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        plan.spmm_host(Bh, Ch)  # returns after the stream has been synchronised
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    t_e = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
    if dist:
        dist.all_reduce(t_e, op=dist.ReduceOp.MAX)
    e2e_s = float(t_e.item())
    check = float(Ch.double().abs().sum())  # the device->host result is consumed

    flops = 2.0 * nnz * N
    gflops = flops / (ms_per_step * 1e-3) / 1e9
    # roofline of the dominant kernel on rank 0's shard (all ranks run the same kernel on equal cost)
    # (a shard reads only the rows of B its columns name: min(K, distinct columns) of them)
    distinct_cols = int(torch.unique(mine.cols).numel()) if world > 1 else K
    bytes_alg = 8 * mine.nnz + 4 * (mine.M + 1) + 4 * N * min(K, distinct_cols) + 4 * mine.M * N
    peak, peak_src = measured_hbm_peak()
    achieved = bytes_alg / (ms_per_step * 1e-3) / 1e9
    line = {
        "metric": "spmm_gflops", "value": round(gflops, 2), "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "M": M, "K": K, "nnz": nnz, "N": N, "path": args.path,
                   "matrix": mine.name, "rows_per_rank": [int(bounds[i + 1] - bounds[i]) for i in range(world)],
                   "l2": "not flushed" if args.no_flush else "flushed between steps (256 MiB write)",
                   "operands_bytes": bytes_alg, "parallelism": f"row panels over {world} GPU(s), B replicated, C row-sharded"},
        "ms_median": round(med_ms, 5), "ms_min": round(min_ms, 5), "ms_per_step_l2_not_flushed": None if warm_ms is None else round(warm_ms, 5), "wall_ms_per_step": round(wall * 1e3 / args.steps, 4),
        "plan_create_ms": round(plan_ms, 1), "plan_create_device_ms": None if plan_dev_ms is None else round(plan_dev_ms, 1), "plan": {k: info[k] for k in ("num_tiles", "num_long_rows", "num_chunks", "brick_panels", "num_bricks", "device_bytes")},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                     "traffic": dram_traffic_for(args.workload, args.path), "peak_source": peak_src,
                     "bytes_model": "8*nnz + 4*(M+1) + 4*N*min(K, distinct columns) + 4*M*N per launch and rank (A as CSR once, the rows of B it names once, C once)",
                     "frac_of_8TBs_nominal": round(achieved / 8000.0, 4),
                     # secondary model for matrices whose B cannot live in L2: every nonzero fetches its row of B (no reuse)
                     "gather_model_bytes": 8 * mine.nnz + 4 * (mine.M + 1) + 4 * N * mine.nnz + 4 * mine.M * N,
                     "gather_model_GBs": round((8 * mine.nnz + 4 * (mine.M + 1) + 4 * N * mine.nnz + 4 * mine.M * N) / (ms_per_step * 1e-3) / 1e9, 1)},
        "e2e": {"value": round(flops / e2e_s / 1e9, 2), "unit": "GFLOP/s", "h2d_bytes_per_step": K * N * 4,
                "d2h_bytes_per_step": mine.M * N * 4, "ms_per_step": round(e2e_s * 1e3, 3), "steps": e2e_steps,
                "checksum": check},
        "gpu_launches": args.steps * plan.launch_count(N),
        "clocks": clocks,
    }
    if bcast_ms is not None:
        line["bcast_ms"] = round(bcast_ms, 3)
        line["bcast_bytes"] = K * N * 4
        # B starting on rank 0 only: the whole job including the broadcast
        from_root["value"] = round(flops / (from_root["ms_per_step"] * 1e-3) / 1e9, 2)
        line["from_root"] = from_root
    if rank == 0 and world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(mine, N, b_seed, b_dist)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
