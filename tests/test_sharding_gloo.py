"""Host side of the multi-GPU path on CPU ranks (gloo, world size 2 and 3): nnz-balanced contiguous
row ranges, one plan per rank over its own rows, B delivered by a broadcast, C left row-sharded.
The device kernels are not involved: each rank checks its plan's packed format against its slice of A
and multiplies its slice with the CPU oracle, and the union of the shards must equal the
single-process product bit for bit."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import cutespmm_ae_b200 as cs
        import oracle
        from cutespmm_ae_b200 import generators as g

        A = g.rmat(11, 8, seed=77, values="uniform")  # every rank derives the same matrix from the seed
        N = 24
        bounds = cs.partition_rows(A.row_ptr, world, align_rows=16)
        r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
        mine = A.row_slice(r0, r1)
        plan = cs.Plan.from_csr(mine, host_only=True)
        rp, cols, vals = plan.decode_csr()
        assert np.array_equal(cols, mine.cols.numpy().astype(np.uint32))
        assert np.array_equal(vals, mine.vals.numpy())
        # B lives on rank 0 and reaches the others by one broadcast
        B = g.dense_operand(A.K, N, 78) if rank == 0 else torch.empty((A.K, N), dtype=torch.float32)
        dist.broadcast(B, 0)
        C_mine = torch.from_numpy(oracle.spmm_csr(mine.row_ptr, mine.cols, mine.vals, B.numpy(), mine.M, mine.K))
        # bookkeeping every rank agrees on
        counts = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(counts, torch.tensor([mine.M, mine.nnz], dtype=torch.int64))
        assert sum(int(c[0]) for c in counts) == A.M and sum(int(c[1]) for c in counts) == A.nnz
        nnzs = np.array([int(c[1]) for c in counts], dtype=np.float64)
        assert nnzs.max() <= 1.3 * nnzs.mean() + 2048  # balanced by nonzeros, up to one hub row
        torch.save({"r0": r0, "r1": r1, "C": C_mine}, Path(out_dir) / f"shard{rank}.pt")
        dist.barrier()
        if rank == 0:
            full = oracle.spmm_csr(A.row_ptr, A.cols, A.vals, B.numpy(), A.M, A.K)
            got = np.empty_like(full)
            covered = 0
            for r in range(world):
                sh = torch.load(Path(out_dir) / f"shard{r}.pt")
                got[sh["r0"] : sh["r1"]] = sh["C"].numpy()
                covered += sh["r1"] - sh["r0"]
            assert covered == A.M
            assert np.array_equal(full.view(np.uint32), got.view(np.uint32))  # row shards: bit-identical union
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _worker_windows(rank, world, port, out_dir):
    """ShardedSpmm.spmm_from_root on CPU ranks: B on the last rank only, broadcast in column windows,
    each window multiplied as it arrives (by the CPU oracle standing in for the device product)."""
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from cutespmm_ae_b200 import generators as g
        from cutespmm_ae_b200.sharded import ShardedSpmm, column_windows

        A = g.stencil9(24)
        N, root = 80, world - 1
        sh = ShardedSpmm(A, host_only=True)
        assert (sh.world, sh.rank) == (world, rank)
        assert sh.r0 % 16 == 0 and int(sh.bounds[0]) == 0 and int(sh.bounds[-1]) == A.M
        assert column_windows(N, 4, 32) == [(0, 64), (64, 80)]
        calls = []

        def product(Bw, Cw):
            calls.append(tuple(Bw.shape))
            Cw.copy_(torch.from_numpy(oracle.spmm_csr(sh.rows.row_ptr, sh.rows.cols, sh.rows.vals, Bw.numpy(), sh.rows.M, sh.rows.K)))

        B = g.dense_operand(A.K, N, 91) if rank == root else None
        C_mine, blocks = sh.spmm_from_root(B, N, root=root, max_windows=4, min_cols=32, product=product, device=torch.device("cpu"))
        assert calls == [(A.K, 64), (A.K, 16)]
        assert [tuple(b.shape) for b in blocks] == calls and all(b.is_contiguous() for b in blocks)
        C_mine = C_mine.clone()
        C_one, one = sh.spmm_from_root(B, N, root=root, product=product, device=torch.device("cpu"))  # default: one window
        assert len(one) == 1 and tuple(one[0].shape) == (A.K, N) and torch.equal(C_one, C_mine)
        torch.save({"r0": sh.r0, "r1": sh.r1, "C": C_mine, "B": torch.cat(blocks, dim=1)}, Path(out_dir) / f"win{rank}.pt")
        dist.barrier()
        if rank == 0:
            parts = [torch.load(Path(out_dir) / f"win{r}.pt") for r in range(world)]
            Bfull = parts[root]["B"].numpy()
            assert all(np.array_equal(p["B"].numpy(), Bfull) for p in parts)  # every rank received all of B
            full = oracle.spmm_csr(A.row_ptr, A.cols, A.vals, Bfull, A.M, A.K)
            got = np.concatenate([p["C"].numpy() for p in parts], axis=0)
            assert [p["r0"] for p in parts[1:]] == [p["r1"] for p in parts[:-1]]
            assert np.array_equal(full.view(np.uint32), got.view(np.uint32))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_row_sharding_over_gloo_ranks(tmp_path, world):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)


@pytest.mark.parametrize("world", [2, 3])
def test_windowed_broadcast_pipeline_over_gloo_ranks(tmp_path, world):
    mp.spawn(_worker_windows, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)


def test_column_windows():
    from cutespmm_ae_b200.sharded import column_windows

    assert column_windows(128, 4, 32) == [(0, 32), (32, 64), (64, 96), (96, 128)]
    assert column_windows(128, 2, 64) == [(0, 64), (64, 128)]
    assert column_windows(24, 4, 32) == [(0, 24)]
    assert column_windows(100, 4, 32) == [(0, 64), (64, 100)]
    assert column_windows(0) == []
    for N in range(1, 300, 7):
        w = column_windows(N, 4, 32)
        assert w[0][0] == 0 and w[-1][1] == N and all(a[1] == b[0] for a, b in zip(w, w[1:])) and len(w) <= 4


@pytest.mark.parametrize("world", [2, 3, 8])
def test_sharded_entry_point_bookkeeping_with_a_stub_communicator(world):
    """cutespmm_spmm_sharded / cutespmm_sharded_transfers through the C ABI with a communicator that records its
    collectives instead of sending them: which rank sends which element range of B, for every exchange mode, and
    the argument errors -- everything of the multi-GPU entry point that needs no GPU."""
    import ctypes as C

    import cutespmm_ae_b200 as cs
    from cutespmm_ae_b200 import generators as g

    A = g.rmat(10, 8, seed=79, values="uniform")
    K, N = A.K, 24
    bounds = cs.partition_rows(A.row_ptr, world, align_rows=16)
    dummy = C.create_string_buffer(64)  # stands for device buffers: a stub communicator and a host-only plan touch neither
    ptr = C.addressof(dummy)
    even = np.minimum(np.arange(world + 1, dtype=np.uint64) * np.uint64(-(-K // world)), np.uint64(K))
    ragged = even.copy()
    ragged[1] = ragged[0]  # rank 0 holds no rows of B
    for rank in range(world):
        comm = cs.Comm.stub(world, rank)
        mine = A.row_slice(int(bounds[rank]), int(bounds[rank + 1]))
        plan = cs.Plan.from_csr(mine, host_only=True)

        def call(mode, root=0, bb=None, ldb=N):
            b = None if bb is None else np.ascontiguousarray(bb, dtype=np.uint64)
            return cs.lib.cutespmm_spmm_sharded(plan._h, comm._h, mode, root, ptr, ldb, None if b is None else b.ctypes.data, ptr, N, N, None)

        assert call(cs.B_RESIDENT) == 0 and comm.stub_log() == []
        assert call(cs.B_FROM_ROOT, root=world - 1) == 0
        assert comm.stub_log() == [(world - 1, 0, K * N)] == comm.transfers(cs.B_FROM_ROOT, K, N, root=world - 1)
        assert call(cs.B_ROW_SHARDED, bb=even) == 0
        want = [(r, int(even[r]) * N, int(even[r + 1] - even[r]) * N) for r in range(world) if even[r + 1] > even[r]]
        assert comm.stub_log() == want == comm.transfers(cs.B_ROW_SHARDED, K, N, even)
        assert sum(c for _, _, c in want) == K * N  # the slices tile B exactly
        assert call(cs.B_ROW_SHARDED, bb=ragged) == 0
        log = comm.stub_log()
        assert [r for r, _, _ in log] == list(range(1, world)) and sum(c for _, _, c in log) == K * N
        # errors: strided B cannot be exchanged, bounds must tile [0, K], the root must be a rank, bounds are required
        assert call(cs.B_FROM_ROOT, ldb=N + 4) == -4
        bad = even.copy()
        bad[-1] -= 1
        assert call(cs.B_ROW_SHARDED, bb=bad) == -1
        assert call(cs.B_FROM_ROOT, root=world) == -1
        assert call(cs.B_ROW_SHARDED) == -1
        assert comm.stub_log() == []
        comm.close()
