"""Row-sharded SpMM over the ranks of a torch.distributed process group (one process per GPU).

Row panels are independent, so A is cut into contiguous row ranges of equal cost (nonzeros plus a
per-row term, 16-row aligned: `cutespmm_partition_rows`), every rank builds a plan over its own rows
only, and C stays row-sharded: rank p owns rows [bounds[p], bounds[p+1]).  The one exchange of the
path is B, which every rank needs in its own memory.  Two ways to run a product:

* `spmm(B)`              B is already replicated (iterative solvers, the layers of a GNN after the
                         first): purely local, no collective.
* `spmm_from_root(B)`    B lives on one rank and reaches the others by broadcast.
* `spmm_row_sharded(B)`  every rank holds a row range of B in place inside its K x N buffer (the C
                         of a previous sharded product): one all-gather, then the product.
* `spmm_host(B_rows)`    host buffers: every rank uploads only its own slice of B over its own PCIe
                         link, the slices are exchanged over NVLink, C rows go back to the host.

On GPU ranks these are calls of the library's C entry points (cutespmm_spmm_sharded,
cutespmm_spmm_sharded_host) over the library's own communicator (cutespmm_comm_*, NCCL underneath);
this class only adds the partition and the plan.  On CPU ranks (tests of the host logic under gloo)
`spmm_from_root` runs the same schedule over torch.distributed with a caller-supplied product.

The reference has no multi-GPU path; its single-GPU driver loop (run.cu:38-53) is what a rank runs
on its shard.  No kernel reads another GPU's memory: B comes into local memory first (NCCL).
"""
from __future__ import annotations

from typing import Callable, Optional

import numpy as np

from . import B_FROM_ROOT, B_ROW_SHARDED, PATH_AUTO, Comm, Plan, partition_rows


def column_windows(N: int, max_windows: int = 4, min_cols: int = 32) -> list[tuple[int, int]]:
    """Cuts N columns into at most `max_windows` windows [c0, c1) whose width is a multiple of
    `min_cols` (the last may be narrower)."""
    if N <= 0:
        return []
    nw = max(1, min(max_windows, N // min_cols))
    width = -(-N // nw)
    width = -(-width // min_cols) * min_cols
    return [(c0, min(c0 + width, N)) for c0 in range(0, N, width)]


class ShardedSpmm:
    """This rank's shard of A and the operations on it.

    A: anything with M, K, row_ptr, cols, vals and row_slice(r0, r1) (generators.CsrMatrix); every
    rank passes the same matrix (or its own way of producing the same rows).  `group` is a
    torch.distributed process group (None: the default group; a single process works without one).
    `host_only=True` builds the plan without touching CUDA (tests of the host logic on CPU ranks).
    `row_cost`: what a row costs in units of one nonzero when the rows are cut into ranges of equal cost.  At
    N = 128 a row is one 512-byte store of C plus the claim of the row, a nonzero one 512-byte gather; measured on
    the eight shards of R-MAT 2^24, 2 balances them within 9 % (1.83 .. 2.00 ms), 4 leaves the hub-heavy shard at
    2.18 ms and 1 the many-rows shard at 2.12 ms.
    """

    def __init__(self, A, group=None, *, path: int = PATH_AUTO, host_only: bool = False, align_rows: int = 16, row_cost: int = 2,
                 **plan_kw):
        import torch.distributed as dist

        self.group = group
        self.dist = dist if dist.is_available() and dist.is_initialized() else None
        self.world = self.dist.get_world_size(group) if self.dist else 1
        self.rank = self.dist.get_rank(group) if self.dist else 0
        self.M, self.K = A.M, A.K
        rp = A.row_ptr.cpu() if hasattr(A.row_ptr, "cpu") else A.row_ptr
        self.bounds = partition_rows(rp, self.world, align_rows=align_rows, row_cost=row_cost) if self.world > 1 else np.array([0, A.M], dtype=np.uint64)
        self.r0, self.r1 = int(self.bounds[self.rank]), int(self.bounds[self.rank + 1])
        mine = A.row_slice(self.r0, self.r1) if self.world > 1 else A
        if hasattr(mine, "cpu"):
            mine = mine.cpu()
        self.rows = mine
        self.plan = Plan.from_csr(mine, path=path, host_only=host_only, **plan_kw)
        self._recv = {}  # receive buffers of spmm_from_root, by (window, width, device)
        self._comm = None

    @property
    def comm(self) -> Comm:
        """The library communicator of this rank (created on first use; collective: every rank must ask for it)."""
        if self._comm is None:
            if self.world == 1:
                raise RuntimeError("a single rank needs no communicator")
            self._comm = Comm.from_torch(self.group)
        return self._comm

    def even_row_bounds(self) -> np.ndarray:
        """Row bounds of B cut into `world` slices of equal size (the last takes the remainder): equal slices travel
        as one in-place all-gather."""
        step = -(-self.K // self.world)
        return np.minimum(np.arange(self.world + 1, dtype=np.uint64) * np.uint64(step), np.uint64(self.K))

    # ---- B already in every rank's memory --------------------------------------------------------
    def spmm(self, B, Cout=None, stream=None):
        """Rows [r0, r1) of A @ B; B is a K x N CUDA tensor resident on this rank."""
        return self.plan.spmm(B, Cout, stream)

    # ---- B row-sharded over the ranks --------------------------------------------------------------
    def spmm_row_sharded(self, B, b_bounds, Cout=None, stream=None):
        """Rows [r0, r1) of A @ B where this rank's K x N buffer B holds rows [b_bounds[rank], b_bounds[rank+1]) and
        the rest arrives by one all-gather in place (cutespmm_spmm_sharded, CUTESPMM_B_ROW_SHARDED)."""
        if self.world == 1:
            return self.plan.spmm(B, Cout, stream)
        return self.plan.spmm_sharded(self.comm, B, Cout, b_mode=B_ROW_SHARDED, b_bounds=b_bounds, stream=stream)

    # ---- host buffers ------------------------------------------------------------------------------
    def spmm_host(self, B_rows, b_bounds=None, Cout=None, stream=None):
        """Host in, host out: B_rows is this rank's slice of B (rows [b_bounds[rank], b_bounds[rank+1]), default
        even_row_bounds()); returns (C rows of this rank on the host, kernel_ms, exchange_ms)."""
        if b_bounds is None:
            b_bounds = self.even_row_bounds()
        return self.plan.spmm_sharded_host(self.comm if self.world > 1 else None, B_rows, b_bounds, Cout, stream)

    # ---- B on one rank ---------------------------------------------------------------------------
    def spmm_from_root(self, B, N: int, root: int = 0, Cout=None, *, max_windows: int = 1, min_cols: int = 64,
                       product: Optional[Callable] = None, device=None):
        """Rows [r0, r1) of A @ B where B (K x N) is given on rank `root` only (None elsewhere).

        B is sent window-major (each column window a contiguous K x w block), all broadcasts are
        queued at once, and the product of window w is queued behind the arrival of window w only.
        Returns (C, windows): C is this rank's (r1-r0) x N block, `windows` the received K x w
        blocks (kept so that a caller can reuse B without a second transfer; they are buffers of
        this object, overwritten by the next call).  One window (the default) is a plain broadcast
        followed by the product; more windows pay when the transfer is long against the product
        (measured on two GPUs over NVLink it is not: 268 MB arrive in 0.47 ms, and two half-width
        products cost more than one full-width product).

        `product(Bw, Cw)` computes Cw = A_rows @ Bw; default: this rank's plan on the GPU.  Tests on
        CPU ranks pass a CPU product of their own.
        """
        import torch

        if product is None and self.world > 1 and max_windows == 1:
            # GPU ranks, one window: the library's own broadcast + product (cutespmm_spmm_sharded)
            if self.rank == root:
                if B is None or tuple(B.shape) != (self.K, N):
                    raise ValueError("the root rank must pass B with shape (K, N)")
                buf = B if B.is_contiguous() else B.contiguous()
            else:
                if device is None:
                    raise ValueError("ranks other than the root must say on which device B is to be received")
                key = (0, N, str(device))
                buf = self._recv.get(key)
                if buf is None:
                    buf = self._recv[key] = torch.empty((self.K, N), dtype=torch.float32, device=device)
            Cout = self.plan.spmm_sharded(self.comm, buf, Cout, b_mode=B_FROM_ROOT, root=root)
            return Cout, [buf]
        if product is None:
            product = lambda Bw, Cw: self.plan.spmm(Bw, Cw)  # noqa: E731
        wins = column_windows(N, max_windows, min_cols)
        if self.rank == root:
            if B is None or tuple(B.shape) != (self.K, N):
                raise ValueError("the root rank must pass B with shape (K, N)")
            device = B.device
        elif device is None:
            raise ValueError("ranks other than the root must say on which device B is to be received")
        if Cout is None:
            Cout = torch.empty((self.r1 - self.r0, N), dtype=torch.float32, device=device)
        blocks, works = [], []
        for i, (c0, c1) in enumerate(wins):
            if self.rank == root and len(wins) == 1 and B.is_contiguous():
                blk = B  # one window: B goes as it is
            else:
                key = (i, c1 - c0, str(device))
                blk = self._recv.get(key)
                if blk is None:
                    blk = self._recv[key] = torch.empty((self.K, c1 - c0), dtype=torch.float32, device=device)
                if self.rank == root:
                    blk.copy_(B[:, c0:c1])
            blocks.append(blk)
            if self.world > 1:
                works.append(self.dist.broadcast(blk, src=self._global_rank(root), group=self.group, async_op=True))
        for i, (c0, c1) in enumerate(wins):
            if works:
                works[i].wait()  # CUDA: the current stream waits for window i only; the host does not block
            product(blocks[i], Cout[:, c0:c1])
        return Cout, blocks

    def _global_rank(self, group_rank: int) -> int:
        if self.dist is None or self.group is None:
            return group_rank
        return self.dist.get_global_rank(self.group, group_rank)
