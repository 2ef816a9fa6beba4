"""Seeded synthetic sparse matrices and dense operands for the SpMM workloads.

The reference project measures on SuiteSparse matrices read from MatrixMarket
files (run.cu:10-18, meta.data).  Those files are not available to a test or
benchmark run, so five synthetic matrix families with the same structural
classes (uniform random, 2-D stencil, block-structured 3-D elasticity, power-law
graph at two sizes) stand in for them.  Everything here is a pure function of
(shape parameters, seed): a counter-based hash (SplitMix64 finaliser) indexed by
element number replaces a stateful RNG, so the same matrix comes out on a CPU
tensor and on a CUDA tensor, in one piece or generated shard by shard.

All matrices are returned as CSR with int64 row pointers, int32 column indices
(ascending and unique inside every row) and fp32 values, the layout the plan
builder (`cutespmm_plan_create`) takes.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

_M1 = -4658895280553007687  # 0xbf58476d1ce4e5b9 as signed 64-bit
_M2 = -7723592293110705685  # 0x94d049bb133111eb as signed 64-bit
_GOLD = -7046029254386353131  # 0x9e3779b97f4a7c15 as signed 64-bit


def _lsr(x: torch.Tensor, s: int) -> torch.Tensor:
    """Logical right shift of an int64 tensor."""
    return (x >> s) & ((1 << (64 - s)) - 1)


def hash64(idx: torch.Tensor, seed: int, stream: int = 0) -> torch.Tensor:
    """SplitMix64 finaliser of (idx, seed, stream) -> 64 uniformly mixed bits (int64)."""
    key = (seed * 0x100000001B3 + stream * 0x9E3779B1 + 0x632BE59BD9B4E019) & 0x7FFFFFFFFFFFFFFF
    x = idx * _GOLD + key
    x = (x ^ _lsr(x, 30)) * _M1
    x = (x ^ _lsr(x, 27)) * _M2
    return x ^ _lsr(x, 31)


def uniform01(idx: torch.Tensor, seed: int, stream: int = 0) -> torch.Tensor:
    """Uniform doubles in [0, 1) with 53 random bits."""
    return _lsr(hash64(idx, seed, stream), 11).to(torch.float64) * (1.0 / 9007199254740992.0)


def normal01(idx: torch.Tensor, seed: int, stream: int = 0) -> torch.Tensor:
    """Standard normal doubles (Box-Muller on two hashed uniforms)."""
    u1 = 1.0 - uniform01(idx, seed, 2 * stream + 101)  # (0, 1]
    u2 = uniform01(idx, seed, 2 * stream + 102)
    return torch.sqrt(-2.0 * torch.log(u1)) * torch.cos((2.0 * math.pi) * u2)


@dataclass
class CsrMatrix:
    """CSR on one device.  `row_ptr` int64 [M+1], `cols` int32 [nnz], `vals` fp32 [nnz]."""

    M: int
    K: int
    row_ptr: torch.Tensor
    cols: torch.Tensor
    vals: torch.Tensor
    name: str = ""

    @property
    def nnz(self) -> int:
        return int(self.cols.numel())

    def cpu(self) -> "CsrMatrix":
        return CsrMatrix(self.M, self.K, self.row_ptr.cpu(), self.cols.cpu(), self.vals.cpu(), self.name)

    def row_slice(self, r0: int, r1: int) -> "CsrMatrix":
        """Rows [r0, r1) as their own CSR (column space unchanged)."""
        j0, j1 = int(self.row_ptr[r0]), int(self.row_ptr[r1])
        return CsrMatrix(r1 - r0, self.K, self.row_ptr[r0 : r1 + 1] - j0, self.cols[j0:j1], self.vals[j0:j1], self.name)


def _csr_from_sorted_keys(keys: torch.Tensor, M: int, K: int):
    """keys = row*K + col, ascending and unique -> (row_ptr, cols)."""
    rows = torch.div(keys, K, rounding_mode="floor")
    cols = (keys - rows * K).to(torch.int32)
    counts = torch.bincount(rows, minlength=M)
    row_ptr = torch.zeros(M + 1, dtype=torch.int64, device=keys.device)
    torch.cumsum(counts, 0, out=row_ptr[1:])
    return row_ptr, cols


def uniform_random(M: int = 4096, K: int = 4096, nnz_per_row: int = 16, seed: int = 1001, device="cpu") -> CsrMatrix:
    """Every row holds `nnz_per_row` distinct uniformly random columns; values U[-1, 1)."""
    dev = torch.device(device)
    r = torch.arange(M, dtype=torch.int64, device=dev).repeat_interleave(nnz_per_row)
    slot = torch.arange(M * nnz_per_row, dtype=torch.int64, device=dev)
    c = (uniform01(slot, seed, 0) * K).to(torch.int64).clamp_(max=K - 1)
    keys = r * K + c
    attempt = 1
    while True:
        keys, order = torch.sort(keys)
        slot = slot[order]
        dup = torch.zeros_like(keys, dtype=torch.bool)
        dup[1:] = keys[1:] == keys[:-1]
        if not bool(dup.any()):
            break
        rr = torch.div(keys[dup], K, rounding_mode="floor")
        cc = (uniform01(slot[dup], seed, 7 * attempt) * K).to(torch.int64).clamp_(max=K - 1)
        keys[dup] = rr * K + cc
        attempt += 1
    row_ptr, cols = _csr_from_sorted_keys(keys, M, K)
    nnz = keys.numel()
    vals = (2.0 * uniform01(torch.arange(nnz, dtype=torch.int64, device=dev), seed, 1) - 1.0).to(torch.float32)
    return CsrMatrix(M, K, row_ptr, cols, vals, f"uniform_{M}x{K}_{nnz_per_row}pr")


def stencil9(nx: int = 512, ny: int = 512, seed: int = 1002, device="cpu") -> CsrMatrix:
    """9-point stencil on an nx x ny grid (row index = y*nx + x): off-diagonals U[0.5, 1.5), diagonal 8."""
    dev = torch.device(device)
    n = nx * ny
    i = torch.arange(n, dtype=torch.int64, device=dev)
    x, y = i % nx, torch.div(i, nx, rounding_mode="floor")
    keys = []
    for dy in (-1, 0, 1):
        for dx in (-1, 0, 1):
            ok = (x + dx >= 0) & (x + dx < nx) & (y + dy >= 0) & (y + dy < ny)
            keys.append((i * n + (i + dy * nx + dx))[ok])
    keys = torch.sort(torch.cat(keys)).values
    row_ptr, cols = _csr_from_sorted_keys(keys, n, n)
    nnz = keys.numel()
    vals = (0.5 + uniform01(torch.arange(nnz, dtype=torch.int64, device=dev), seed, 1)).to(torch.float32)
    rows = torch.div(keys, n, rounding_mode="floor")
    vals[cols.to(torch.int64) == rows] = 8.0
    return CsrMatrix(n, n, row_ptr, cols, vals, f"stencil9_{nx}x{ny}")


def elasticity3d(n: int = 40, block: int = 3, seed: int = 1003, device="cpu") -> CsrMatrix:
    """7-point adjacency of an n^3 grid, every node pair expanded into a dense block x block tile; values N(0, 1)."""
    dev = torch.device(device)
    nodes = n * n * n
    i = torch.arange(nodes, dtype=torch.int64, device=dev)
    x, y, z = i % n, torch.div(i, n, rounding_mode="floor") % n, torch.div(i, n * n, rounding_mode="floor")
    pairs_r, pairs_c = [], []
    for dx, dy, dz in ((0, 0, 0), (1, 0, 0), (-1, 0, 0), (0, 1, 0), (0, -1, 0), (0, 0, 1), (0, 0, -1)):
        ok = (x + dx >= 0) & (x + dx < n) & (y + dy >= 0) & (y + dy < n) & (z + dz >= 0) & (z + dz < n)
        pairs_r.append(i[ok])
        pairs_c.append((i + dx + dy * n + dz * n * n)[ok])
    pr, pc = torch.cat(pairs_r), torch.cat(pairs_c)
    M = nodes * block
    br = torch.arange(block, dtype=torch.int64, device=dev)
    rows = (pr[:, None, None] * block + br[None, :, None]).expand(-1, block, block)
    cols = (pc[:, None, None] * block + br[None, None, :]).expand(-1, block, block)
    keys = torch.sort((rows * M + cols).reshape(-1)).values
    row_ptr, cols = _csr_from_sorted_keys(keys, M, M)
    nnz = keys.numel()
    vals = normal01(torch.arange(nnz, dtype=torch.int64, device=dev), seed, 1).to(torch.float32)
    return CsrMatrix(M, M, row_ptr, cols, vals, f"elasticity_{n}^3_b{block}")


def rmat(scale: int = 20, edge_factor: int = 8, a=0.57, b=0.19, c=0.19, seed: int = 1004,
         values: str = "rownorm", device="cpu", chunk: int = 1 << 24) -> CsrMatrix:
    """R-MAT graph with 2^scale nodes: edge_factor * 2^scale directed draws, symmetrised and
    deduplicated (average degree about 2 * edge_factor).  `values`: "rownorm" (1 / row degree)
    or "uniform" (U[-1, 1))."""
    dev = torch.device(device)
    n = 1 << scale
    draws = edge_factor * n
    parts = []
    for e0 in range(0, draws, chunk):
        e = torch.arange(e0, min(draws, e0 + chunk), dtype=torch.int64, device=dev)
        r = torch.zeros_like(e)
        col = torch.zeros_like(e)
        for level in range(scale):
            u = uniform01(e, seed, 16 + level)
            rbit = (u >= a + b).to(torch.int64)
            cbit = (((u >= a) & (u < a + b)) | (u >= a + b + c)).to(torch.int64)
            r = (r << 1) | rbit
            col = (col << 1) | cbit
        parts.append(r * n + col)
        parts.append(col * n + r)
        del e, r, col
    keys = torch.cat(parts)
    del parts
    keys = torch.unique(keys)  # sorted + deduplicated
    row_ptr, cols = _csr_from_sorted_keys(keys, n, n)
    nnz = keys.numel()
    if values == "rownorm":
        deg = (row_ptr[1:] - row_ptr[:-1]).clamp(min=1)
        rows = torch.div(keys, n, rounding_mode="floor")
        vals = (1.0 / deg.to(torch.float64))[rows].to(torch.float32)
    else:
        vals = (2.0 * uniform01(keys, seed, 1) - 1.0).to(torch.float32)
    del keys
    return CsrMatrix(n, n, row_ptr, cols, vals, f"rmat_s{scale}_ef{edge_factor}")


def dense_operand(K: int, N: int, seed: int, dist: str = "normal", device="cpu", row0: int = 0,
                  rows: int | None = None, chunk_rows: int = 1 << 20) -> torch.Tensor:
    """Row-major fp32 B[K x N] (or rows [row0, row0+rows) of it): element (k, n) depends on (seed, k*N+n) only."""
    dev = torch.device(device)
    rows = K - row0 if rows is None else rows
    out = torch.empty((rows, N), dtype=torch.float32, device=dev)
    for r in range(0, rows, chunk_rows):
        rr = min(rows, r + chunk_rows)
        idx = torch.arange((row0 + r) * N, (row0 + rr) * N, dtype=torch.int64, device=dev)
        if dist == "normal":
            v = normal01(idx, seed, 3)
        elif dist == "uniform_pm1":
            v = 2.0 * uniform01(idx, seed, 3) - 1.0
        else:
            raise ValueError(dist)
        out[r:rr] = v.to(torch.float32).view(rr - r, N)
    return out


# The five workloads, keyed by the short names used by the tests and the benchmark.
WORKLOADS = {
    "uniform4096": dict(make=lambda device="cpu": uniform_random(4096, 4096, 16, 1001, device), N=32, b_seed=2001, b_dist="uniform_pm1"),
    "stencil512": dict(make=lambda device="cpu": stencil9(512, 512, 1002, device), N=128, b_seed=2002, b_dist="normal"),
    "elasticity40": dict(make=lambda device="cpu": elasticity3d(40, 3, 1003, device), N=128, b_seed=2003, b_dist="normal"),
    "rmat20": dict(make=lambda device="cpu": rmat(20, 8, seed=1004, values="rownorm", device=device), N=128, b_seed=2004, b_dist="normal"),
    "rmat24": dict(make=lambda device="cpu": rmat(24, 8, seed=1005, values="uniform", device=device), N=128, b_seed=2005, b_dist="normal"),
}


def algorithmic_bytes(M: int, K: int, N: int, nnz: int) -> int:
    """Bytes one SpMM must move if A (as CSR: 8 B per nonzero + row pointers), B and C each cross HBM once."""
    return 8 * nnz + 4 * (M + 1) + 4 * K * N + 4 * M * N
