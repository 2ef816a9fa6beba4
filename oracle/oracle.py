"""ctypes access to the CPU oracle (oracle/spmm_oracle.c) and, when it has been built, to the
reference project's own host routines (oracle/_ref/libcutespmm_ref.so, see oracle/Makefile).

TEST INFRASTRUCTURE ONLY: the checker, never the thing measured or shipped.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "liboracle.so"
REF_PATH = HERE / "_ref" / "libcutespmm_ref.so"
REF_LOADERS_PATH = HERE / "_ref" / "libcutespmm_ref_loaders.so"
REF_GPU_PATH = HERE / "_ref" / "libcutespmm_ref_gpu.so"

__all__ = ["build", "reference_root", "set_threads", "spmm_coo", "spmm_csr", "spmm_csr_rows", "sddmm_csr", "max_rel_err", "rel_fro", "ref_available", "ref_gpu_available", "ref_gpu_spmm", "Ref", "LIB_PATH", "REF_PATH"]


def reference_root() -> Path | None:
    """Where a checkout of the reference project lies: $CUTESPMM_REF, else a directory named
    "reference" beside this repository.  None when there is none (a machine that only runs the tests)."""
    import os

    for cand in (os.environ.get("CUTESPMM_REF"), HERE.parent.parent / "reference"):
        if cand and (Path(cand) / "data.cu").exists():
            return Path(cand)
    return None


def _nvcc() -> str:
    import os
    import shutil

    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    return "nvcc"


def build(ref_root="auto") -> None:
    """Compiles liboracle.so (gcc) and, if a reference checkout is found (reference_root(), or the
    path given), oracle/_ref.  ref_root=None builds the oracle alone."""
    subprocess.run(["make", "-s", "-C", str(HERE)], check=True)
    root = reference_root() if ref_root == "auto" else (Path(ref_root) if ref_root else None)
    if root and (root / "data.cu").exists():
        subprocess.run(["make", "-s", "-C", str(HERE), "ref", f"REF={root}", f"NVCC={_nvcc()}"], check=True)


_lib = None


def _load():
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build(ref_root=None)
        _lib = C.CDLL(str(LIB_PATH))
        vp = C.c_void_p
        _lib.oracle_spmm_coo.argtypes = [vp, vp, vp, vp, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64]
        _lib.oracle_spmm_coo.restype = None
        _lib.oracle_spmm_csr.argtypes = [vp, vp, vp, vp, vp, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint64, C.c_uint64]
        _lib.oracle_spmm_csr.restype = None
        _lib.oracle_spmm_csr_rows.argtypes = [vp, vp, vp, vp, vp, vp, C.c_uint64, C.c_uint32, C.c_uint64]
        _lib.oracle_spmm_csr_rows.restype = None
        _lib.oracle_max_rel_err.argtypes = [vp, vp, C.c_uint32, C.c_uint32]
        _lib.oracle_max_rel_err.restype = C.c_float
        _lib.oracle_rel_fro.argtypes = [vp, vp, C.c_uint64]
        _lib.oracle_rel_fro.restype = C.c_double
        _lib.oracle_sddmm_csr.argtypes = [vp, vp, vp, vp, vp, vp, C.c_uint64, C.c_uint32, C.c_uint64, C.c_uint64]
        _lib.oracle_sddmm_csr.restype = None
        _lib.oracle_set_threads.argtypes = [C.c_int]
        _lib.oracle_set_threads.restype = None
        _lib.oracle_max_threads.argtypes = []
        _lib.oracle_max_threads.restype = C.c_int
    return _lib


def set_threads(n: int) -> int:
    """Sets the OpenMP thread count of the oracle's loops; returns the count in force."""
    lib = _load()
    lib.oracle_set_threads(int(n))
    return int(lib.oracle_max_threads())


def _a(x, dt):
    if hasattr(x, "detach"):
        x = x.detach().cpu().numpy()
    return np.ascontiguousarray(x, dtype=dt)


def spmm_coo(rows, cols, vals, B, M: int, K: int) -> np.ndarray:
    """inc.h:71-83 restated: in-order accumulation over a COO list."""
    rows, cols, vals, B = _a(rows, np.uint32), _a(cols, np.uint32), _a(vals, np.float32), _a(B, np.float32)
    N = B.shape[1]
    out = np.empty((M, N), dtype=np.float32)
    _load().oracle_spmm_coo(rows.ctypes.data, cols.ctypes.data, vals.ctypes.data, B.ctypes.data, out.ctypes.data, M, K, N, rows.size)
    return out


def spmm_csr(row_ptr, cols, vals, B, M: int, K: int) -> np.ndarray:
    """Row-parallel form of the same arithmetic (bit-identical on row-sorted input)."""
    rp, cols, vals, B = _a(row_ptr, np.uint64), _a(cols, np.uint32), _a(vals, np.float32), _a(B, np.float32)
    N = B.shape[1]
    out = np.empty((M, N), dtype=np.float32)
    _load().oracle_spmm_csr(rp.ctypes.data, cols.ctypes.data, vals.ctypes.data, B.ctypes.data, out.ctypes.data, M, K, N, N, N)
    return out


def spmm_csr_rows(row_ptr, cols, vals, B, which) -> np.ndarray:
    """Rows `which` of the product only."""
    rp, cols, vals, B = _a(row_ptr, np.uint64), _a(cols, np.uint32), _a(vals, np.float32), _a(B, np.float32)
    which = _a(which, np.uint64)
    N = B.shape[1]
    out = np.empty((which.size, N), dtype=np.float32)
    _load().oracle_spmm_csr_rows(rp.ctypes.data, cols.ctypes.data, vals.ctypes.data, B.ctypes.data, out.ctypes.data,
                                 which.ctypes.data, which.size, N, N)
    return out


def sddmm_csr(row_ptr, cols, vals, X, Y) -> np.ndarray:
    """out[j] = (vals[j] if vals is not None else 1) * <X[row of j], Y[cols[j]]> for every stored position j."""
    rp, cols, X, Y = _a(row_ptr, np.uint64), _a(cols, np.uint32), _a(X, np.float32), _a(Y, np.float32)
    v = None if vals is None else _a(vals, np.float32)
    out = np.empty(cols.size, dtype=np.float32)
    _load().oracle_sddmm_csr(rp.ctypes.data, cols.ctypes.data, None if v is None else v.ctypes.data, X.ctypes.data, Y.ctypes.data,
                             out.ctypes.data, rp.size - 1, X.shape[1], X.shape[1], Y.shape[1])
    return out


def max_rel_err(C_ref, C_test) -> float:
    """inc.h:84-110 restated."""
    a, b = _a(C_ref, np.float32), _a(C_test, np.float32)
    return float(_load().oracle_max_rel_err(a.ctypes.data, b.ctypes.data, a.shape[0], a.shape[1]))


def rel_fro(C_ref, C_test) -> float:
    a, b = _a(C_ref, np.float32), _a(C_test, np.float32)
    assert a.shape == b.shape
    return float(_load().oracle_rel_fro(a.ctypes.data, b.ctypes.data, a.size))


def ref_available() -> bool:
    return REF_PATH.exists()


def ref_gpu_available() -> bool:
    return REF_GPU_PATH.exists()


def ref_gpu_spmm(M: int, K: int, row_ptr, cols, vals, B, iters: int = 10):
    """The reference project's own GPU path (HRPB preprocessing, SPMM_TC work list, its kernel; oracle/ref_gpu_shim.cu)
    on the current CUDA device.  Rows need ascending unique columns, M and K multiples of 16, N one of the widths its
    launcher knows.  Returns (C, preprocessing ms, first-launch ms, mean ms of `iters` back-to-back launches, mean ms of
    `iters` launches each after an L2 flush)."""
    L = C.CDLL(str(REF_GPU_PATH))
    vp = C.c_void_p
    L.ref_gpu_spmm.argtypes = [C.c_uint, C.c_uint, C.c_uint, vp, vp, vp, vp, vp, C.c_int, vp, vp, vp, vp]
    L.ref_gpu_spmm.restype = C.c_int
    rp, cols, vals, B = _a(row_ptr, np.uint32), _a(cols, np.uint32), _a(vals, np.float32), _a(B, np.float32)
    N = B.shape[1]
    out = np.empty((M, N), dtype=np.float32)
    prep, cold, warm, flushed = C.c_float(), C.c_float(), C.c_float(), C.c_float()
    st = L.ref_gpu_spmm(M, K, N, rp.ctypes.data, cols.ctypes.data, vals.ctypes.data, B.ctypes.data, out.ctypes.data, iters,
                        C.byref(prep), C.byref(cold), C.byref(warm), C.byref(flushed))
    if st != 0:
        raise RuntimeError(f"the reference's GPU path failed with CUDA error {st}")
    return out, prep.value, cold.value, warm.value, flushed.value


class Ref:
    """The reference project's own host routines (compiled from its sources into oracle/_ref)."""

    def __init__(self):
        self.lib = C.CDLL(str(REF_PATH))
        vp = C.c_void_p
        L = self.lib
        L.ref_spmm_coo.argtypes = [vp, vp, vp, vp, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint]
        L.ref_spmm_coo.restype = None
        L.ref_check_gemm_correctness_coo.argtypes = [vp, vp, C.c_uint32, C.c_uint32]
        L.ref_check_gemm_correctness_coo.restype = C.c_float
        if hasattr(L, "ref_set_threads"):
            L.ref_set_threads.argtypes = [C.c_int]
            L.ref_set_threads.restype = None
            L.ref_max_threads.argtypes = []
            L.ref_max_threads.restype = C.c_int
        L.ref_mtx_open.argtypes = [C.c_char_p]
        L.ref_mtx_open.restype = vp
        for f in ("ref_mtx_M", "ref_mtx_K", "ref_mtx_nnz", "ref_hrpb_num_panels", "ref_hrpb_num_blocks"):
            getattr(L, f).argtypes = [vp]
            getattr(L, f).restype = C.c_uint
        L.ref_mtx_copy.argtypes = [vp, vp, vp, vp]
        L.ref_mtx_copy.restype = None
        L.ref_hrpb_build.argtypes = [C.c_uint, C.c_uint, vp, vp, vp]
        L.ref_hrpb_build.restype = vp
        L.ref_hrpb_copy.argtypes = [vp, vp, vp]
        L.ref_hrpb_copy.restype = None
        L.ref_hrpb_stream_words.argtypes = [vp]
        L.ref_hrpb_stream_words.restype = C.c_ulonglong

    def set_threads(self, n: int) -> int:
        self.lib.ref_set_threads(int(n))
        return int(self.lib.ref_max_threads())

    def spmm_coo(self, rows, cols, vals, B, M, K):
        rows, cols, vals, B = _a(rows, np.uint32), _a(cols, np.uint32), _a(vals, np.float32), _a(B, np.float32)
        N = B.shape[1]
        out = np.empty((M, N), dtype=np.float32)
        self.lib.ref_spmm_coo(rows.ctypes.data, cols.ctypes.data, vals.ctypes.data, B.ctypes.data, out.ctypes.data, M, K, N, rows.size)
        return out

    def max_rel_err(self, C_ref, C_test):
        a, b = _a(C_ref, np.float32), _a(C_test, np.float32)
        return float(self.lib.ref_check_gemm_correctness_coo(a.ctypes.data, b.ctypes.data, a.shape[0], a.shape[1]))

    def mtx_read(self, path):
        h = self.lib.ref_mtx_open(str(path).encode())
        M, K, nnz = self.lib.ref_mtx_M(h), self.lib.ref_mtx_K(h), self.lib.ref_mtx_nnz(h)
        rp = np.empty(M + 1, np.uint32)
        cols = np.empty(max(nnz, 1), np.uint32)
        vals = np.empty(max(nnz, 1), np.float32)
        self.lib.ref_mtx_copy(h, rp.ctypes.data, cols.ctypes.data, vals.ctypes.data)
        return M, K, nnz, rp, cols[:nnz], vals[:nnz]

    def csr_from_mtx(self, path):
        """The reference's SparseCoo(path) -> CSR_Matrix(coo) (inc/SparseCoo.hpp:91, inc/CSR.hpp:69): nrows, ncols, nnz, rowPtr, cols, values."""
        L = C.CDLL(str(REF_LOADERS_PATH))
        L.ref_csr_from_mtx.argtypes = [C.c_char_p]
        L.ref_csr_from_mtx.restype = C.c_void_p
        for f in ("ref_csr_nrows", "ref_csr_ncols", "ref_csr_nnz"):
            getattr(L, f).argtypes = [C.c_void_p]
            getattr(L, f).restype = C.c_int
        L.ref_csr_copy.argtypes = [C.c_void_p] * 4
        h = L.ref_csr_from_mtx(str(path).encode())
        m, n, nnz = L.ref_csr_nrows(h), L.ref_csr_ncols(h), L.ref_csr_nnz(h)
        rp, cols, vals = np.empty(m + 1, np.int32), np.empty(max(nnz, 1), np.int32), np.empty(max(nnz, 1), np.float32)
        L.ref_csr_copy(h, rp.ctypes.data, cols.ctypes.data, vals.ctypes.data)
        return m, n, nnz, rp, cols[:nnz], vals[:nnz]

    def hrpb(self, M, K, row_ptr, cols, vals):
        """blockedRowPtr, activeCols and packed-stream size of the reference's preprocessing.
        Needs ascending unique columns per row and M, K multiples of 16 (data.cu:80-93)."""
        rp, cols, vals = _a(row_ptr, np.uint32), _a(cols, np.uint32), _a(vals, np.float32)
        h = self.lib.ref_hrpb_build(M, K, rp.ctypes.data, cols.ctypes.data, vals.ctypes.data)
        P, nb = self.lib.ref_hrpb_num_panels(h), self.lib.ref_hrpb_num_blocks(h)
        brp = np.empty(P + 1, np.uint32)
        ac = np.empty(max(nb * 16, 1), np.uint32)
        self.lib.ref_hrpb_copy(h, brp.ctypes.data, ac.ctypes.data)
        return brp, ac[: nb * 16], int(self.lib.ref_hrpb_stream_words(h))
