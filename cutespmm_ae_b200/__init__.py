"""cutespmm_ae_b200 -- Python binding of libcutespmm, the B200 (sm_100a) sparse x dense product.

Everything here is a thin ctypes layer over the C ABI declared in include/cutespmm.h; the classes
mirror the reference project's operator objects for this path:

    reference (aFatCa/cuTeSpMM_AE)                    here
    ------------------------------------------------  ---------------------------------
    MTX_READER(path)               IO.cu:10           MtxReader(path)
    HRPB(M, K, rowPtr, cols, vals) data.cu:80         Plan(M, K, row_ptr, cols, vals)
    SPMM_TC(M, K, N, blockedRowPtr).run(...)          Plan.spmm(B, C) / Plan.spmm_host(B, C)
                                   spmm.cu:276,823

There is no CPU implementation behind these calls: if the shared library is missing the import
fails, and executing a plan without a CUDA device returns an error.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import _build

__all__ = ["CuteSpmmError", "Plan", "Comm", "MtxReader", "partition_rows", "spmm_csr_noalloc", "lib", "PATH_AUTO", "PATH_ROWS",
           "PATH_BRICK", "PATH_SLAB", "B_RESIDENT", "B_FROM_ROOT", "B_ROW_SHARDED"]

PATH_AUTO, PATH_ROWS, PATH_BRICK, PATH_SLAB = 0, 1, 2, 3
FLAG_ROUND_B_NEAREST = 1
REORDER_NONE, REORDER_CLUSTER_ROWS, REORDER_SIMILAR_ROWS = 0, 1, 2
B_RESIDENT, B_FROM_ROOT, B_ROW_SHARDED = 0, 1, 2  # cutespmm_b_mode_t
COMM_ID_BYTES = 128
# What Plan(...) passes as cutespmm_options_t::min_brick_panels when the caller gives none (0 = the library's default).
default_min_brick_panels = 0


class CuteSpmmError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"libcutespmm: {message} (status {status})")
        self.status = status


class Options(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("path", C.c_uint32), ("split_nnz", C.c_uint32),
                ("tile_nnz", C.c_uint32), ("brick_density", C.c_float), ("flags", C.c_uint32), ("reorder", C.c_uint32),
                ("min_brick_panels", C.c_uint32)]


class PlanInfo(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "M", "K", "nnz", "num_panels", "num_blocks", "num_tiles", "num_long_rows", "num_chunks",
        "brick_panels", "num_bricks", "device_bytes", "scratch_bytes_per_col")]


def _load() -> C.CDLL:
    path = _build.LIB
    # (re)build when the library is missing or older than its sources; needs nvcc only, not a GPU
    if not path.exists() or (_build.stale() and Path(_build.NVCC).exists()):
        _build.build()
    lib = C.CDLL(str(path))
    u64p, u32p, f32p, vp = C.POINTER(C.c_uint64), C.POINTER(C.c_uint32), C.POINTER(C.c_float), C.c_void_p
    sig = {
        "cutespmm_status_string": (C.c_char_p, [C.c_int]),
        "cutespmm_last_error": (C.c_char_p, []),
        "cutespmm_version": (C.c_int, []),
        "cutespmm_plan_create": (C.c_int, [C.POINTER(vp), C.c_uint64, C.c_uint64, vp, vp, vp, C.POINTER(Options)]),
        "cutespmm_plan_create_u32": (C.c_int, [C.POINTER(vp), C.c_uint32, C.c_uint32, vp, vp, vp, C.POINTER(Options)]),
        "cutespmm_plan_build_host": (C.c_int, [C.POINTER(vp), C.c_uint64, C.c_uint64, vp, vp, vp, C.POINTER(Options)]),
        "cutespmm_plan_create_device": (C.c_int, [C.POINTER(vp), C.c_uint64, C.c_uint64, vp, vp, vp, C.POINTER(Options), vp]),
        "cutespmm_plan_destroy": (C.c_int, [vp]),
        "cutespmm_plan_save": (C.c_int, [vp, C.c_char_p]),
        "cutespmm_plan_load": (C.c_int, [C.POINTER(vp), C.c_char_p, C.c_int]),
        "cutespmm_plan_info": (C.c_int, [vp, C.POINTER(PlanInfo)]),
        "cutespmm_plan_blocked_row_ptr": (C.c_int, [vp, vp]),
        "cutespmm_plan_active_cols": (C.c_int, [vp, vp]),
        "cutespmm_plan_decode_csr": (C.c_int, [vp, vp, vp, vp]),
        "cutespmm_spmm": (C.c_int, [vp, vp, C.c_uint64, vp, C.c_uint64, C.c_uint32, vp]),
        "cutespmm_spmm_host": (C.c_int, [vp, vp, C.c_uint64, vp, C.c_uint64, C.c_uint32, vp, f32p]),
        "cutespmm_spmm_launch_count": (C.c_int, [vp, C.c_uint32]),
        "cutespmm_spmm_kernels": (C.c_int, [vp, C.c_uint32]),
        "cutespmm_plan_set_values": (C.c_int, [vp, vp, vp]),
        "cutespmm_spmm_csr_noalloc": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, vp, vp, vp, vp, C.c_uint64, vp,
                                                C.c_uint64, C.c_uint32, vp]),
        "cutespmm_plan_device_status": (C.c_int, [vp, u32p]),
        "cutespmm_sddmm": (C.c_int, [vp, vp, C.c_uint64, vp, C.c_uint64, C.c_uint32, C.c_int, vp, vp]),
        "cutespmm_comm_unique_id": (C.c_int, [vp]),
        "cutespmm_comm_create": (C.c_int, [C.POINTER(vp), C.c_int, C.c_int, vp]),
        "cutespmm_comm_create_all": (C.c_int, [C.POINTER(vp), C.c_int, C.POINTER(C.c_int)]),
        "cutespmm_comm_adopt": (C.c_int, [C.POINTER(vp), vp, C.c_int, C.c_int]),
        "cutespmm_comm_create_stub": (C.c_int, [C.POINTER(vp), C.c_int, C.c_int]),
        "cutespmm_comm_stub_log": (C.c_int, [vp, C.c_uint32, vp, vp, vp, u32p]),
        "cutespmm_comm_info": (C.c_int, [vp, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
        "cutespmm_comm_destroy": (C.c_int, [vp]),
        "cutespmm_spmm_sharded": (C.c_int, [vp, vp, C.c_int, C.c_int, vp, C.c_uint64, vp, vp, C.c_uint64, C.c_uint32, vp]),
        "cutespmm_spmm_sharded_host": (C.c_int, [vp, vp, vp, C.c_uint64, vp, vp, C.c_uint64, C.c_uint32, vp, f32p, f32p]),
        "cutespmm_plan_reserve_host_staging": (C.c_int, [vp, C.c_uint32, C.c_int]),
        "cutespmm_sharded_transfers": (C.c_int, [vp, C.c_int, C.c_int, C.c_uint64, C.c_uint64, vp, C.c_uint32, vp, vp, vp, u32p]),
        "cutespmm_partition_rows": (C.c_int, [C.c_uint64, vp, C.c_uint32, C.c_uint32, C.c_uint32, vp]),
        "cutespmm_mtx_open": (C.c_int, [C.POINTER(vp), C.c_char_p, C.c_int]),
        "cutespmm_mtx_dims": (C.c_int, [vp, u32p, u32p, u32p]),
        "cutespmm_mtx_arrays": (C.c_int, [vp, C.POINTER(u32p), C.POINTER(u32p), C.POINTER(f32p)]),
        "cutespmm_mtx_close": (C.c_int, [vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def _check(status: int) -> None:
    if status != 0:
        msg = lib.cutespmm_last_error().decode() or lib.cutespmm_status_string(status).decode()
        raise CuteSpmmError(status, msg)


def _np(a, dtype) -> np.ndarray:
    """Host array view of a numpy array or CPU torch tensor, converted to `dtype`, contiguous."""
    if hasattr(a, "detach"):
        a = a.detach().cpu().numpy()
    return np.ascontiguousarray(a, dtype=dtype)


class Plan:
    """Device-resident, preprocessed A.  Counterpart of HRPB (data.cu:54-340) plus the work list
    of SPMM_TC (spmm.cu:691-822).  `host_only=True` builds the plan without touching CUDA."""

    def __init__(self, M: int, K: int, row_ptr, cols, vals, *, path: int = PATH_AUTO, split_nnz: int = 0,
                 tile_nnz: int = 0, brick_density: float = 0.0, round_b_nearest: bool = False, reorder: int | str = 0, min_brick_panels: int = 0,
                 host_only: bool = False):
        self._h = C.c_void_p()
        rp, cc, vv = _np(row_ptr, np.uint64), _np(cols, np.uint32), _np(vals, np.float32)
        if rp.shape[0] != M + 1:
            raise ValueError("row_ptr must have M+1 entries")
        reorder = {"none": REORDER_NONE, "cluster": REORDER_CLUSTER_ROWS, "similar": REORDER_SIMILAR_ROWS}.get(reorder, reorder)
        opts = Options(C.sizeof(Options), path, split_nnz, tile_nnz, brick_density, FLAG_ROUND_B_NEAREST if round_b_nearest else 0, reorder,
                       min_brick_panels or default_min_brick_panels)
        fn = lib.cutespmm_plan_build_host if host_only else lib.cutespmm_plan_create
        _check(fn(C.byref(self._h), M, K, rp.ctypes.data, cc.ctypes.data, vv.ctypes.data, C.byref(opts)))
        self.M, self.K, self.nnz = M, K, int(rp[-1])

    @classmethod
    def from_csr(cls, A, **kw) -> "Plan":
        """From a generators.CsrMatrix (or anything with M, K, row_ptr, cols, vals)."""
        return cls(A.M, A.K, A.row_ptr, A.cols, A.vals, **kw)

    @classmethod
    def from_device_csr(cls, M: int, K: int, row_ptr, cols, vals, *, path: int = PATH_AUTO, split_nnz: int = 0,
                        tile_nnz: int = 0, min_brick_panels: int = 0, stream=None) -> "Plan":
        """From CSR tensors that live on the GPU (row_ptr: M+1 int32, cols: nnz int32, vals: nnz float32): the
        nonzeros are packed, the 16-row panels analysed and the tensor-core bricks written on the device
        (cutespmm_plan_create_device); path auto, rows or brick."""
        import torch

        for t, dt in ((row_ptr, torch.int32), (cols, torch.int32), (vals, torch.float32)):
            if not t.is_cuda or t.dtype != dt or not t.is_contiguous():
                raise ValueError("row_ptr/cols must be contiguous CUDA int32 tensors, vals a contiguous CUDA float32 tensor")
        if row_ptr.numel() != M + 1 or cols.numel() != vals.numel():
            raise ValueError("row_ptr must have M+1 entries; cols and vals the same length")
        self = cls.__new__(cls)
        self._h = C.c_void_p()
        opts = Options(C.sizeof(Options), path, split_nnz, tile_nnz, 0.0, 0, 0, min_brick_panels or default_min_brick_panels)
        st = (stream or torch.cuda.current_stream(vals.device)).cuda_stream
        _check(lib.cutespmm_plan_create_device(C.byref(self._h), M, K, row_ptr.data_ptr(), cols.data_ptr(), vals.data_ptr(),
                                               C.byref(opts), st))
        self.M, self.K = M, K
        self.nnz = self.info()["nnz"]
        return self

    def save(self, path) -> None:
        """Writes the plan to `path` (cutespmm_plan_save)."""
        _check(lib.cutespmm_plan_save(self._h, str(path).encode()))

    @classmethod
    def load(cls, path, host_only: bool = False) -> "Plan":
        """A plan saved with `save`, uploaded to the current CUDA device (or host-only)."""
        self = cls.__new__(cls)
        self._h = C.c_void_p()
        _check(lib.cutespmm_plan_load(C.byref(self._h), str(path).encode(), 1 if host_only else 0))
        i = self.info()
        self.M, self.K, self.nnz = i["M"], i["K"], i["nnz"]
        return self

    def close(self) -> None:
        if getattr(self, "_h", None) and self._h.value and lib is not None:  # lib is None at interpreter shutdown
            lib.cutespmm_plan_destroy(self._h)
            self._h = C.c_void_p()

    __del__ = close

    def info(self) -> dict:
        i = PlanInfo()
        _check(lib.cutespmm_plan_info(self._h, C.byref(i)))
        return {n: int(getattr(i, n)) for n, _ in PlanInfo._fields_}

    def blocked_row_ptr(self) -> np.ndarray:
        out = np.empty(self.info()["num_panels"] + 1, dtype=np.uint32)
        _check(lib.cutespmm_plan_blocked_row_ptr(self._h, out.ctypes.data))
        return out

    def active_cols(self) -> np.ndarray:
        out = np.empty(self.info()["num_blocks"] * 16, dtype=np.uint32)
        _check(lib.cutespmm_plan_active_cols(self._h, out.ctypes.data))
        return out

    def decode_csr(self):
        rp = np.empty(self.M + 1, dtype=np.uint64)
        cc = np.empty(self.nnz, dtype=np.uint32)
        vv = np.empty(self.nnz, dtype=np.float32)
        _check(lib.cutespmm_plan_decode_csr(self._h, rp.ctypes.data, cc.ctypes.data, vv.ctypes.data))
        n = int(rp[-1])
        return rp, cc[:n], vv[:n]

    def launch_count(self, N: int) -> int:
        return lib.cutespmm_spmm_launch_count(self._h, N)

    def kernels(self, N: int) -> str:
        """The kernels a product of N columns runs: "rows", "brick", "slab" or a "+"-joined combination."""
        mask = lib.cutespmm_spmm_kernels(self._h, N)
        return "+".join(n for b, n in ((2, "brick"), (4, "slab"), (1, "rows")) if mask & b) or "none"

    def device_status(self) -> int:
        s = C.c_uint32()
        _check(lib.cutespmm_plan_device_status(self._h, C.byref(s)))
        return s.value

    def spmm(self, B, Cout=None, stream=None):
        """C = A @ B with B, C CUDA fp32 torch tensors (row-major, last stride 1).  Runs on
        `stream` (a torch.cuda.Stream) or on torch's current stream."""
        import torch

        if not B.is_cuda or B.dtype != torch.float32 or B.dim() != 2 or B.stride(1) != 1:
            raise ValueError("B must be a 2-D CUDA fp32 tensor with unit column stride")
        if B.shape[0] != self.K:
            raise ValueError(f"B has {B.shape[0]} rows, A has {self.K} columns")
        N = B.shape[1]
        if Cout is None:
            Cout = torch.empty((self.M, N), dtype=torch.float32, device=B.device)
        if not Cout.is_cuda or Cout.dtype != torch.float32 or Cout.shape != (self.M, N) or Cout.stride(1) != 1:
            raise ValueError("C must be an M x N CUDA fp32 tensor with unit column stride")
        st = (stream or torch.cuda.current_stream(B.device)).cuda_stream
        _check(lib.cutespmm_spmm(self._h, B.data_ptr(), B.stride(0) if B.shape[0] > 1 else max(N, 1), Cout.data_ptr(),
                                 Cout.stride(0) if self.M > 1 else max(N, 1), N, st))
        return Cout

    def spmm_host(self, B, Cout=None, stream=None):
        """Host buffers in, host buffers out (numpy arrays or CPU torch tensors; pin them for full
        copy bandwidth).  Returns (C, kernel_ms)."""
        import torch

        tb = B if hasattr(B, "data_ptr") else torch.from_numpy(np.ascontiguousarray(B, dtype=np.float32))
        if tb.is_cuda or tb.dtype != torch.float32 or tb.dim() != 2 or tb.stride(1) != 1 or tb.shape[0] != self.K:
            raise ValueError("B must be a K x N CPU fp32 tensor with unit column stride")
        N = tb.shape[1]
        if Cout is None:
            Cout = torch.empty((self.M, N), dtype=torch.float32)
        tc = Cout if hasattr(Cout, "data_ptr") else torch.from_numpy(Cout)
        ms = C.c_float(0.0)
        st = stream.cuda_stream if stream is not None else None
        _check(lib.cutespmm_spmm_host(self._h, tb.data_ptr(), tb.stride(0) if self.K > 1 else max(N, 1), tc.data_ptr(),
                                      tc.stride(0) if self.M > 1 else max(N, 1), N, st, C.byref(ms)))
        return Cout, ms.value

    def sddmm(self, X, Y, out=None, *, scale_by_values: bool = False, stream=None):
        """out[j] = (A_j if scale_by_values else 1) * <X[row of j], Y[column of j]> for every stored nonzero j, in the
        plan's storage order (cutespmm_sddmm).  X: M x N, Y: K x N CUDA fp32 tensors with unit column stride."""
        import torch

        for t, rows, name in ((X, self.M, "X"), (Y, self.K, "Y")):
            if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1 or t.shape[0] != rows:
                raise ValueError(f"{name} must be a {rows} x N CUDA fp32 tensor with unit column stride")
        if X.shape[1] != Y.shape[1]:
            raise ValueError("X and Y must have the same number of columns")
        N = X.shape[1]
        if out is None:
            out = torch.empty(self.nnz, dtype=torch.float32, device=X.device)
        if not out.is_cuda or out.dtype != torch.float32 or out.numel() != self.nnz or not out.is_contiguous():
            raise ValueError("out must be a contiguous CUDA fp32 tensor with one element per nonzero")
        st = (stream or torch.cuda.current_stream(X.device)).cuda_stream
        _check(lib.cutespmm_sddmm(self._h, X.data_ptr(), X.stride(0) if self.M > 1 else max(N, 1), Y.data_ptr(),
                                  Y.stride(0) if self.K > 1 else max(N, 1), N, 1 if scale_by_values else 0, out.data_ptr(), st))
        return out

    def set_values(self, vals, stream=None):
        """New values for the same pattern (cutespmm_plan_set_values): vals is a CUDA fp32 tensor with one element per
        nonzero in the plan's storage order, e.g. normalised output of `sddmm`."""
        import torch

        if not vals.is_cuda or vals.dtype != torch.float32 or vals.numel() != self.nnz or not vals.is_contiguous():
            raise ValueError("vals must be a contiguous CUDA fp32 tensor with one element per nonzero")
        st = (stream or torch.cuda.current_stream(vals.device)).cuda_stream
        _check(lib.cutespmm_plan_set_values(self._h, vals.data_ptr(), st))

    def spmm_sharded(self, comm: "Comm", B, Cout=None, *, b_mode: int = B_RESIDENT, root: int = 0, b_bounds=None, stream=None):
        """This rank's rows of A @ B through cutespmm_spmm_sharded: B (K x N, contiguous, on this rank's GPU) is
        completed in place by the exchange `b_mode` names (B_FROM_ROOT: broadcast from `root`; B_ROW_SHARDED: this
        rank holds rows [b_bounds[rank], b_bounds[rank+1]) and the others arrive by all-gather), then multiplied."""
        import torch

        if not B.is_cuda or B.dtype != torch.float32 or B.dim() != 2 or B.shape[0] != self.K or not B.is_contiguous():
            raise ValueError("B must be a contiguous K x N CUDA fp32 tensor")
        N = B.shape[1]
        if Cout is None:
            Cout = torch.empty((self.M, N), dtype=torch.float32, device=B.device)
        if not Cout.is_cuda or Cout.dtype != torch.float32 or Cout.shape != (self.M, N) or Cout.stride(1) != 1:
            raise ValueError("C must be an M x N CUDA fp32 tensor with unit column stride")
        bb = None if b_bounds is None else _np(b_bounds, np.uint64)
        if bb is not None and bb.shape[0] != comm.nranks + 1:
            raise ValueError("b_bounds must have nranks+1 entries")
        st = (stream or torch.cuda.current_stream(B.device)).cuda_stream
        _check(lib.cutespmm_spmm_sharded(self._h, comm._h, b_mode, root, B.data_ptr(), max(N, 1), None if bb is None else bb.ctypes.data,
                                         Cout.data_ptr(), Cout.stride(0) if self.M > 1 else max(N, 1), N, st))
        return Cout

    def spmm_sharded_host(self, comm, B_rows, b_bounds, Cout=None, stream=None):
        """Host buffers in and out with several ranks (cutespmm_spmm_sharded_host): `B_rows` is this rank's slice of B
        only, rows [b_bounds[rank], b_bounds[rank+1]) as a CPU fp32 tensor (pinned for full copy bandwidth); every rank
        uploads its slice over its own PCIe link and the slices are exchanged over NVLink.  Returns
        (C rows of this rank, kernel_ms, exchange_ms)."""
        import torch

        bb = _np(b_bounds, np.uint64)
        nranks, rank = (comm.nranks, comm.rank) if comm is not None else (1, 0)
        if bb.shape[0] != nranks + 1:
            raise ValueError("b_bounds must have nranks+1 entries")
        rows = int(bb[rank + 1] - bb[rank])
        tb = B_rows
        if tb.is_cuda or tb.dtype != torch.float32 or tb.dim() != 2 or tb.stride(1) != 1 or tb.shape[0] != rows:
            raise ValueError(f"B_rows must be a {rows} x N CPU fp32 tensor with unit column stride")
        N = tb.shape[1]
        if Cout is None:
            Cout = torch.empty((self.M, N), dtype=torch.float32)
        if Cout.is_cuda or Cout.dtype != torch.float32 or tuple(Cout.shape) != (self.M, N) or Cout.stride(1) != 1:
            raise ValueError("C must be an M x N CPU fp32 tensor with unit column stride")
        kms, xms = C.c_float(0.0), C.c_float(0.0)
        st = stream.cuda_stream if stream is not None else None
        _check(lib.cutespmm_spmm_sharded_host(self._h, comm._h if comm is not None else None, tb.data_ptr(),
                                              tb.stride(0) if rows > 1 else max(N, 1), bb.ctypes.data, Cout.data_ptr(),
                                              Cout.stride(0) if self.M > 1 else max(N, 1), N, st, C.byref(kms), C.byref(xms)))
        return Cout, kms.value, xms.value


class Comm:
    """A communicator of the library (cutespmm_comm_*): NCCL underneath, opened at run time.  One per rank; the
    rank's CUDA device must be current when it is created.

    `Comm.from_torch(group)` builds one for every rank of a torch.distributed group (the id travels through the
    group); `Comm.stub(nranks, rank)` records transfers instead of sending them (tests without GPUs)."""

    def __init__(self, handle, nranks: int, rank: int):
        self._h, self.nranks, self.rank = handle, nranks, rank

    @classmethod
    def create(cls, nranks: int, rank: int, unique_id: bytes) -> "Comm":
        h = C.c_void_p()
        buf = C.create_string_buffer(bytes(unique_id), COMM_ID_BYTES)
        _check(lib.cutespmm_comm_create(C.byref(h), nranks, rank, buf))
        return cls(h, nranks, rank)

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(COMM_ID_BYTES)
        _check(lib.cutespmm_comm_unique_id(buf))
        return buf.raw

    @classmethod
    def from_torch(cls, group=None) -> "Comm":
        import torch.distributed as dist

        rank, world = dist.get_rank(group), dist.get_world_size(group)
        box = [cls.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return cls.create(world, rank, box[0])

    @classmethod
    def stub(cls, nranks: int, rank: int) -> "Comm":
        h = C.c_void_p()
        _check(lib.cutespmm_comm_create_stub(C.byref(h), nranks, rank))
        return cls(h, nranks, rank)

    def transfers(self, b_mode: int, K: int, N: int, b_bounds=None, root: int = 0):
        """[(root, element offset, element count)] of the exchange of one contiguous K x N block of B."""
        bb = None if b_bounds is None else _np(b_bounds, np.uint64)
        cap = self.nranks + 1
        roots, offs, cnts, n = np.zeros(cap, np.int32), np.zeros(cap, np.uint64), np.zeros(cap, np.uint64), C.c_uint32()
        _check(lib.cutespmm_sharded_transfers(self._h, b_mode, root, K, N, None if bb is None else bb.ctypes.data, cap,
                                              roots.ctypes.data, offs.ctypes.data, cnts.ctypes.data, C.byref(n)))
        return [(int(roots[i]), int(offs[i]), int(cnts[i])) for i in range(n.value)]

    def stub_log(self):
        cap = 4096
        roots, offs, cnts, n = np.zeros(cap, np.int32), np.zeros(cap, np.uint64), np.zeros(cap, np.uint64), C.c_uint32()
        _check(lib.cutespmm_comm_stub_log(self._h, cap, roots.ctypes.data, offs.ctypes.data, cnts.ctypes.data, C.byref(n)))
        return [(int(roots[i]), int(offs[i]), int(cnts[i])) for i in range(min(n.value, cap))]

    def close(self) -> None:
        if getattr(self, "_h", None) and self._h.value and lib is not None:
            lib.cutespmm_comm_destroy(self._h)
            self._h = C.c_void_p()

    __del__ = close


def spmm_csr_noalloc(M: int, K: int, row_ptr, cols, vals, B, Cout, stream=None):
    """C = A @ B from CSR tensors that already live on the GPU (row_ptr/cols int32, vals/B/C fp32),
    through the entry point that allocates nothing (cutespmm_spmm_csr_noalloc): for callers that
    may not allocate device memory when they call.  The caller provides C."""
    import torch

    for t, dt in ((row_ptr, torch.int32), (cols, torch.int32), (vals, torch.float32), (B, torch.float32), (Cout, torch.float32)):
        if not t.is_cuda or t.dtype != dt:
            raise ValueError("all operands must be CUDA tensors: row_ptr/cols int32, vals/B/C float32")
    if B.dim() != 2 or Cout.dim() != 2:
        raise ValueError("B and C must be 2-D")
    if not (row_ptr.is_contiguous() and cols.is_contiguous() and vals.is_contiguous()) or B.stride(1) != 1 or Cout.stride(1) != 1:
        raise ValueError("CSR arrays must be contiguous; B and C need unit column stride")
    N = B.shape[1]
    # the call itself cannot see the sizes of the buffers behind the pointers: check them here, as Plan.spmm does
    if row_ptr.numel() != M + 1 or cols.numel() != vals.numel():
        raise ValueError("row_ptr must have M+1 entries; cols and vals the same length")
    if B.shape[0] != K:
        raise ValueError(f"B has {B.shape[0]} rows, A has {K} columns")
    if tuple(Cout.shape) != (M, N):
        raise ValueError(f"C must be {M} x {N}, got {tuple(Cout.shape)}")
    if len({t.device for t in (row_ptr, cols, vals, B, Cout)}) != 1:
        raise ValueError("all operands must live on one device")
    st = (stream or torch.cuda.current_stream(B.device)).cuda_stream
    _check(lib.cutespmm_spmm_csr_noalloc(M, K, cols.numel(), row_ptr.data_ptr(), cols.data_ptr(), vals.data_ptr(), B.data_ptr(),
                                         B.stride(0) if K > 1 else max(N, 1), Cout.data_ptr(),
                                         Cout.stride(0) if M > 1 else max(N, 1), N, st))
    return Cout


def partition_rows(row_ptr, nparts: int, align_rows: int = 16, row_cost: int = 2) -> np.ndarray:
    """nnz-balanced contiguous row ranges, boundaries multiples of `align_rows`; returns nparts+1 bounds."""
    rp = _np(row_ptr, np.uint64)
    out = np.empty(nparts + 1, dtype=np.uint64)
    _check(lib.cutespmm_partition_rows(rp.shape[0] - 1, rp.ctypes.data, nparts, align_rows, row_cost, out.ctypes.data))
    return out


class MtxReader:
    """MatrixMarket loader with the fields MTX_READER exposes (IO.cu:4-9): M, K, nnz, rowPtr, cols, vals."""

    def __init__(self, path: str | Path, pattern_only: bool = True):
        h = C.c_void_p()
        st = lib.cutespmm_mtx_open(C.byref(h), str(path).encode(), 1 if pattern_only else 0)
        if st != 0:
            raise CuteSpmmError(st, f"cannot read MatrixMarket file {path}")
        try:
            M, K, nnz = C.c_uint32(), C.c_uint32(), C.c_uint32()
            _check(lib.cutespmm_mtx_dims(h, C.byref(M), C.byref(K), C.byref(nnz)))
            rp, cc, vv = C.POINTER(C.c_uint32)(), C.POINTER(C.c_uint32)(), C.POINTER(C.c_float)()
            _check(lib.cutespmm_mtx_arrays(h, C.byref(rp), C.byref(cc), C.byref(vv)))
            self.M, self.K, self.nnz = M.value, K.value, nnz.value
            self.rowPtr = np.ctypeslib.as_array(rp, shape=(self.M + 1,)).copy()
            self.cols = np.ctypeslib.as_array(cc, shape=(max(self.nnz, 1),))[: self.nnz].copy()
            self.vals = np.ctypeslib.as_array(vv, shape=(max(self.nnz, 1),))[: self.nnz].copy()
        finally:
            lib.cutespmm_mtx_close(h)
