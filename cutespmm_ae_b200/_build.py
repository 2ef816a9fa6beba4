"""Builds libcutespmm.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m cutespmm_ae_b200._build [--force]

The shared object lands in cutespmm_ae_b200/lib/ next to the sources, so a snapshot of the tree
carries it to a machine that has a GPU but no compiler cache.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIBDIR = HERE / "lib"
LIB = LIBDIR / "libcutespmm.so"
SOURCES = ["capi.cu", "rows_kernel.cu", "brick_kernel.cu", "noalloc.cu", "slab_kernel.cu", "device_build.cu", "sharded.cu", "sddmm_kernel.cu", "plan_io.cu", "plan.cpp", "brick_build.cpp", "slab_build.cpp", "mtx_io.cpp"]
def _find_nvcc() -> str:
    import shutil

    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    return "nvcc"


NVCC = _find_nvcc()
CUDA_HOME = Path(os.environ.get("CUDA_HOME") or Path(NVCC).resolve().parent.parent)  # headers and libcudart for C++ hosts
FLAGS = [
    "-O3", "-std=c++17", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC,-fopenmp,-O3,-Wall,-Wno-unknown-pragmas",
    "-shared", "-lgomp", "-ldl",
]


def _sources():
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def _stamp() -> str:
    h = hashlib.sha256()
    for f in sorted(list(CSRC.glob("*")) + [HERE.parent / "include" / "cutespmm.h"]):
        if f.is_file():
            h.update(f.name.encode())
            h.update(f.read_bytes())
    h.update(" ".join(FLAGS).encode())
    return h.hexdigest()


def stale() -> bool:
    """True when the built library does not correspond to the current sources and flags."""
    stamp_file = LIBDIR / (LIB.name + ".stamp")
    return not (LIB.exists() and stamp_file.exists() and stamp_file.read_text() == _stamp())


def build(force: bool = False, verbose: bool = False) -> Path:
    LIBDIR.mkdir(exist_ok=True)
    stamp_file = LIBDIR / (LIB.name + ".stamp")
    stamp = _stamp()
    if not force and LIB.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return LIB
    cmd = [NVCC, *FLAGS, "-o", str(LIB), *map(str, _sources())]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd))
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libcutespmm.so")
    stamp_file.write_text(stamp)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
    print(LIB)
