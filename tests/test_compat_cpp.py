"""The C++ compatibility header (MTX_READER / HRPB / SPMM_TC over the C ABI): a driver written like
the reference's run.cu compiles against it (CPU check) and produces the oracle's result on a GPU."""
import subprocess
from pathlib import Path

import numpy as np
import pytest

import cutespmm_ae_b200 as cs
import oracle
from conftest import GOLDEN, ROOT

CUDA = cs._build.CUDA_HOME


def build_driver(tmp: Path) -> Path:
    if not oracle.LIB_PATH.exists():
        oracle.build(ref_root=None)
    exe = tmp / "compat_driver"
    cmd = ["g++", "-O2", "-std=c++17", f"-I{ROOT / 'include'}", f"-I{CUDA / 'include'}",
           str(ROOT / "tests" / "cpp" / "compat_driver.cpp"), "-o", str(exe),
           str(cs._build.LIB), str(oracle.LIB_PATH), f"-L{CUDA / 'lib64'}", "-lcudart",
           f"-Wl,-rpath,{cs._build.LIB.parent}", f"-Wl,-rpath,{oracle.LIB_PATH.parent}", f"-Wl,-rpath,{CUDA / 'lib64'}"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


def write_mtx(path: Path, n=200, per_row=7, seed=3):
    rng = np.random.default_rng(seed)
    lines = []
    for r in range(n):
        for c in sorted(rng.choice(n, size=per_row, replace=False)):
            lines.append(f"{r + 1} {c + 1} 1.0")
    path.write_text(f"%%MatrixMarket matrix coordinate real general\n{n} {n} {len(lines)}\n" + "\n".join(lines) + "\n")


def test_compat_driver_compiles(tmp_path):
    assert build_driver(tmp_path).exists()


@pytest.mark.gpu
def test_compat_driver_matches_oracle(tmp_path):
    exe = build_driver(tmp_path)
    mtx = tmp_path / "rand200.mtx"
    write_mtx(mtx)
    for f in (mtx, GOLDEN / "symmetric_20.mtx"):
        res = subprocess.run([str(exe), str(f)], capture_output=True, text=True, timeout=300)
        assert res.returncode == 0, res.stdout + res.stderr
        assert res.stdout.count("relFro=") == 3
    bad = subprocess.run([str(exe), str(tmp_path / "missing.mtx")], capture_output=True, text=True)
    assert bad.returncode != 0 and "ERROR!!!" in bad.stderr  # the reference's error style: message, then exit
