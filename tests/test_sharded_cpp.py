"""A C++ host that drives several GPUs from one process (one thread per GPU) through the C ABI:
cutespmm_comm_create_all, cutespmm_spmm_sharded (B from one rank; B row-sharded) and
cutespmm_spmm_sharded_host, every rank's rows checked against the CPU oracle inside the driver
(tests/cpp/sharded_driver.cpp).  The driver compiles anywhere (CPU check); it runs where at least two
GPUs are visible and skips itself elsewhere."""
import subprocess
from pathlib import Path

import pytest

import cutespmm_ae_b200 as cs
import oracle
from conftest import ROOT

CUDA = cs._build.CUDA_HOME


def build_driver(tmp: Path) -> Path:
    if not oracle.LIB_PATH.exists():
        oracle.build(ref_root=None)
    exe = tmp / "sharded_driver"
    cmd = ["g++", "-O2", "-std=c++17", "-pthread", f"-I{ROOT / 'include'}", f"-I{CUDA / 'include'}",
           str(ROOT / "tests" / "cpp" / "sharded_driver.cpp"), "-o", str(exe),
           str(cs._build.LIB), str(oracle.LIB_PATH), f"-L{CUDA / 'lib64'}", "-lcudart",
           f"-Wl,-rpath,{cs._build.LIB.parent}", f"-Wl,-rpath,{oracle.LIB_PATH.parent}", f"-Wl,-rpath,{CUDA / 'lib64'}"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


def test_sharded_driver_compiles(tmp_path):
    assert build_driver(tmp_path).exists()


@pytest.mark.gpu
def test_sharded_driver_matches_oracle_on_every_rank(tmp_path):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs in one process")
    exe = build_driver(tmp_path)
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    print(res.stdout)
    assert res.returncode == 0, res.stdout + res.stderr
    n = torch.cuda.device_count()
    assert res.stdout.count("relFro=") == 3 * n and "PASSED" in res.stdout
