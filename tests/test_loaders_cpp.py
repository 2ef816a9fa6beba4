"""include/cutespmm_loaders.hpp (SparseCoo, CSR_Matrix, SMA) against what the reference's own loaders
(inc/SparseCoo.hpp:91-157, inc/CSR.hpp:162-187) produced for the same MatrixMarket files (golden vectors)."""
import subprocess
from pathlib import Path

import numpy as np
import pytest

import cutespmm_ae_b200 as cs
from conftest import GOLDEN, ROOT


@pytest.fixture(scope="module")
def dumper(tmp_path_factory):
    exe = tmp_path_factory.mktemp("loaders") / "loaders_dump"
    cmd = ["g++", "-O2", "-std=c++17", f"-I{ROOT / 'include'}", str(ROOT / "tests" / "cpp" / "loaders_dump.cpp"), "-o", str(exe),
           str(cs._build.LIB), f"-Wl,-rpath,{cs._build.LIB.parent}"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


@pytest.mark.parametrize("name", ["general_5x7", "symmetric_20", "values_unsorted_6x6"])
def test_sparsecoo_and_csr_match_reference_loaders(dumper, tmp_path, name):
    gd = dict(np.load(GOLDEN / f"loader_{name}.npz"))
    res = subprocess.run([str(dumper), str(GOLDEN / f"{name}.mtx"), str(tmp_path / "resaved.mtx")], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    lines = res.stdout.strip().split("\n")
    m, n, nnz = map(int, lines[0].split())
    assert (m, n, nnz) == (int(gd["nrows"]), int(gd["ncols"]), int(gd["nnz"]))
    assert np.array_equal(np.array(lines[1].split(), dtype=np.int64), gd["row_ptr"])
    assert np.array_equal(np.array(lines[2].split(), dtype=np.int64), gd["cols"])
    assert np.array_equal(np.array(lines[3].split(), dtype=np.float32), gd["vals"])
    assert lines[4] == "selfcheck ok"
