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


def _write_mtx_with_values(path: Path, n=200, per_row=9, seed=11):
    rng = np.random.default_rng(seed)
    lines = []
    for r in rng.permutation(n):  # rows in shuffled order: the loaders sort the coordinate list
        for c in rng.choice(n, size=per_row, replace=False):
            lines.append(f"{r + 1} {c + 1} {rng.uniform(-2.0, 2.0):.6f}")
    path.write_text(f"%%MatrixMarket matrix coordinate real general\n{n} {n} {len(lines)}\n" + "\n".join(lines) + "\n")


@pytest.mark.gpu
def test_loader_surface_through_the_gpu(tmp_path):
    """SparseCoo(path) -> CSR_Matrix -> cutespmm_plan_from_csr -> product on the device -> CPU oracle, the file's own
    values honoured (the reference harness's call shape, gpu_kernels.cu:1290-1291)."""
    import oracle

    if not oracle.LIB_PATH.exists():
        oracle.build(ref_root=None)
    cuda = cs._build.CUDA_HOME
    exe = tmp_path / "loaders_gpu_driver"
    cmd = ["g++", "-O2", "-std=c++17", f"-I{ROOT / 'include'}", f"-I{cuda / 'include'}", str(ROOT / "tests" / "cpp" / "loaders_gpu_driver.cpp"),
           "-o", str(exe), str(cs._build.LIB), str(oracle.LIB_PATH), f"-L{cuda / 'lib64'}", "-lcudart",
           f"-Wl,-rpath,{cs._build.LIB.parent}", f"-Wl,-rpath,{oracle.LIB_PATH.parent}", f"-Wl,-rpath,{cuda / 'lib64'}"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    gen = tmp_path / "values200.mtx"
    _write_mtx_with_values(gen)
    for f, n in ((GOLDEN / "values_unsorted_6x6.mtx", 40), (gen, 64), (gen, 128), (GOLDEN / "symmetric_20.mtx", 33)):
        res = subprocess.run([str(exe), str(f), str(n)], capture_output=True, text=True, timeout=300)
        assert res.returncode == 0, res.stdout + res.stderr
        assert "relFro=" in res.stdout
