import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"
GOLDEN_CASES = ["uniform_256", "stencil_16x16", "elasticity_4", "rmat_s8", "ragged_48x64", "uniform_256_unsorted"]

# relative Frobenius error allowed between the GPU product and the CPU oracle: the bound the
# project states for TF32 multiplication with fp32 accumulation.  The CUDA-core kernel computes in
# full fp32 and lands orders of magnitude below it.
REL_FRO_TOL = 1e-3
REL_FRO_TOL_FP32 = 2e-6


@pytest.fixture(autouse=True)
def _mixed_plans_on_small_matrices():
    """Path auto sends a matrix with fewer than 4440 dense panels to the row kernel alone (it is faster there).  The
    fixtures of this suite are far smaller, and the point of most tests is the mixed plan -- tensor-core panels, row-kernel
    panels and the hand-over between them -- so the suite lowers the threshold to one panel; the default itself is
    checked by tests/test_host.py::test_auto_keeps_small_matrices_on_the_row_kernel."""
    import cutespmm_ae_b200 as cs

    old = cs.default_min_brick_panels
    cs.default_min_brick_panels = 1
    yield
    cs.default_min_brick_panels = old


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def load_golden(name):
    return dict(np.load(GOLDEN / f"{name}.npz"))


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle

    return oracle
