import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


# The library picks the window kernel by problem size (small problems: the warp-level kernel).  The parity
# tests are small, so they ask for the persistent tcgen05 kernel wherever it applies; the size rule and the
# warp-level kernels have tests of their own that set the variable themselves.
import os
os.environ.setdefault("MAT_WINDOW_KERNEL", "band")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    return np.load(ROOT / "tests" / "golden" / "reference_window.npz")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.lib()
    return O
