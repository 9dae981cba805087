import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "low-bit-optimizers_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def qmaps():
    import numpy as np
    out = {}
    for f in ("qmaps.npz", "qmaps_wide.npz"):
        z = np.load(os.path.join(GOLDEN, f))
        out.update({k: z[k] for k in z.files})
    return out
