import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def lib_path():
    from turborag_b200 import build
    return build.build()


@pytest.fixture(scope="session")
def tq(lib_path):
    import turborag_b200
    return turborag_b200.TurboQuantWrapper(lib_path)


def load_golden(name):
    return np.load(GOLDEN / f"{name}.npz")


def rowwise_rel_err(a, b):
    """max over rows of max|a-b| / max|b| (rows = all leading dims)."""
    a = np.asarray(a, np.float32).reshape(-1, a.shape[-1])
    b = np.asarray(b, np.float32).reshape(-1, b.shape[-1])
    den = np.abs(b).max(axis=1)
    den[den == 0] = 1.0
    return float((np.abs(a - b).max(axis=1) / den).max())
