import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden_ref():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_fixtures.npz"))


@pytest.fixture(scope="session")
def golden_nvfp4():
    return np.load(os.path.join(ROOT, "tests", "golden", "nvfp4_golden.npz"))


@pytest.fixture(scope="session")
def backend():
    """One context for the whole GPU session. Fails (does not skip) when the CUDA library is missing."""
    import thinfer_b200 as T

    be = T.Backend(0)
    yield be
    be.close()


def dev_scales_to_canonical(dev: np.ndarray, rows: int, k: int) -> np.ndarray:
    """Host-side inverse of the 128x4 tiled scale layout (for comparisons only)."""
    nb = k // 16
    ka = ((k + 63) // 64 + 3) // 4 * 4
    r = np.arange(rows)[:, None]
    b = np.arange(nb)[None, :]
    off = ((r // 128) * ka + b // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + (b % 4)
    return dev[off]


def rel_fro(a: np.ndarray, b: np.ndarray) -> float:
    a = a.astype(np.float64)
    b = b.astype(np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
