"""Shared test plumbing.

`-m "not gpu"` tests need no CUDA device: they pin the CPU checker (oracle/)
against the golden vectors the unmodified reference produced, and check the
host-side logic and the C ABI's symbol table.  `-m gpu` tests are the parity
tests proper: CUDA path (through the C ABI) against the checker."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden", "golden.npz")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def golden():
    return np.load(GOLDEN)


@pytest.fixture(scope="session")
def golden_cases():
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_golden
    return make_golden.cases()


def rel_to_max(a: np.ndarray, b: np.ndarray) -> float:
    """max |a-b| / max |b|: the per-layer relative error the tolerances refer to."""
    a = np.asarray(a, np.float64).reshape(-1)
    b = np.asarray(b, np.float64).reshape(-1)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))
