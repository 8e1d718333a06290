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


def rel_elementwise(a: np.ndarray, b: np.ndarray, floor: float = 1e-3) -> float:
    """max over elements of |a-b| / max(|b|, floor * max |b|): the stricter, element-wise reading of
    "max-rel".  An output far below the layer's maximum is held to its own size (down to the floor)
    instead of to the maximum, so a layer whose small outputs are all off shows up here and not in
    rel_to_max.  Sums of products that cancel carry an absolute error of the size of their terms, so
    near the floor this figure is legitimately orders of magnitude above rel_to_max."""
    a = np.asarray(a, np.float64).reshape(-1)
    b = np.asarray(b, np.float64).reshape(-1)
    m = max(np.abs(b).max(), 1e-30)
    return float((np.abs(a - b) / np.maximum(np.abs(b), floor * m)).max())


# (test id, label, rel_to_max, rel_elementwise, tolerance on rel_to_max): printed after the run, worst first per test
PARITY_LOG: list[tuple] = []


def parity(got, want, tol: float, label: str = "") -> float:
    """The parity check of one output: asserts rel_to_max < tol, records both error figures for the
    end-of-run table, returns rel_to_max."""
    r, e = rel_to_max(got, want), rel_elementwise(got, want)
    test = os.environ.get("PYTEST_CURRENT_TEST", "").split(" ")[0]
    PARITY_LOG.append((test, label, r, e, tol))
    assert r < tol, f"{label}: max|d|/max|ref| = {r:.3g} (tolerance {tol:g}); element-wise with floor {e:.3g}"
    return r


def pytest_terminal_summary(terminalreporter):
    if not PARITY_LOG:
        return
    worst: dict[str, tuple] = {}
    for test, label, r, e, tol in PARITY_LOG:
        w = worst.get(test)
        worst[test] = (max(r, w[0]) if w else r, max(e, w[1]) if w else e, tol, (w[3] if w else 0) + 1)
    tr = terminalreporter
    tr.write_line("parity: worst per test of max|d|/max|ref| (asserted) and of the element-wise max|d|/max(|ref|, 1e-3 max|ref|) (reported)")
    for test, (r, e, tol, count) in sorted(worst.items()):
        tr.write_line(f"  {test.split('::', 1)[-1][:100]:100s} n={count:<4d} rel_to_max={r:.3g} (tol {tol:g})  elementwise={e:.3g}")
