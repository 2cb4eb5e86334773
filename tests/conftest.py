"""Shared pytest setup: marker registration, repo root on sys.path, golden-fixture loader."""

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


class GoldenCase:
    """One case of a golden ``.npz``: attribute access to its arrays, ``None`` when absent."""

    def __init__(self, data, name):
        self._d, self.name = data, name

    def __getattr__(self, key):
        k = f"{self.name}_{key}"
        return self._d[k] if k in self._d else None


def load_golden(kind):
    data = dict(np.load(GOLDEN / f"{kind}.npz"))
    return [GoldenCase(data, str(n)) for n in data["names"]]


def rel_err(a, b):
    """max|a-b| / max|b|, the metric of the reference's backend-equivalence tests."""
    a, b = np.asarray(a), np.asarray(b)
    if a.size == 0:
        return 0.0
    return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-30))


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O

    O.build()
    return O
