"""Shared pytest setup: marker registration, repo root on sys.path, golden-fixture loader."""

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def reference_checkout():
    """Folder holding an importable, unmodified tsfast: ``$TSFAST_CHECKOUT`` or the copy that
    ``oracle/make_ref.py`` places under ``oracle/_ref``; None when neither exists."""
    import os

    env = os.environ.get("TSFAST_CHECKOUT")
    for cand in ([Path(env)] if env else []) + [ROOT / "oracle" / "_ref"]:
        if (cand / "tsfast" / "models" / "_core" / "scan.py").exists():
            return cand
    return None


def import_tsfast_models():
    """``tsfast.models`` from the reference checkout (skips the calling test when unavailable).

    tsfast compiles its CPU kernels at run time with ``$CXX``; the system g++ is named because some
    images export a compiler without OpenMP support."""
    import os

    ref = reference_checkout()
    if ref is None:
        pytest.skip("no tsfast checkout (run `python oracle/make_ref.py <checkout>` or set TSFAST_CHECKOUT)")
    for var, exe in (("CXX", "/usr/bin/g++"), ("CC", "/usr/bin/gcc")):
        if os.path.exists(exe):
            os.environ[var] = exe
    if str(ref) not in sys.path:
        sys.path.insert(0, str(ref))
    try:
        import tsfast.models as m
    except Exception as e:  # a dependency of tsfast is missing on this machine
        pytest.skip(f"tsfast not importable: {e!r}")
    return m


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
