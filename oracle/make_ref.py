"""TEST INFRASTRUCTURE: place an unmodified copy of the reference where the GPU tests can import it.

The reference (tsfast) is pure Python: its CPU kernels are C++ strings it compiles at run time
and its GPU kernels are Triton strings.  Parity of the drop-in is shown by running tsfast's OWN
modules and its OWN test files against the kernels of this repository, and the CPU/Triton
baselines of ``bench.py`` are tsfast's own code paths; both need the package on the machine with
the GPU.  This script copies

* the ``tsfast`` package                       -> ``oracle/_ref/tsfast/``
* the test files that cover the scan hot path  -> ``oracle/_ref/tests/``
* an empty ``test_data/`` (tsfast's ``conftest.py`` asserts that the folder exists; none of the
  copied tests reads from it)

from a tsfast checkout (``$TSFAST_CHECKOUT`` or the path given on the command line).  Nothing is
edited.  ``oracle/_ref/`` is listed in ``.gitignore``: the copy is never committed, it only
travels with the working tree.  Only tests, ``smoke()`` and ``bench.py``'s baseline legs import it;
the product (``tsfast_b200``) never does.

    python oracle/make_ref.py [/path/to/tsfast/checkout]
"""

from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"

# the reference's tests of the scan path: the scans, their backends, dispatch, and the four model
# families that call them
HOT_PATH_TESTS = [
    "conftest.py",
    "test_scan.py",
    "test_scan_diagonal_backends.py",
    "test_scan_selective_backends.py",
    "test_scan_allpole_backend.py",
    "test_scan_dispatch.py",
    "test_mamba.py",
    "test_lru.py",
    "test_s5.py",
    "test_dynonet.py",
    "test_dynonet_adjoint.py",
]


def make(checkout: Path) -> Path:
    pkg = checkout / "tsfast"
    if not (pkg / "models" / "_core" / "scan.py").exists():
        raise SystemExit(f"{checkout} is not a tsfast checkout (tsfast/models/_core/scan.py missing)")
    if DEST.exists():
        shutil.rmtree(DEST)
    DEST.mkdir(parents=True)
    shutil.copytree(pkg, DEST / "tsfast", ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    (DEST / "tests").mkdir()
    for name in HOT_PATH_TESTS:
        shutil.copy2(checkout / "tests" / name, DEST / "tests" / name)
    (DEST / "test_data").mkdir()
    (DEST / "SOURCE.txt").write_text(f"unmodified copy of the tsfast package and {len(HOT_PATH_TESTS)} of its test files, "
                                     "made by oracle/make_ref.py; not part of this repository's sources\n")
    return DEST


def available() -> Path | None:
    """The copied checkout, or None when it has not been made on this machine."""
    return DEST if (DEST / "tsfast" / "models" / "_core" / "scan.py").exists() else None


if __name__ == "__main__":
    src = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TSFAST_CHECKOUT", ""))
    if not str(src) or not src.exists():
        raise SystemExit("usage: python oracle/make_ref.py /path/to/tsfast/checkout   (or set TSFAST_CHECKOUT)")
    print(make(src))
