"""CPU-side checks of the C-ABI boundary: the library loads without a GPU, exports every symbol
the public header declares, the Python binding lists exactly those symbols, and the host-side
argument checks answer without touching a device."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "b200scan.h"


def _declared():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from tsfast_b200 import build, _lib

    build.build()
    return _lib.lib()


def test_header_symbols_exported(lib):
    names = _declared()
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), f"{n} declared in b200scan.h but not exported"


def test_binding_covers_header(lib):
    from tsfast_b200 import _lib

    assert sorted(_lib.SIGNATURES) == _declared()


def test_version_and_workspace_queries(lib):
    assert lib.b200_version() >= 100
    for fn in (lib.b200_diag_workspace_bytes, lib.b200_sel_workspace_bytes):
        small, big = fn(0, 0, 2, 7, 3), fn(0, 1, 64, 4096, 256)
        assert 0 < small < big
        assert fn(0, 0, 0, 0, 0) > 0  # empty problems still get a valid size


def test_argument_errors_without_gpu(lib):
    """Rejected on the host before any CUDA call: bad dtype, null pointers, missing workspace."""
    z = ctypes.c_void_p(None)
    assert lib.b200_sel_fwd(7, 1, 1, 1, z, z, z, z, z, 0, z) == 1
    assert lib.b200_sel_fwd(0, 1, 1, 1, z, z, z, z, z, 0, z) == 1
    fake = ctypes.c_void_p(256)
    assert lib.b200_sel_fwd(0, 1, 1, 1, fake, fake, z, fake, z, 0, z) == 2
    assert lib.b200_diag_fwd(0, 0, 5, 3, z, z, z, z, z, 0, z) == 0  # empty problem is a no-op


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from tsfast_b200 import _lib

    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setenv("B200SCAN_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()
    monkeypatch.delenv("B200SCAN_LIB")
    monkeypatch.setattr(_lib, "_LIB", None)
    _lib.lib()


def test_ops_refuse_cpu_tensors():
    import torch
    import tsfast_b200

    with pytest.raises(RuntimeError, match="CUDA"):
        tsfast_b200.selective_recurrence(torch.rand(2, 5, 3), torch.rand(2, 5, 3))
