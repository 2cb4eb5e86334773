"""ctypes binding of ``libb200scan.so``, the C-ABI CUDA library behind every op of this package.

The library is built in-tree by ``python -m tsfast_b200.build``.  There is no fallback: a missing
or unloadable library raises, and so does every non-zero status an entry point returns.
"""

from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
_DEFAULT = _PKG / "lib" / "libb200scan.so"
_LIB: ctypes.CDLL | None = None

F32, C64 = 0, 1
_ERRORS = {
    1: "B200_ERR_ARG (bad pointer, size or dtype)",
    2: "B200_ERR_WORKSPACE (workspace missing, misaligned or too small)",
    3: "B200_ERR_LAUNCH (the CUDA runtime refused a memset or launch)",
    4: "B200_ERR_UNSUPPORTED (size outside what the kernel handles)",
    5: "B200_ERR_TIMEOUT (a look-back wait ran out of polls on the device)",
}

_i64, _int, _vp, _sz = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t
# name -> (restype, argtypes); must list every symbol include/b200scan.h declares
SIGNATURES = {
    "b200_version": (_int, []),
    "b200_workspace_status": (_int, [_vp, _vp]),
    "b200_diag_workspace_bytes": (_sz, [_int, _int, _i64, _i64, _i64]),
    "b200_diag_fwd": (_int, [_int, _i64, _i64, _i64] + [_vp] * 5 + [_sz, _vp]),
    "b200_diag_bwd": (_int, [_int, _i64, _i64, _i64] + [_vp] * 8 + [_sz, _vp]),
    "b200_diag_fwd_static": (_int, [_int, _i64, _i64, _i64] + [_vp] * 5),
    "b200_diag_static_status": (_int, [_vp]),
    "b200_diag_probe": (_int, [_int, _int, _int, _i64, _int, _int, _int, _i64, _i64, _i64] + [_vp] * 8 + [_sz, _vp]),
    "b200_sel_workspace_bytes": (_sz, [_int, _int, _i64, _i64, _i64]),
    "b200_sel_fwd": (_int, [_int, _i64, _i64, _i64] + [_vp] * 5 + [_sz, _vp]),
    "b200_sel_bwd": (_int, [_int, _i64, _i64, _i64] + [_vp] * 8 + [_sz, _vp]),
    "b200_allpole_fwd": (_int, [_i64, _i64, _i64] + [_vp] * 5),
    "b200_allpole_bwd": (_int, [_i64, _i64, _i64] + [_vp] * 8),
    "b200_gblock_pack_rows": (_int, [_i64] * 6 + [_vp] * 4),
    "b200_gblock_fwd": (_int, [_i64] * 7 + [_vp] * 8),
    "b200_gblock_bwd_workspace_bytes": (_sz, [_i64] * 4),
    "b200_gblock_bwd": (_int, [_i64] * 7 + [_vp] * 7 + [_i64] + [_vp] * 4 + [_sz, _vp]),
    "b200_mamba_chk_interval": (_int, []),
    "b200_mamba_fwd": (_int, [_i64] * 4 + [_vp] * 12),
    "b200_mamba_bwd_workspace_bytes": (_sz, [_i64] * 4),
    "b200_mamba_bwd": (_int, [_i64] * 4 + [_vp] * 20 + [_sz, _vp]),
    "b200_proj_gemm_workspace_bytes": (_sz, [_i64] * 3),
    "b200_proj_gemm": (_int, [_i64, _i64, _i64, _vp, _i64, _vp, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _vp, _sz, _vp]),
    "b200_proj_wgrad_workspace_bytes": (_sz, [_i64] * 3),
    "b200_proj_wgrad": (_int, [_i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _sz, _vp]),
    "b200_layernorm_fwd": (_int, [_i64, _i64, _vp, _vp, _vp, ctypes.c_float, _vp, _vp, _vp, _vp]),
    "b200_layernorm_bwd_workspace_bytes": (_sz, [_i64, _i64]),
    "b200_layernorm_bwd": (_int, [_i64, _i64] + [_vp] * 9 + [_sz, _vp]),
    "b200_gated_residual_fwd": (_int, [_i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "b200_gated_residual_bwd": (_int, [_i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "b200_lru_prologue_fwd": (_int, [_i64, _i64] + [_vp] * 8),
    "b200_lru_prologue_bwd": (_int, [_i64, _i64] + [_vp] * 13),
    "b200_s5_discretize_fwd": (_int, [_i64, _i64, _int, _int, ctypes.c_float] + [_vp] * 8),
    "b200_s5_discretize_bwd": (_int, [_i64, _i64, _int, _int, ctypes.c_float] + [_vp] * 13),
    "b200_colsum_workspace_bytes": (_sz, [_i64, _i64]),
    "b200_colsum": (_int, [_i64, _i64, _vp, _i64, _vp, _vp, _sz, _vp]),
    "b200_conv_silu_fwd": (_int, [_i64] * 4 + [_vp, _i64, _i64] + [_vp] * 5),
    "b200_conv_silu_bwd_workspace_bytes": (_sz, [_i64] * 4),
    "b200_conv_silu_bwd": (_int, [_i64] * 4 + [_vp, _vp, _i64, _i64] + [_vp] * 8 + [_sz, _vp]),
}


def lib_path() -> Path:
    """Path of the library to load: ``$B200SCAN_LIB`` (an alternative build) or the in-tree one."""
    return Path(os.environ.get("B200SCAN_LIB", _DEFAULT))


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = lib_path()
        if not path.exists():
            raise RuntimeError(
                f"{path} not found: build the CUDA library first with `python -m tsfast_b200.build` "
                "(tsfast_b200 has no CPU or PyTorch fallback)"
            )
        handle = ctypes.CDLL(str(path))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _LIB = handle
    return _LIB


def check(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"{what} failed: {_ERRORS.get(status, f'status {status}')}")


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def dtype_tag(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.complex64:
        return C64
    raise TypeError(f"unsupported dtype {dt}: the scan kernels take float32 or complex64")


def workspace(nbytes: int, device) -> torch.Tensor:
    """Scratch for one call, from torch's caching allocator (legal under graph capture)."""
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def require_dense_cuda(**tensors) -> None:
    """The kernels index raw pointers: reject anything that is not a dense CUDA tensor."""
    for name, t in tensors.items():
        if t is None:
            continue
        if t.device.type != "cuda":
            raise TypeError(f"{name} must be a CUDA tensor, got {t.device}")
        if not t.is_contiguous():
            raise TypeError(f"{name} must be contiguous")


def workspace_status(ws: torch.Tensor) -> int:
    """Device-side status of the launch that used ``ws`` (synchronises the current stream)."""
    return int(lib().b200_workspace_status(ptr(ws), stream_ptr(ws.device)))
