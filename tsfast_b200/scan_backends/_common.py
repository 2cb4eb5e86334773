"""Shared launch plumbing of the two diagonal-scan backends."""

from __future__ import annotations

import torch

from .. import _lib

# Workspace of the most recent launch per op, kept so tests can read the device status word.
LAST_WS: dict[str, torch.Tensor] = {}


def _supports(lam, v, x0, varying: bool) -> str | None:
    if not torch.cuda.is_available():
        return "CUDA not available"
    if v.device.type != "cuda" or lam.device.type != "cuda":
        return "inputs not on CUDA"
    if v.dtype not in (torch.float32, torch.complex64):
        return f"dtype {v.dtype} unsupported (need float32 or complex64)"
    if lam.dtype != v.dtype:
        return f"lam dtype {lam.dtype} != v dtype {v.dtype}"
    if x0 is not None and (x0.dtype != v.dtype or x0.device != v.device):
        return f"x0 must match v in dtype and device, got {x0.dtype} on {x0.device}"
    if v.dim() != 3:
        return f"v must be [rows, L, n] on the lane layout, got {v.dim()} dims"
    M, L, N = v.shape
    if varying:
        if lam.shape != v.shape:
            return f"lam.shape {tuple(lam.shape)} != v.shape {tuple(v.shape)}"
    elif tuple(lam.shape) != (M, N):
        return f"lam.shape {tuple(lam.shape)} != {(M, N)}"
    if x0 is not None and tuple(x0.shape) != (M, N):
        return f"x0.shape {tuple(x0.shape)} != {(M, N)}"
    return None


def run_forward(op: str, lam, v, x0):
    L_ = _lib.lib()
    _lib.require_dense_cuda(lam=lam, v=v, x0=x0)
    M, L, N = v.shape
    tag = _lib.dtype_tag(v.dtype)
    out = torch.empty_like(v)
    if out.numel() == 0:
        return out
    ws = _lib.workspace(getattr(L_, f"b200_{op}_workspace_bytes")(tag, 0, M, L, N), v.device)
    st = getattr(L_, f"b200_{op}_fwd")(tag, M, L, N, _lib.ptr(lam), _lib.ptr(v), _lib.ptr(x0), _lib.ptr(out),
                                        _lib.ptr(ws), ws.numel(), _lib.stream_ptr(v.device))
    _lib.check(st, f"b200_{op}_fwd")
    LAST_WS[op] = ws
    return out


def run_backward(op: str, g, lam, out, x0):
    L_ = _lib.lib()
    _lib.require_dense_cuda(g=g, lam=lam, out=out, x0=x0)
    M, L, N = out.shape
    tag = _lib.dtype_tag(out.dtype)
    glam = torch.empty_like(lam)
    gv = torch.empty_like(out)
    gx0 = torch.empty_like(x0) if x0 is not None else None
    if out.numel() == 0:
        glam.zero_()
        if gx0 is not None:
            gx0.zero_()
        return glam, gv, (gx0 if gx0 is not None else lam.new_empty(0))
    ws = _lib.workspace(getattr(L_, f"b200_{op}_workspace_bytes")(tag, 1, M, L, N), out.device)
    st = getattr(L_, f"b200_{op}_bwd")(tag, M, L, N, _lib.ptr(g), _lib.ptr(lam), _lib.ptr(out), _lib.ptr(x0),
                                        _lib.ptr(glam), _lib.ptr(gv), _lib.ptr(gx0), _lib.ptr(ws), ws.numel(),
                                        _lib.stream_ptr(out.device))
    _lib.check(st, f"b200_{op}_bwd")
    LAST_WS[op] = ws
    return glam, gv, (gx0 if gx0 is not None else lam.new_empty(0))
