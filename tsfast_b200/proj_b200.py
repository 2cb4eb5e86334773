"""Boundary projections of the diagonal-scan layers on B200's tensor cores.

tsfast's LRU and S5 layers enter and leave complex state space through two real GEMMs
(``complex_in_proj`` / ``real_out_proj``, ``tsfast/models/_core/scan.py:272-313``); with the scans at
HBM speed these GEMMs, run as float32 SIMT kernels, are most of a training step.  This module offers
the same two functions (same arguments, same results, differentiable) on ``b200_proj_gemm``:
``tcgen05`` TF32 MMAs fed by TMA with every operand split into a TF32 head and a float32 tail, so the
result is float32-faithful (TF32 stays "off" in the sense of tsfast's tests: no precision is traded).

* ``linear_nt(a, w)``      – ``a [..., K] @ w [N, K]^T`` with autograd (input gradient on the same
  kernel; the weight gradient, a reduction over all tokens into a small matrix, through cuBLAS);
* ``complex_in_proj(u, W_re, W_im)`` / ``real_out_proj(x, W_re, W_im)`` – drop-ins for tsfast's;
* ``supports(a, w)``       – reason the kernel cannot take these tensors, or None.

``tsfast_b200.install(fuse_projections=True)`` points tsfast's LRU and S5 modules at them.
"""

from __future__ import annotations

import torch

from . import _lib

__all__ = ["linear_nt", "complex_in_proj", "real_out_proj", "supports", "calls"]

calls = 0  # launches through this module since import (the drop-in tests read it)
_BLOCK_K = 32


def supports(a: torch.Tensor, w: torch.Tensor) -> str | None:
    """Reason ``linear_nt(a, w)`` cannot run on the tensor-core kernel, or None when it can."""
    if not torch.cuda.is_available():
        return "no CUDA device is visible to this process"
    if a.device.type != "cuda" or w.device.type != "cuda":
        return "the kernels only read CUDA memory"
    if a.dtype != torch.float32 or w.dtype != torch.float32:
        return f"needs float32 operands, got {a.dtype} and {w.dtype}"
    if w.dim() != 2 or a.dim() < 1 or a.shape[-1] != w.shape[1]:
        return f"shapes {tuple(a.shape)} and {tuple(w.shape)} do not form a [..., K] x [N, K]^T product"
    if w.shape[1] % _BLOCK_K != 0:
        return f"the reduction width {w.shape[1]} is not a multiple of {_BLOCK_K}"
    return None


def _rows(a: torch.Tensor) -> torch.Tensor:
    """``a`` as a 2-D matrix the kernel can read: unit column stride, row pitch a multiple of 4 floats,
    16-byte aligned (a dense copy only when the view does not already qualify)."""
    a2 = a.reshape(-1, a.shape[-1])
    ok = a2.stride(1) == 1 and a2.stride(0) % 4 == 0 and a2.stride(0) >= a2.shape[1] and a2.data_ptr() % 16 == 0
    return a2 if ok else a2.clone(memory_format=torch.contiguous_format)


def _launch(a1, b1, a2=None, b2=None):
    global calls
    L_ = _lib.lib()
    m, k1 = a1.shape
    n = b1.shape[0]
    k2 = 0 if a2 is None else a2.shape[1]
    out = torch.empty(m, n, device=a1.device, dtype=torch.float32)
    if m == 0:
        return out
    ws = _lib.workspace(L_.b200_proj_gemm_workspace_bytes(n, k1, k2), a1.device)
    calls += 1
    rc = L_.b200_proj_gemm(m, n, k1, _lib.ptr(a1), a1.stride(0), _lib.ptr(b1), b1.stride(0), k2, _lib.ptr(a2),
                           0 if a2 is None else a2.stride(0), _lib.ptr(b2), 0 if b2 is None else b2.stride(0),
                           _lib.ptr(out), out.stride(0), _lib.ptr(ws), ws.numel(), _lib.stream_ptr(a1.device))
    _lib.check(rc, "b200_proj_gemm")
    return out


@torch.library.custom_op("b200scan::proj_gemm", mutates_args=())
def _proj_gemm_op(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``a [M, K] @ w [N, K]^T`` -> ``[M, N]``."""
    why = supports(a, w)
    if why is not None:
        raise RuntimeError(f"b200scan::proj_gemm: {why}")
    return _launch(_rows(a), w.contiguous())


@_proj_gemm_op.register_fake
def _(a, w):
    return a.new_empty(a.shape[0], w.shape[0])


@torch.library.custom_op("b200scan::proj_gemm2", mutates_args=())
def _proj_gemm2_op(a1: torch.Tensor, w1: torch.Tensor, a2: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """``a1 @ w1^T + a2 @ w2^T`` in one pass over the output (readout plus feed-through)."""
    for a, w in ((a1, w1), (a2, w2)):
        why = supports(a, w)
        if why is not None:
            raise RuntimeError(f"b200scan::proj_gemm2: {why}")
    if a1.shape[0] != a2.shape[0] or w1.shape[0] != w2.shape[0]:
        raise RuntimeError("b200scan::proj_gemm2: the two products must have the same output shape")
    return _launch(_rows(a1), w1.contiguous(), _rows(a2), w2.contiguous())


@_proj_gemm2_op.register_fake
def _(a1, w1, a2, w2):
    return a1.new_empty(a1.shape[0], w1.shape[0])


def _input_grad(g: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``g [M, N] @ w [N, K]`` on the kernel when N (now the reduction) allows, else through cuBLAS."""
    wt = w.t().contiguous()  # [K, N]: rows are the output features of this product
    return _proj_gemm_op(g, wt) if supports(g, wt) is None else g @ w


def _remember(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _adjoint(ctx, g):
    a, w = ctx.saved_tensors
    g = g.contiguous()
    ga = _input_grad(g, w) if ctx.needs_input_grad[0] else None
    gw = g.t() @ a if ctx.needs_input_grad[1] else None  # [N, K]: reduction over all tokens
    return ga, gw


def _adjoint2(ctx, g):
    a1, w1, a2, w2 = ctx.saved_tensors
    g = g.contiguous()
    need = ctx.needs_input_grad
    return (_input_grad(g, w1) if need[0] else None, g.t() @ a1 if need[1] else None,
            _input_grad(g, w2) if need[2] else None, g.t() @ a2 if need[3] else None)


_proj_gemm_op.register_autograd(_adjoint, setup_context=_remember)
_proj_gemm2_op.register_autograd(_adjoint2, setup_context=_remember)


def linear_nt(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``a [..., K] @ w [N, K]^T`` -> ``[..., N]`` (float32 CUDA, ``K`` a multiple of 32)."""
    return _proj_gemm_op(a.reshape(-1, a.shape[-1]), w).reshape(*a.shape[:-1], w.shape[0])


def complex_in_proj(u: torch.Tensor, W_re: torch.Tensor, W_im: torch.Tensor) -> torch.Tensor:
    """``u @ (W_re + i W_im)^T`` for real ``u [..., d]`` and ``W [n, d]`` -> complex ``[..., n]``.

    The weight rows are interleaved (re, im) so that the real GEMM result already has
    ``view_as_complex``'s memory layout, as in tsfast's function of the same name."""
    n, d = W_re.shape
    w = torch.stack((W_re, W_im), dim=1).reshape(2 * n, d)
    return torch.view_as_complex(linear_nt(u, w).unflatten(-1, (n, 2)))


def real_out_proj(x: torch.Tensor, W_re: torch.Tensor, W_im: torch.Tensor) -> torch.Tensor:
    """``Re(x @ (W_re + i W_im)^T)`` for complex ``x [..., n]`` and ``W [out, n]`` -> real ``[..., out]``."""
    out, n = W_re.shape
    w = torch.stack((W_re, -W_im), dim=-1).reshape(out, 2 * n)
    return linear_nt(torch.view_as_real(x).flatten(-2), w)
