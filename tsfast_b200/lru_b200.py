"""tsfast's LRU layer as ONE differentiable op on B200: input projection, diagonal scan, readout.

``LRU.forward`` (``architectures/lru.py:85-110``) is ``v = u W_in^T`` (complex), ``x = scan(lam, v)``,
``y = Re(x C^T) + u D^T``.  Run as three separate autograd nodes, the layer input ``u`` collects its
gradient from two places (the feed-through ``D`` and the input projection), i.e. two GEMMs and an
addition over ``[B*L, d]``.  As one op the adjoint computes it as a single two-product GEMM
``du = gy D + gv W_in`` and everything else (the readout's input gradient, the scan adjoint, the
three weight gradients) in a fixed order with no autograd bookkeeping in between:

    lru_layer(u, lam, W_in, C_ro, D, x0) -> (y [B, L, out], x_last [B, n])

with ``lam [n]`` complex64, ``W_in [2n, d]`` in interleaved (re, im) row order (``prologue_b200``),
``C_ro [out, 2n]`` the readout weight in (re, -im) column order and ``x0 [B, n]`` complex64 or None.
All GEMMs run on the tcgen05 kernels (``proj_b200``), the scan on ``diag_scan.cu``.  The full state
sequence is kept for the adjoint only (never returned), so a caller that carries the state forward
hands back ``x_last`` and its gradient enters the adjoint at the last step.
"""

from __future__ import annotations

import torch

from . import proj_b200
from .scan_backends import diagonal_b200

__all__ = ["lru_layer", "readout_weight"]


def readout_weight(C_re: torch.Tensor, C_im: torch.Tensor) -> torch.Tensor:
    """``[out, 2n]`` real weight with ``Re(x C^T) = view_as_real(x).flatten(-2) @ W^T``."""
    out, n = C_re.shape
    return torch.stack((C_re, -C_im), dim=-1).reshape(out, 2 * n)


def _check(u, lam, W_in, C_ro, D, x0):
    n = lam.numel()
    ok = (u.dim() == 3 and u.is_cuda and u.dtype == torch.float32 and lam.dtype == torch.complex64 and lam.dim() == 1
          and tuple(W_in.shape) == (2 * n, u.shape[-1]) and C_ro.dim() == 2 and C_ro.shape[1] == 2 * n
          and tuple(D.shape) == (C_ro.shape[0], u.shape[-1])
          and (x0 is None or (tuple(x0.shape) == (u.shape[0], n) and x0.dtype == torch.complex64)))
    if not ok:
        raise RuntimeError("b200scan::lru_layer: expected float32 CUDA u [B, L, d], lam [n] complex64, W_in [2n, d], "
                           f"C_ro [out, 2n], D [out, d], x0 [B, n] complex64 or None; got {tuple(u.shape)} {u.dtype}, "
                           f"{tuple(lam.shape)} {lam.dtype}, {tuple(W_in.shape)}, {tuple(C_ro.shape)}, {tuple(D.shape)}")


@torch.library.custom_op("b200scan::lru_layer", mutates_args=())
def _lru_op(u: torch.Tensor, lam: torch.Tensor, W_in: torch.Tensor, C_ro: torch.Tensor, D: torch.Tensor,
            x0: torch.Tensor | None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    _check(u, lam, W_in, C_ro, D, x0)
    B, L, d = u.shape
    n = lam.numel()
    u2 = proj_b200._rows(u)
    v = torch.view_as_complex(proj_b200._gemm(u2, W_in.contiguous()).contiguous().view(B, L, n, 2))
    x = diagonal_b200.forward(lam.expand(B, n).contiguous(), v, None if x0 is None else x0.contiguous())
    xr = proj_b200._rows(torch.view_as_real(x).view(B * L, 2 * n))  # in place unless n is odd (rows of 8n bytes)
    y = proj_b200._gemm(xr, C_ro.contiguous(), u2, D.contiguous())
    return y.reshape(B, L, D.shape[0]), x[:, -1, :].clone() if L > 0 else lam.new_zeros(B, n), x


@_lru_op.register_fake
def _(u, lam, W_in, C_ro, D, x0):
    B, L, _ = u.shape
    n = lam.numel()
    return u.new_empty(B, L, D.shape[0]), lam.new_empty(B, n), lam.new_empty(B, L, n)


@torch.library.custom_op("b200scan::lru_layer_bwd", mutates_args=())
def _lru_bwd_op(gy: torch.Tensor | None, gx_last: torch.Tensor | None, u: torch.Tensor, lam: torch.Tensor, W_in: torch.Tensor,
                C_ro: torch.Tensor, D: torch.Tensor, x0: torch.Tensor | None,
                x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    B, L, d = u.shape
    n = lam.numel()
    out = D.shape[0]
    u2 = proj_b200._rows(u)
    xr = proj_b200._rows(torch.view_as_real(x).view(B * L, 2 * n))
    # gy is None when only the carried state was used downstream
    gy2 = proj_b200._rows(u.new_zeros(B * L, out) if gy is None else gy)
    # readout: state gradient, weight gradients of C and D
    gx = torch.view_as_complex(proj_b200._gemm(gy2, C_ro.t().contiguous()).contiguous().view(B, L, n, 2))
    if gx_last is not None and L > 0:
        gx[:, -1, :] += gx_last
    gC = proj_b200._wgrad(gy2, xr)
    gD = proj_b200._wgrad(gy2, u2)
    # scan adjoint (the eigenvalue gradient comes per batch row: summed here)
    glam_rows, gv, gx0 = diagonal_b200.backward(gx, lam.expand(B, n).contiguous(), x, None if x0 is None else x0.contiguous())
    gvr = proj_b200._rows(torch.view_as_real(gv).view(B * L, 2 * n))
    gW = proj_b200._wgrad(gvr, u2)
    # the layer input collects feed-through and input projection in one two-product GEMM
    du = proj_b200._gemm(gy2, D.t().contiguous(), gvr, W_in.t().contiguous())
    return (du.reshape(B, L, d), glam_rows.sum(0), gW, gC, gD, gx0 if x0 is not None else lam.new_empty(0))


@_lru_bwd_op.register_fake
def _(gy, gx_last, u, lam, W_in, C_ro, D, x0, x):
    return (torch.empty_like(u), torch.empty_like(lam), torch.empty_like(W_in), torch.empty_like(C_ro), torch.empty_like(D),
            torch.empty_like(x0) if x0 is not None else lam.new_empty(0))


def _remember(ctx, inputs, output):
    u, lam, W_in, C_ro, D, x0 = inputs
    ctx.has_x0 = x0 is not None
    ctx.save_for_backward(u, lam, W_in, C_ro, D, *([x0] if x0 is not None else []), output[2])
    ctx.set_materialize_grads(False)


def _adjoint(ctx, gy, gx_last, _gx):
    saved = ctx.saved_tensors
    u, lam, W_in, C_ro, D = saved[:5]
    x0 = saved[5] if ctx.has_x0 else None
    x = saved[-1]
    du, glam, gW, gC, gD, gx0 = _lru_bwd_op(gy, gx_last, u, lam, W_in, C_ro, D, x0, x)
    return du, glam, gW, gC, gD, (gx0 if ctx.has_x0 else None)


_lru_op.register_autograd(_adjoint, setup_context=_remember)


def lru_layer(u, lam, W_in, C_ro, D, x0=None):
    """``(y [B, L, out], x_last [B, n])`` of the LRU layer; differentiable in every argument and in ``x_last``."""
    y, x_last, _x = _lru_op(u, lam, W_in, C_ro, D, x0)
    return y, x_last
