"""Diagonal linear recurrences on B200: the public functions and their custom ops.

Host-side mirror of the reference's ``tsfast/models/_core/scan.py``: the same two public
functions with the same argument meaning,

* ``diagonal_recurrence(lam, v, x0=None)``  – ``x_t = lam * x_{t-1} + v_t``, ``lam [..., n]``
  constant over time (reference ``scan.py:221-243``);
* ``selective_recurrence(lam, v, x0=None)`` – ``x_t = lam_t * x_{t-1} + v_t``, ``lam [..., L, n]``
  (reference ``scan.py:246-269``);

each a forward/backward pair of ``torch.library`` custom ops (namespace ``b200scan``, so they
can live beside the reference's ``tsfast::`` ops) with fake implementations and the analytic
reverse-scan adjoint registered for autograd.  Broadcasting is materialised outside the ops,
exactly as the reference does, so plain autograd folds lane gradients back onto broadcast
shapes.  Only ``(lam, out, x0)`` are saved for backward.  There is no fallback path: the ops
call the CUDA library and raise if it is missing or the tensors are not float32/complex64 CUDA.
"""

from __future__ import annotations

import torch

from .scan_backends import diagonal_b200, selective_b200

__all__ = ["diagonal_recurrence", "selective_recurrence"]


def _dense(*ts):
    return [None if t is None else t.contiguous() for t in ts]


def _require(mod, lam, v, x0, name):
    reason = mod.supports(lam, v, x0)
    if reason is not None:
        raise RuntimeError(f"b200scan::{name}: {reason}")


# ------------------------------------------------------------------------- S1 ops
@torch.library.custom_op("b200scan::scan_diagonal", mutates_args=())
def _scan_diagonal_op(lam: torch.Tensor, v: torch.Tensor, x0: torch.Tensor | None) -> torch.Tensor:
    lam, v, x0 = _dense(lam, v, x0)
    _require(diagonal_b200, lam, v, x0, "scan_diagonal")
    return diagonal_b200.forward(lam, v, x0)


@_scan_diagonal_op.register_fake
def _(lam, v, x0):
    return torch.empty_like(v)


@torch.library.custom_op("b200scan::scan_diagonal_bwd", mutates_args=())
def _scan_diagonal_bwd_op(
    g: torch.Tensor, lam: torch.Tensor, out: torch.Tensor, x0: torch.Tensor | None
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    g, lam, out, x0 = _dense(g, lam, out, x0)
    _require(diagonal_b200, lam, g, x0, "scan_diagonal_bwd")
    return diagonal_b200.backward(g, lam, out, x0)


@_scan_diagonal_bwd_op.register_fake
def _(g, lam, out, x0):
    gx0 = torch.empty_like(lam) if x0 is not None else lam.new_empty(0)
    return torch.empty_like(lam), torch.empty_like(g), gx0


def _diag_setup(ctx, inputs, output):
    lam, v, x0 = inputs
    ctx.save_for_backward(lam, output, x0)


def _diag_backward(ctx, g):
    lam, out, x0 = ctx.saved_tensors
    glam, gv, gx0 = _scan_diagonal_bwd_op(g, lam, out, x0)
    return glam, gv, (gx0 if x0 is not None else None)


_scan_diagonal_op.register_autograd(_diag_backward, setup_context=_diag_setup)


# ------------------------------------------------------------------------- S2 ops
@torch.library.custom_op("b200scan::scan_selective", mutates_args=())
def _scan_selective_op(lam: torch.Tensor, v: torch.Tensor, x0: torch.Tensor | None) -> torch.Tensor:
    lam, v, x0 = _dense(lam, v, x0)
    _require(selective_b200, lam, v, x0, "scan_selective")
    return selective_b200.forward(lam, v, x0)


@_scan_selective_op.register_fake
def _(lam, v, x0):
    return torch.empty_like(v)


@torch.library.custom_op("b200scan::scan_selective_bwd", mutates_args=())
def _scan_selective_bwd_op(
    g: torch.Tensor, lam: torch.Tensor, out: torch.Tensor, x0: torch.Tensor | None
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    g, lam, out, x0 = _dense(g, lam, out, x0)
    _require(selective_b200, lam, g, x0, "scan_selective_bwd")
    return selective_b200.backward(g, lam, out, x0)


@_scan_selective_bwd_op.register_fake
def _(g, lam, out, x0):
    gx0 = torch.empty_like(lam[..., 0, :]) if x0 is not None else lam.new_empty(0)
    return torch.empty_like(lam), torch.empty_like(g), gx0


def _sel_setup(ctx, inputs, output):
    lam, v, x0 = inputs
    ctx.save_for_backward(lam, output, x0)


def _sel_backward(ctx, g):
    lam, out, x0 = ctx.saved_tensors
    glam, gv, gx0 = _scan_selective_bwd_op(g, lam, out, x0)
    return glam, gv, (gx0 if x0 is not None else None)


_scan_selective_op.register_autograd(_sel_backward, setup_context=_sel_setup)


# ------------------------------------------------------------------------- public API
def diagonal_recurrence(lam: torch.Tensor, v: torch.Tensor, x0: torch.Tensor | None = None) -> torch.Tensor:
    """``x_t = lam * x_{t-1} + v_t`` with constant diagonal ``lam``; returns ``x_1..x_L``.

    Args:
        lam: diagonal coefficients ``[..., n]``, broadcast against the leading dims of ``v``.
        v: input sequence ``[..., L, n]`` (float32 or complex64, CUDA).
        x0: initial state ``[..., n]``; zeros if None.
    """
    out_shape = torch.broadcast_shapes(lam.unsqueeze(-2).shape, v.shape)
    bdims, L, n = out_shape[:-2], out_shape[-2], out_shape[-1]
    lam_lane = lam.broadcast_to(bdims + (n,)).reshape(-1, n)
    v_flat = v.broadcast_to(out_shape).reshape(-1, L, n)
    x0_lane = None if x0 is None else x0.broadcast_to(bdims + (n,)).reshape(-1, n)
    return _scan_diagonal_op(lam_lane, v_flat, x0_lane).reshape(out_shape)


def selective_recurrence(lam: torch.Tensor, v: torch.Tensor, x0: torch.Tensor | None = None) -> torch.Tensor:
    """``x_t = lam_t * x_{t-1} + v_t`` with time-varying diagonal ``lam_t``; returns ``x_1..x_L``.

    Args:
        lam: coefficients per step ``[..., L, n]``, broadcast against ``v``.
        v: input sequence ``[..., L, n]`` (float32 or complex64, CUDA).
        x0: initial state ``[..., n]``; zeros if None.
    """
    out_shape = torch.broadcast_shapes(lam.shape, v.shape)
    bdims, L, n = out_shape[:-2], out_shape[-2], out_shape[-1]
    lam3 = lam.broadcast_to(out_shape).reshape(-1, L, n)
    v3 = v.broadcast_to(out_shape).reshape(-1, L, n)
    x03 = None if x0 is None else x0.broadcast_to(bdims + (n,)).reshape(-1, n)
    return _scan_selective_op(lam3, v3, x03).reshape(out_shape)
