"""Diagonal linear recurrences on B200: the public functions and their custom ops.

Host-side mirror of the reference's ``tsfast/models/_core/scan.py``: the same two public
functions with the same argument meaning,

* ``diagonal_recurrence(lam, v, x0=None)``  – ``x_t = lam * x_{t-1} + v_t``, ``lam [..., n]``
  constant over time (reference ``scan.py:221-243``);
* ``selective_recurrence(lam, v, x0=None)`` – ``x_t = lam_t * x_{t-1} + v_t``, ``lam [..., L, n]``
  (reference ``scan.py:246-269``);

each a forward/backward pair of ``torch.library`` custom ops (namespace ``b200scan``, so they
can live beside the reference's ``tsfast::`` ops) with fake implementations and the analytic
reverse-scan adjoint registered for autograd.  Both functions and all four ops are generated from
one description of a scan (``_Kind``); broadcasting is spread onto the lane layout outside the ops
(``_on_lanes``), so plain autograd folds lane gradients back onto broadcast shapes.  Only
``(lam, out, x0)`` are saved for backward, as the interface prescribes.  There is no fallback path:
the ops call the CUDA library and raise if it is missing or the tensors are not float32/complex64
CUDA tensors.
"""

from __future__ import annotations

import torch

from . import _spec
from .scan_backends import _common

__all__ = ["diagonal_recurrence", "selective_recurrence"]


class _Kind:
    """One diagonal scan: its launcher and whether the coefficient carries a time axis."""

    def __init__(self, name: str, launcher: _common.Scan, per_step: bool):
        self.name, self.launcher, self.per_step = name, launcher, per_step

    def guard(self, lam, v, x0, suffix=""):
        why = self.launcher.why_not(lam, v, x0)
        if why is not None:
            raise RuntimeError(f"b200scan::{self.name}{suffix}: {why}")

    def state_like(self, lam):
        """An empty tensor shaped like one state ``[rows, n]`` of this scan."""
        return torch.empty_like(lam[:, 0] if self.per_step else lam)

    def build(self):
        kind = self

        @torch.library.custom_op(f"b200scan::{kind.name}", mutates_args=())
        def fwd(lam: torch.Tensor, v: torch.Tensor, x0: torch.Tensor | None) -> torch.Tensor:
            lam, v, x0 = _spec.dense(lam, v, x0)
            kind.guard(lam, v, x0)
            return kind.launcher.forward(lam, v, x0)

        @fwd.register_fake
        def _(lam, v, x0):
            return torch.empty_like(v)

        @torch.library.custom_op(f"b200scan::{kind.name}_bwd", mutates_args=())
        def bwd(g: torch.Tensor, lam: torch.Tensor, out: torch.Tensor,
                x0: torch.Tensor | None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
            g, lam, out, x0 = _spec.dense(g, lam, out, x0)
            kind.guard(lam, g, x0, "_bwd")
            return kind.launcher.backward(g, lam, out, x0)

        @bwd.register_fake
        def _(g, lam, out, x0):
            return torch.empty_like(lam), torch.empty_like(g), (lam.new_empty(0) if x0 is None else kind.state_like(lam))

        def remember(ctx, inputs, output):
            lam, _, x0 = inputs
            ctx.save_for_backward(lam, output, x0)

        def adjoint(ctx, g):
            lam, out, x0 = ctx.saved_tensors
            glam, gv, gx0 = bwd(g, lam, out, x0)
            return glam, gv, (None if x0 is None else gx0)

        fwd.register_autograd(adjoint, setup_context=remember)
        return fwd, bwd


_DIAG = _Kind("scan_diagonal", _common.DIAGONAL, per_step=False)
_SEL = _Kind("scan_selective", _common.SELECTIVE, per_step=True)
_scan_diagonal_op, _scan_diagonal_bwd_op = _DIAG.build()
_scan_selective_op, _scan_selective_bwd_op = _SEL.build()


def _on_lanes(kind: _Kind, lam, v, x0):
    """Spread ``lam``, ``v``, ``x0`` over their common leading dims and flatten those to rows."""
    coef_shape = tuple(lam.shape) if kind.per_step else tuple(lam.shape[:-1]) + (1, lam.shape[-1])
    full = torch.broadcast_shapes(coef_shape, v.shape)
    lead, steps, n = tuple(full[:-2]), full[-2], full[-1]
    rows_v = v.expand(full).reshape(-1, steps, n)
    if kind.per_step:
        rows_lam = lam.expand(full).reshape(-1, steps, n)
    else:
        rows_lam = lam.expand(lead + (n,)).reshape(-1, n)
    rows_x0 = None if x0 is None else x0.expand(lead + (n,)).reshape(-1, n)
    return rows_lam, rows_v, rows_x0, full


def diagonal_recurrence(lam: torch.Tensor, v: torch.Tensor, x0: torch.Tensor | None = None) -> torch.Tensor:
    """``x_t = lam * x_{t-1} + v_t`` with constant diagonal ``lam``; returns ``x_1..x_L``.

    Args:
        lam: diagonal coefficients ``[..., n]``, broadcast against the leading dims of ``v``.
        v: input sequence ``[..., L, n]`` (float32 or complex64, CUDA).
        x0: initial state ``[..., n]``; zeros if None.
    """
    rows_lam, rows_v, rows_x0, full = _on_lanes(_DIAG, lam, v, x0)
    return _scan_diagonal_op(rows_lam, rows_v, rows_x0).reshape(full)


def selective_recurrence(lam: torch.Tensor, v: torch.Tensor, x0: torch.Tensor | None = None) -> torch.Tensor:
    """``x_t = lam_t * x_{t-1} + v_t`` with time-varying diagonal ``lam_t``; returns ``x_1..x_L``.

    Args:
        lam: coefficients per step ``[..., L, n]``, broadcast against ``v``.
        v: input sequence ``[..., L, n]`` (float32 or complex64, CUDA).
        x0: initial state ``[..., n]``; zeros if None.
    """
    rows_lam, rows_v, rows_x0, full = _on_lanes(_SEL, lam, v, x0)
    return _scan_selective_op(rows_lam, rows_v, rows_x0).reshape(full)
