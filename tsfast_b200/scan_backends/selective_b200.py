"""B200 backend of the time-varying diagonal scan ``x_t = lam_t * x_{t-1} + v_t``.

Drop-in for the reference's ``scan_backends/selective_triton.py`` / ``selective_c.py`` modules
(``lam, v [B,L,N]``, ``x0 [B,N] | None``, contiguous).  Unlike those it also takes complex64,
with the conjugation rules of the reference's doubling scan (``_core/scan.py:173-195``).
"""

from __future__ import annotations

import torch

from . import _common

__all__ = ["supports", "forward", "backward"]


def supports(lam: torch.Tensor, v: torch.Tensor, x0: torch.Tensor | None) -> str | None:
    """Reason these tensors cannot be handled, or None when they can."""
    return _common._supports(lam, v, x0, varying=True)


def forward(lam: torch.Tensor, v: torch.Tensor, x0: torch.Tensor | None) -> torch.Tensor:
    """States ``x_1..x_L`` as ``[B, L, N]``."""
    return _common.run_forward("sel", lam, v, x0)


def backward(g, lam, out, x0):
    """Adjoint sweep → ``(glam [B,L,N], gv [B,L,N], gx0 [B,N])``; ``gx0`` is empty when ``x0 is None``."""
    return _common.run_backward("sel", g, lam, out, x0)
