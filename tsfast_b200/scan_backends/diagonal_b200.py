"""B200 backend of the constant-coefficient diagonal scan ``x_t = lam * x_{t-1} + v_t``.

Drop-in for the reference's ``scan_backends/diagonal_triton.py`` / ``diagonal_c.py`` modules:
same ``supports`` / ``forward`` / ``backward`` protocol on the lane layout (``lam [M,N]``,
``v [M,L,N]``, ``x0 [M,N] | None``, all contiguous, float32 or complex64).  The work is done by
``b200_diag_fwd`` / ``b200_diag_bwd`` of ``libb200scan.so`` on the current CUDA stream.
"""

from __future__ import annotations

import torch

from . import _common

__all__ = ["supports", "forward", "backward"]


def supports(lam: torch.Tensor, v: torch.Tensor, x0: torch.Tensor | None) -> str | None:
    """Reason these tensors cannot be handled, or None when they can."""
    return _common._supports(lam, v, x0, varying=False)


def forward(lam: torch.Tensor, v: torch.Tensor, x0: torch.Tensor | None) -> torch.Tensor:
    """States ``x_1..x_L`` as ``[M, L, N]``."""
    return _common.run_forward("diag", lam, v, x0)


def backward(g, lam, out, x0):
    """Adjoint sweep → ``(glam [M,N], gv [M,L,N], gx0 [M,N])``; ``gx0`` is empty when ``x0 is None``."""
    return _common.run_backward("diag", g, lam, out, x0)
