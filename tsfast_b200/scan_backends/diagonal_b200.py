"""B200 backend of the constant-coefficient diagonal scan ``x_t = lam * x_{t-1} + v_t``.

Drop-in for the reference's ``scan_backends/diagonal_triton.py`` / ``diagonal_c.py`` modules:
same ``supports`` / ``forward`` / ``backward`` protocol on the lane layout (``lam [M,N]``,
``v [M,L,N]``, ``x0 [M,N] | None``, all contiguous, float32 or complex64).  The work is done by
``b200_diag_fwd`` / ``b200_diag_bwd`` of ``libb200scan.so`` on the current CUDA stream.
"""

from __future__ import annotations

from ._common import DIAGONAL as _scan

__all__ = ["supports", "forward", "backward", "calls"]

calls = 0  # launches through this module since import (the drop-in tests read it)


def supports(lam, v, x0):
    """Reason these tensors cannot be handled, or None when they can."""
    return _scan.why_not(lam, v, x0)


def forward(lam, v, x0):
    """States ``x_1..x_L`` as ``[M, L, N]``."""
    global calls
    calls += 1
    return _scan.forward(lam, v, x0)


def backward(g, lam, out, x0):
    """Adjoint sweep → ``(glam [M,N], gv [M,L,N], gx0 [M,N])``; ``gx0`` is empty when ``x0 is None``."""
    global calls
    calls += 1
    return _scan.backward(g, lam, out, x0)
