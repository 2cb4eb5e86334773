"""B200 backend of the time-varying diagonal scan ``x_t = lam_t * x_{t-1} + v_t``.

Drop-in for the reference's ``scan_backends/selective_triton.py`` / ``selective_c.py`` modules:
same ``supports`` / ``forward`` / ``backward`` protocol on the lane layout (``lam``, ``v``
``[B,L,N]``, ``x0 [B,N] | None``, contiguous).  Unlike the reference's CUDA kernel (float32 only)
this one also takes complex64.  Entry points: ``b200_sel_fwd`` / ``b200_sel_bwd``.
"""

from __future__ import annotations

from ._common import SELECTIVE as _scan

__all__ = ["supports", "forward", "backward", "calls"]

calls = 0  # launches through this module since import (the drop-in tests read it)


def supports(lam, v, x0):
    """Reason these tensors cannot be handled, or None when they can."""
    return _scan.why_not(lam, v, x0)


def forward(lam, v, x0):
    """States ``x_1..x_L`` as ``[B, L, N]``."""
    global calls
    calls += 1
    return _scan.forward(lam, v, x0)


def backward(g, lam, out, x0):
    """Adjoint sweep → ``(glam [B,L,N], gv [B,L,N], gx0 [B,N])``; ``gx0`` is empty when ``x0 is None``."""
    global calls
    calls += 1
    return _scan.backward(g, lam, out, x0)
