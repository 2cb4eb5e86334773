"""Host-side mirror of tsfast's LRU caller stack, running its recurrence on the B200 scan.

tsfast's ``LRU`` / ``LRUBlock`` / ``DeepLRU`` (``tsfast/models/architectures/lru.py:16-234``) are the
modules that call ``diagonal_recurrence``.  With tsfast importable they are used unchanged after
``tsfast_b200.install()``.  This file exists for machines where tsfast is not installed (the
benchmark's full-model configuration and its tests): the same layer stack with the same parameter
names and shapes, so a tsfast ``DeepLRU.state_dict()`` loads into ``DeepLRU`` here and both
produce the same numbers, but with the recurrence hard-wired to
``tsfast_b200.diagonal_recurrence`` (no backend switch, no CPU path).

Layer maths (Orvieto et al. 2023; tsfast ``lru.py:79-110``, ``_core/scan.py:272-313``):
``lam = exp(-exp(nu_log) + i exp(theta_log))``; ``v_k = exp(gamma_log) * (B u_k)`` with complex
``B = B_re + i B_im``; ``x_k = lam x_{k-1} + v_k``; ``y_k = Re(C x_k) + D u_k``.  The two boundary
projections are single real GEMMs against interleaved weights, so the complex views are free.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from .scan import diagonal_recurrence

__all__ = ["LRU", "LRUBlock", "DeepLRU", "project_in", "project_out"]


def project_in(u: torch.Tensor, w_re: torch.Tensor, w_im: torch.Tensor) -> torch.Tensor:
    """Real ``u [..., d]`` times complex ``(w_re + i w_im) [n, d]`` → complex ``[..., n]``, one real GEMM.

    The weight is laid out ``[d, n, 2]`` so the GEMM result already has ``view_as_complex``'s
    memory layout (mirrors ``complex_in_proj``, tsfast ``_core/scan.py:272-292``).
    """
    n, d = w_re.shape
    packed = torch.stack((w_re.t(), w_im.t()), dim=-1).reshape(d, 2 * n)
    return torch.view_as_complex((u @ packed).unflatten(-1, (n, 2)))


def project_out(x: torch.Tensor, w_re: torch.Tensor, w_im: torch.Tensor) -> torch.Tensor:
    """``Re(x (w_re + i w_im)^T)`` for complex ``x [..., n]`` → real ``[..., out]``, one real GEMM
    (mirrors ``real_out_proj``, tsfast ``_core/scan.py:295-313``)."""
    out, n = w_re.shape
    packed = torch.stack((w_re, w_im.neg()), dim=-1).reshape(out, 2 * n)
    return torch.view_as_real(x).flatten(-2) @ packed.t()


class LRU(nn.Module):
    """One diagonal complex linear state-space layer with full real feedthrough ``D``."""

    def __init__(self, in_features: int, out_features: int, state_features: int, r_min: float = 0.0,
                 r_max: float = 1.0, max_phase: float = 6.283):
        super().__init__()
        n, h = state_features, in_features
        ring = torch.rand(n) * (r_max**2 - r_min**2) + r_min**2  # |lam|^2 uniform on the ring
        self.nu_log = nn.Parameter(torch.log(-0.5 * torch.log(ring)))
        self.theta_log = nn.Parameter(torch.log(max_phase * torch.rand(n)))
        mag = torch.exp(-torch.exp(self.nu_log.detach()))
        self.gamma_log = nn.Parameter(0.5 * torch.log1p(-mag.square()))
        self.B_re = nn.Parameter(torch.randn(n, h) / math.sqrt(2 * h))
        self.B_im = nn.Parameter(torch.randn(n, h) / math.sqrt(2 * h))
        self.C_re = nn.Parameter(torch.randn(out_features, n) / math.sqrt(n))
        self.C_im = nn.Parameter(torch.randn(out_features, n) / math.sqrt(n))
        self.D = nn.Parameter(torch.randn(out_features, h) / math.sqrt(h))

    def eigenvalues(self) -> torch.Tensor:
        return torch.polar(torch.exp(-torch.exp(self.nu_log)), torch.exp(self.theta_log))

    def forward(self, u: torch.Tensor, state: torch.Tensor | None = None):
        """``u [batch, seq, in]`` → ``(y [batch, seq, out], last state [batch, n] complex)``."""
        scale = torch.exp(self.gamma_log).unsqueeze(-1)
        v = project_in(u, scale * self.B_re, scale * self.B_im)
        x = diagonal_recurrence(self.eigenvalues(), v, state)
        y = project_out(x, self.C_re, self.C_im) + u @ self.D.t()
        return y, x[..., -1, :]


class LRUBlock(nn.Module):
    """Pre-norm residual block ``u + GLU(gelu(LRU(LayerNorm(u))))`` (tsfast ``lru.py:113-152``)."""

    def __init__(self, d_model: int, d_state: int, dropout: float = 0.0, **lru_kwargs):
        super().__init__()
        self.norm = nn.LayerNorm(d_model)
        self.lru = LRU(d_model, d_model, d_state, **lru_kwargs)
        self.glu = nn.Linear(d_model, 2 * d_model)
        self.dropout = nn.Dropout(dropout)

    def forward(self, u: torch.Tensor, state: torch.Tensor | None = None):
        h, new_state = self.lru(self.norm(u), state)
        h = self.dropout(F.gelu(h))
        h = self.dropout(F.glu(self.glu(h), dim=-1))
        return u + h, new_state


class DeepLRU(nn.Module):
    """Linear encoder, ``n_layers`` LRU blocks, linear decoder (tsfast ``lru.py:155-234``).

    ``forward(u, state=None)`` returns the output sequence, or ``(output, [state per block])`` when
    ``return_state`` is set; feeding the returned states back continues the sequence exactly
    (truncated back-propagation through time).
    """

    def __init__(self, input_size: int, output_size: int, d_model: int = 32, d_state: int = 64, n_layers: int = 3,
                 dropout: float = 0.0, return_state: bool = False, **lru_kwargs):
        super().__init__()
        self.return_state = return_state
        self.encoder = nn.Linear(input_size, d_model)
        self.blocks = nn.ModuleList(LRUBlock(d_model, d_state, dropout, **lru_kwargs) for _ in range(n_layers))
        self.decoder = nn.Linear(d_model, output_size)

    def forward(self, u: torch.Tensor, state: list | None = None):
        states = state if state is not None else [None] * len(self.blocks)
        h = self.encoder(u)
        carried = []
        for block, s in zip(self.blocks, states):
            h, s_new = block(h, s)
            carried.append(s_new)
        y = self.decoder(h)
        return (y, carried) if self.return_state else y
