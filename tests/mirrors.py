"""TEST HELPERS: small stand-ins for tsfast's caller modules, for machines without a tsfast copy.

The drop-in is shown with tsfast's own modules (``test_dropin_gpu.py``).  These mirrors exist so the
golden fixtures taken from tsfast's ``DeepLRU``, ``LinearDynamicalOperator`` and ``DynoNet`` can also be
replayed where tsfast is not importable: the same layer stacks with the same parameter names and
shapes (a tsfast ``state_dict`` loads unchanged) with the recurrences hard-wired to this package's
ops.  They are not part of the product.

Layer maths of the LRU mirror (Orvieto et al. 2023; tsfast ``lru.py:79-110``, ``_core/scan.py:272-313``):
``lam = exp(-exp(nu_log) + i exp(theta_log))``; ``v_k = exp(gamma_log) * (B u_k)`` with complex
``B = B_re + i B_im``; ``x_k = lam x_{k-1} + v_k``; ``y_k = Re(C x_k) + D u_k``.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from tsfast_b200.dynonet_b200 import _MAX_NA, _NB_SIZES, linear_block
from tsfast_b200.scan import diagonal_recurrence


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


class LinearDynamicalOperator(nn.Module):
    """MIMO bank of rational transfer functions ``B(q)/A(q)``, one SISO filter per (output, input)
    pair, outputs summed over inputs: the mirror of tsfast's module of the same name
    (``dynonet/core.py:144-254``) with the whole forward in one kernel."""

    def __init__(self, in_channels: int, out_channels: int, nb: int = 8, na: int = 2):
        super().__init__()
        if not 1 <= na <= _MAX_NA or not 1 <= nb <= _NB_SIZES[-1]:
            raise ValueError(f"the fused block needs 1 <= na <= {_MAX_NA} and 1 <= nb <= {_NB_SIZES[-1]}")
        self.in_channels, self.out_channels, self.nb, self.na = in_channels, out_channels, nb, na
        self.b_coeff = nn.Parameter(torch.randn(out_channels, in_channels, nb) * 0.01)
        self.a_coeff = nn.Parameter(torch.zeros(out_channels, in_channels, na))

    @property
    def n_pairs(self) -> int:
        return self.in_channels * self.out_channels

    def forward(self, u: torch.Tensor, state: dict | None = None, return_state: bool = False):
        y, new_state = linear_block(u, self.b_coeff, self.a_coeff, state)
        return (y, new_state) if return_state else y


class _PointwiseMLP(nn.Module):
    """The static nonlinearity F: an MLP on the feature axis with the parameter names of tsfast's
    ``SeqLinear`` (``tsfast/models/_core/layers.py:16-60``: ``lin.<k>.0`` hidden layers, last ``lin.<n>``)."""

    def __init__(self, input_size: int, output_size: int, hidden_size: int, hidden_layer: int, act: type[nn.Module]):
        super().__init__()
        if hidden_layer < 1:
            self.lin = nn.Linear(input_size, output_size)
        else:
            sizes = [input_size] + [hidden_size] * hidden_layer
            self.lin = nn.Sequential(*[nn.Sequential(nn.Linear(i, o), act()) for i, o in zip(sizes[:-1], sizes[1:])],
                                     nn.Linear(hidden_size, output_size))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.lin(x)


class DynoNet(nn.Module):
    """``G1 -> F -> G2`` with an optional parallel linear path ``G_lin`` (Forgione & Piga 2021), the
    mirror of tsfast's ``DynoNet`` (``dynonet/core.py:257-346``) on the fused G-blocks: same
    constructor arguments, submodule names (``g1``, ``f``, ``g2``, ``g_lin``) and state protocol
    (``forward(u, state=None)`` with ``{"g1": ..., "g2": ..., "lin": ...}``)."""

    def __init__(self, input_size: int, output_size: int, n_channels: int = 8, nb: int = 8, na: int = 2,
                 hidden_size: int = 32, hidden_layers: int = 1, act: type[nn.Module] = nn.Tanh, bypass: bool = True,
                 return_state: bool = False):
        super().__init__()
        self.return_state = return_state
        self.g1 = LinearDynamicalOperator(input_size, n_channels, nb, na)
        self.f = _PointwiseMLP(n_channels, n_channels, hidden_size, hidden_layers, act)
        self.g2 = LinearDynamicalOperator(n_channels, output_size, nb, na)
        self.g_lin = LinearDynamicalOperator(input_size, output_size, nb, na) if bypass else None

    def forward(self, u: torch.Tensor, state: dict | None = None):
        match state:
            case None:
                s1 = s2 = s_lin = None
            case dict():
                s1, s2, s_lin = state.get("g1"), state.get("g2"), state.get("lin")
            case _:
                raise TypeError(f"expected state dict, got {type(state)}")
        y1, s1 = self.g1(u, state=s1, return_state=True)
        y, s2 = self.g2(self.f(y1), state=s2, return_state=True)
        new_state = {"g1": s1, "g2": s2}
        if self.g_lin is not None:
            y_lin, s_lin = self.g_lin(u, state=s_lin, return_state=True)
            y = y + y_lin
            new_state["lin"] = s_lin
        return (y, new_state) if self.return_state else y
