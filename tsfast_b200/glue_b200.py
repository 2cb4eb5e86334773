"""Pointwise glue of the LRU / S5 blocks on B200: LayerNorm and the gated residual, one HBM pass each.

tsfast's pre-norm blocks wrap the scan layer as ``u + GLU(gelu(layer(LayerNorm(u))))``
(``architectures/lru.py:145-152``, ``s5.py:233-257``).  With the scans and the projections fast, the
LayerNorm over a short feature axis and the separate GLU / multiply / add kernels are what is left
of a block.  This module provides

* ``layer_norm(x, weight, bias, eps)`` – ``F.layer_norm`` over the last axis (width up to 512);
* ``glu_residual(u, z)``               – ``u + F.glu(z, dim=-1)``;
* ``gate_residual(u, a, b)``           – ``u + a * sigmoid(b)``;
* ``column_sums(g)``                   – ``g.sum(0)`` of a ``[M, D]`` matrix in a fixed order (the bias
  gradient of the linear layers; no autograd of its own);

each a custom op pair (forward, adjoint) on ``libb200scan.so`` with fake implementations.
``tsfast_b200.accelerate_linears(model)`` routes a model's ``nn.LayerNorm`` modules here and
``install(fuse_projections=True)`` the block bodies.
"""

from __future__ import annotations

import torch

from . import _lib

__all__ = ["layer_norm", "glu_residual", "gate_residual", "column_sums", "supports_norm", "calls"]

calls = 0  # launches through this module since import (the drop-in tests read it)
_MAX_WIDTH = 512


def _cuda_f32(*ts) -> bool:
    return all(t is None or (t.is_cuda and t.dtype == torch.float32) for t in ts)


@torch.library.custom_op("b200scan::column_sums", mutates_args=())
def _colsum_op(g: torch.Tensor) -> torch.Tensor:
    global calls
    if not _cuda_f32(g) or g.dim() != 2:
        raise RuntimeError("b200scan::column_sums: needs a float32 CUDA matrix [M, D]")
    m, d = g.shape
    if (d > 1 and g.stride(1) != 1) or (m > 1 and g.stride(0) < d):
        g = g.contiguous()  # expanded or transposed views
    if d > (1024 if (g.data_ptr() % 16 == 0 and (m < 2 or g.stride(0) % 4 == 0) and d % 4 == 0) else 256):
        return g.sum(0)  # wider than the kernel's row groups: PyTorch's reduction, same device
    out = g.new_empty(d)
    L_ = _lib.lib()
    ws = _lib.workspace(L_.b200_colsum_workspace_bytes(m, d), g.device)
    calls += 1
    _lib.check(L_.b200_colsum(m, d, _lib.ptr(g), g.stride(0) if m > 1 else d, _lib.ptr(out), _lib.ptr(ws), ws.numel(),
                              _lib.stream_ptr(g.device)), "b200_colsum")
    return out


@_colsum_op.register_fake
def _(g):
    return g.new_empty(g.shape[1])


def column_sums(g: torch.Tensor) -> torch.Tensor:
    """``g.sum(0)`` for a float32 CUDA matrix, one pass over HBM, summed in a fixed order."""
    return _colsum_op(g)


def supports_norm(x: torch.Tensor, normalized_shape) -> str | None:
    """Reason ``layer_norm`` cannot take this input, or None when it can."""
    if not _cuda_f32(x):
        return "needs a float32 CUDA tensor"
    if len(tuple(normalized_shape)) != 1 or x.dim() < 1 or x.shape[-1] != tuple(normalized_shape)[0]:
        return "normalises over the last axis only"
    if not 1 <= x.shape[-1] <= _MAX_WIDTH:
        return f"feature width {x.shape[-1]} outside [1, {_MAX_WIDTH}]"
    return None


@torch.library.custom_op("b200scan::layer_norm", mutates_args=())
def _ln_op(x: torch.Tensor, weight: torch.Tensor | None, bias: torch.Tensor | None,
           eps: float) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    global calls
    if not _cuda_f32(x, weight, bias) or x.dim() != 2 or x.shape[1] > _MAX_WIDTH:
        raise RuntimeError("b200scan::layer_norm: needs float32 CUDA x [M, D] with D <= 512")
    x = x.contiguous()
    m, d = x.shape
    y = torch.empty_like(x)
    mean, rstd = x.new_empty(m), x.new_empty(m)
    if m:
        calls += 1
        _lib.check(_lib.lib().b200_layernorm_fwd(m, d, _lib.ptr(x), _lib.ptr(None if weight is None else weight.contiguous()),
                                                 _lib.ptr(None if bias is None else bias.contiguous()), float(eps), _lib.ptr(y),
                                                 _lib.ptr(mean), _lib.ptr(rstd), _lib.stream_ptr(x.device)), "b200_layernorm_fwd")
    return y, mean, rstd


@_ln_op.register_fake
def _(x, weight, bias, eps):
    return torch.empty_like(x), x.new_empty(x.shape[0]), x.new_empty(x.shape[0])


@torch.library.custom_op("b200scan::layer_norm_bwd", mutates_args=())
def _ln_bwd_op(g: torch.Tensor, x: torch.Tensor, weight: torch.Tensor | None, mean: torch.Tensor,
               rstd: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    global calls
    g, x = g.contiguous(), x.contiguous()
    m, d = x.shape
    dx = torch.empty_like(x)
    dgamma, dbeta = x.new_empty(d), x.new_empty(d)
    L_ = _lib.lib()
    ws = _lib.workspace(L_.b200_layernorm_bwd_workspace_bytes(m, d), x.device)
    calls += 1
    _lib.check(L_.b200_layernorm_bwd(m, d, _lib.ptr(g), _lib.ptr(x), _lib.ptr(None if weight is None else weight.contiguous()),
                                     _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(dx), _lib.ptr(dgamma), _lib.ptr(dbeta),
                                     _lib.ptr(ws), ws.numel(), _lib.stream_ptr(x.device)), "b200_layernorm_bwd")
    return dx, dgamma, dbeta


@_ln_bwd_op.register_fake
def _(g, x, weight, mean, rstd):
    return torch.empty_like(x), x.new_empty(x.shape[1]), x.new_empty(x.shape[1])


def _ln_remember(ctx, inputs, output):
    x, weight, bias, _eps = inputs
    ctx.has_weight, ctx.has_bias = weight is not None, bias is not None
    ctx.save_for_backward(x, weight, output[1], output[2])


def _ln_adjoint(ctx, gy, _gmean, _grstd):
    x, weight, mean, rstd = ctx.saved_tensors
    dx, dgamma, dbeta = _ln_bwd_op(gy, x, weight, mean, rstd)
    return dx, (dgamma if ctx.has_weight else None), (dbeta if ctx.has_bias else None), None


_ln_op.register_autograd(_ln_adjoint, setup_context=_ln_remember)


def layer_norm(x: torch.Tensor, weight: torch.Tensor | None, bias: torch.Tensor | None, eps: float = 1e-5) -> torch.Tensor:
    """``F.layer_norm(x, (x.shape[-1],), weight, bias, eps)`` for float32 CUDA ``x [..., D]``, ``D <= 512``."""
    y, _, _ = _ln_op(x.reshape(-1, x.shape[-1]), weight, bias, eps)
    return y.reshape(x.shape)


def _rows(t: torch.Tensor) -> torch.Tensor:
    """2-D view with unit column stride (dense copy only if the last axis is strided)."""
    t2 = t.reshape(-1, t.shape[-1]) if t.dim() != 2 else t
    return t2 if t2.stride(1) == 1 or t2.shape[1] == 1 else t2.contiguous()


@torch.library.custom_op("b200scan::gate_residual", mutates_args=())
def _gate_op(u: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``u + a * sigmoid(b)`` for 2-D operands of one shape (row pitches are free)."""
    global calls
    if not _cuda_f32(u, a, b) or not (u.shape == a.shape == b.shape) or u.dim() != 2:
        raise RuntimeError("b200scan::gate_residual: needs three float32 CUDA matrices of one shape")
    u, a, b = _rows(u), _rows(a), _rows(b)
    m, d = u.shape
    out = torch.empty(m, d, device=u.device, dtype=u.dtype)
    if out.numel():
        calls += 1
        _lib.check(_lib.lib().b200_gated_residual_fwd(m, d, _lib.ptr(u), u.stride(0), _lib.ptr(a), a.stride(0), _lib.ptr(b),
                                                      b.stride(0), _lib.ptr(out), d, _lib.stream_ptr(u.device)),
                   "b200_gated_residual_fwd")
    return out


@_gate_op.register_fake
def _(u, a, b):
    return u.new_empty(u.shape)


@torch.library.custom_op("b200scan::gate_residual_bwd", mutates_args=())
def _gate_bwd_op(g: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Gradients of ``a`` and ``b`` packed side by side as ``[M, 2D]`` (``[:, :D]`` for a, ``[:, D:]`` for b)."""
    global calls
    g, a, b = _rows(g), _rows(a), _rows(b)
    m, d = a.shape
    packed = torch.empty(m, 2 * d, device=a.device, dtype=a.dtype)
    if packed.numel():
        calls += 1
        base = packed.data_ptr()
        _lib.check(_lib.lib().b200_gated_residual_bwd(m, d, _lib.ptr(g), g.stride(0), _lib.ptr(a), a.stride(0), _lib.ptr(b),
                                                      b.stride(0), base, 2 * d, base + 4 * d, 2 * d,
                                                      _lib.stream_ptr(a.device)), "b200_gated_residual_bwd")
    return packed


@_gate_bwd_op.register_fake
def _(g, a, b):
    return a.new_empty(a.shape[0], 2 * a.shape[1])


def _gate_remember(ctx, inputs, output):
    _, a, b = inputs
    ctx.save_for_backward(a, b)


def _gate_adjoint(ctx, g):
    a, b = ctx.saved_tensors
    d = a.shape[1]
    packed = _gate_bwd_op(g, a, b)
    return g, packed[:, :d], packed[:, d:]


_gate_op.register_autograd(_gate_adjoint, setup_context=_gate_remember)


def gate_residual(u: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``u + a * sigmoid(b)`` (all ``[..., D]``, float32 CUDA), one pass."""
    d = u.shape[-1]
    return _gate_op(u.reshape(-1, d), a.reshape(-1, d), b.reshape(-1, d)).reshape(u.shape)


@torch.library.custom_op("b200scan::glu_residual", mutates_args=())
def _glu_res_op(u: torch.Tensor, z: torch.Tensor) -> torch.Tensor:
    """``u [M, D] + glu(z [M, 2D])``: the two halves of ``z`` are read in place."""
    global calls
    if not _cuda_f32(u, z) or u.dim() != 2 or z.dim() != 2 or z.shape != (u.shape[0], 2 * u.shape[1]):
        raise RuntimeError("b200scan::glu_residual: needs float32 CUDA u [M, D] and z [M, 2D]")
    u, z = _rows(u), _rows(z)
    m, d = u.shape
    out = torch.empty(m, d, device=u.device, dtype=u.dtype)
    if out.numel():
        calls += 1
        zp = z.data_ptr()
        _lib.check(_lib.lib().b200_gated_residual_fwd(m, d, _lib.ptr(u), u.stride(0), zp, z.stride(0), zp + 4 * d, z.stride(0),
                                                      _lib.ptr(out), d, _lib.stream_ptr(u.device)), "b200_gated_residual_fwd")
    return out


@_glu_res_op.register_fake
def _(u, z):
    return u.new_empty(u.shape)


def _glu_remember(ctx, inputs, output):
    ctx.save_for_backward(inputs[1])


def _glu_adjoint(ctx, g):
    (z,) = ctx.saved_tensors
    d = z.shape[1] // 2
    return g, _gate_bwd_op(g, z[:, :d], z[:, d:])  # the packed gradient has exactly z's layout


_glu_res_op.register_autograd(_glu_adjoint, setup_context=_glu_remember)


def glu_residual(u: torch.Tensor, z: torch.Tensor) -> torch.Tensor:
    """``u + F.glu(z, dim=-1)`` for ``u [..., D]``, ``z [..., 2D]`` (float32 CUDA), one pass."""
    d = u.shape[-1]
    return _glu_res_op(u.reshape(-1, d), z.reshape(-1, 2 * d)).reshape(u.shape)
