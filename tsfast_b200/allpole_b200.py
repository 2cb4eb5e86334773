"""B200 backend for banks of scalar all-pole (order-``na`` IIR) recurrences, the dynoNet denominator.

``y_t = w_t - sum_{i=1..na} a_i y_{t-i}`` per lane, with ``y0[..., j] = y_{-1-j}`` the carried state
(newest first).  Drop-in for the reference's ``tsfast/models/architectures/dynonet/allpole_triton.py``
module: the same ``supports(a, w, y0)`` / ``run(a, w, y0)`` protocol, the same forward/backward
custom-op pair with fake implementations and an analytic adjoint (here under the ``b200scan``
namespace), float32, ``1 <= na <= 16``.  The kernels behind it are ``b200_allpole_fwd`` /
``b200_allpole_bwd`` of ``libb200scan.so``; unlike the reference the adjoint kernel finishes
``grad_a`` (sign and initial-state taps) and ``grad_y0`` on the device.
"""

from __future__ import annotations

import torch

from . import _lib

__all__ = ["supports", "run"]

_MAX_NA = 16


def supports(a: torch.Tensor, w: torch.Tensor, y0: torch.Tensor | None) -> str | None:
    """Reason these tensors cannot be handled, or None when they can."""
    if not torch.cuda.is_available():
        return "CUDA not available"
    if w.device.type != "cuda" or a.device.type != "cuda" or (y0 is not None and y0.device.type != "cuda"):
        return "inputs not on CUDA"
    if any(t is not None and t.dtype != torch.float32 for t in (a, w, y0)):
        return "needs float32 tensors"
    if w.dim() < 2:
        return "w must have at least a batch and a time axis"
    na = a.shape[-1]
    if not 1 <= na <= _MAX_NA:
        return f"na={na} outside the supported range [1, {_MAX_NA}]"
    lead = w.shape[:-1]
    try:
        if torch.broadcast_shapes(a.shape[:-1], lead) != lead:
            return f"a leading dims {tuple(a.shape[:-1])} do not broadcast into {tuple(lead)}"
        if y0 is not None and torch.broadcast_shapes(y0.shape[:-1], lead) != lead:
            return f"y0 leading dims {tuple(y0.shape[:-1])} do not broadcast into {tuple(lead)}"
    except RuntimeError as e:
        return f"shape mismatch: {e}"
    if y0 is not None and y0.shape[-1] != na:
        return f"y0 state dim {y0.shape[-1]} != na {na}"
    return None


def _check_lane_layout(a, w, y0, name):
    if w.dim() != 2 or a.dim() != 2 or a.shape[0] != w.shape[0] or not 1 <= a.shape[1] <= _MAX_NA:
        raise RuntimeError(f"b200scan::{name}: expected a [lanes, na<=16] and w [lanes, L], got "
                           f"{tuple(a.shape)} and {tuple(w.shape)}")
    if y0 is not None and y0.shape != a.shape:
        raise RuntimeError(f"b200scan::{name}: y0 {tuple(y0.shape)} must match a {tuple(a.shape)}")
    for t in (a, w, y0):
        if t is not None and t.dtype != torch.float32:
            raise RuntimeError(f"b200scan::{name}: needs float32 tensors")
    _lib.require_dense_cuda(a=a, w=w, y0=y0)


@torch.library.custom_op("b200scan::dynonet_allpole", mutates_args=())
def _allpole_op(a: torch.Tensor, w: torch.Tensor, y0: torch.Tensor | None) -> torch.Tensor:
    a, w = a.contiguous(), w.contiguous()
    y0 = y0.contiguous() if y0 is not None else None
    _check_lane_layout(a, w, y0, "dynonet_allpole")
    lanes, L = w.shape
    y = torch.empty_like(w)
    if y.numel():
        st = _lib.lib().b200_allpole_fwd(lanes, L, a.shape[1], _lib.ptr(a), _lib.ptr(w), _lib.ptr(y0), _lib.ptr(y),
                                         _lib.stream_ptr(w.device))
        _lib.check(st, "b200_allpole_fwd")
    return y


@_allpole_op.register_fake
def _(a, w, y0):
    return torch.empty_like(w)


@torch.library.custom_op("b200scan::dynonet_allpole_bwd", mutates_args=())
def _allpole_bwd_op(
    g: torch.Tensor, a: torch.Tensor, y: torch.Tensor, y0: torch.Tensor | None
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    g, a, y = g.contiguous(), a.contiguous(), y.contiguous()
    y0 = y0.contiguous() if y0 is not None else None
    _check_lane_layout(a, y, y0, "dynonet_allpole_bwd")
    _lib.require_dense_cuda(g=g)
    lanes, L = y.shape
    gw = torch.empty_like(g)
    ga = torch.empty_like(a)
    gy0 = torch.empty_like(y0) if y0 is not None else None
    if lanes:
        st = _lib.lib().b200_allpole_bwd(lanes, L, a.shape[1], _lib.ptr(g), _lib.ptr(a), _lib.ptr(y), _lib.ptr(y0),
                                         _lib.ptr(ga), _lib.ptr(gw), _lib.ptr(gy0), _lib.stream_ptr(y.device))
        _lib.check(st, "b200_allpole_bwd")
    return ga, gw, (gy0 if gy0 is not None else a.new_empty(0))


@_allpole_bwd_op.register_fake
def _(g, a, y, y0):
    gy0 = torch.empty_like(y0) if y0 is not None else a.new_empty(0)
    return torch.empty_like(a), torch.empty_like(g), gy0


def _allpole_setup(ctx, inputs, output):
    a, w, y0 = inputs
    ctx.save_for_backward(a, output, y0)


def _allpole_backward(ctx, g):
    a, y, y0 = ctx.saved_tensors
    grad_a, grad_w, grad_y0 = _allpole_bwd_op(g, a, y, y0)
    return grad_a, grad_w, (grad_y0 if y0 is not None else None)


_allpole_op.register_autograd(_allpole_backward, setup_context=_allpole_setup)


def run(a: torch.Tensor, w: torch.Tensor, y0: torch.Tensor | None) -> torch.Tensor:
    """Run the filter bank; differentiable in ``a``, ``w`` and ``y0``.

    ``a [..., na]`` and ``y0 [..., na]`` broadcast over the leading dims of ``w [..., L]``; the
    broadcast is materialised here, outside the op, so autograd folds lane gradients back.
    """
    lead, L, na = w.shape[:-1], w.shape[-1], a.shape[-1]
    a_lane = a.broadcast_to(lead + (na,)).reshape(-1, na)
    w_flat = w.reshape(-1, L)
    y0_lane = y0.broadcast_to(lead + (na,)).reshape(-1, na) if y0 is not None else None
    return _allpole_op(a_lane, w_flat, y0_lane).reshape(w.shape)
