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

from . import _lib, _spec

__all__ = ["supports", "run", "calls"]

calls = 0  # launches through this module since import (the drop-in tests read it)

_ORDER = {"na": (1, 16)}
# what run() accepts: coefficients and state spread over the leading dims of w
_PUBLIC = _spec.Contract(
    op="dynonet_allpole",
    tensors=(_spec.Tensor("w", (..., "L")), _spec.Tensor("a", ("na",), spread=True, over="w"),
             _spec.Tensor("y0", ("na",), optional=True, spread=True, over="w")),
    dtypes=(torch.float32,), ranges=_ORDER)
# what the ops take: one row per lane
_ON_LANES = _spec.Contract(
    op="dynonet_allpole",
    tensors=(_spec.Tensor("w", ("lanes", "L")), _spec.Tensor("a", ("lanes", "na")),
             _spec.Tensor("y0", ("lanes", "na"), optional=True)),
    dtypes=(torch.float32,), ranges=_ORDER)


def supports(a: torch.Tensor, w: torch.Tensor, y0: torch.Tensor | None) -> str | None:
    """Reason these tensors cannot be handled, or None when they can."""
    if w.dim() < 2:
        return "w needs a lane axis and a time axis"
    return _spec.explain(_PUBLIC, w=w, a=a, y0=y0)


@torch.library.custom_op("b200scan::dynonet_allpole", mutates_args=())
def _allpole_op(a: torch.Tensor, w: torch.Tensor, y0: torch.Tensor | None) -> torch.Tensor:
    global calls
    a, w, y0 = _spec.dense(a, w, y0)
    _spec.demand(_ON_LANES, w=w, a=a, y0=y0)
    y = torch.empty_like(w)
    if y.numel():
        calls += 1
        lanes, steps = w.shape
        _lib.check(_lib.lib().b200_allpole_fwd(lanes, steps, a.shape[1], _lib.ptr(a), _lib.ptr(w), _lib.ptr(y0),
                                               _lib.ptr(y), _lib.stream_ptr(w.device)), "b200_allpole_fwd")
    return y


@_allpole_op.register_fake
def _(a, w, y0):
    return torch.empty_like(w)


@torch.library.custom_op("b200scan::dynonet_allpole_bwd", mutates_args=())
def _allpole_bwd_op(
    g: torch.Tensor, a: torch.Tensor, y: torch.Tensor, y0: torch.Tensor | None
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    global calls
    g, a, y, y0 = _spec.dense(g, a, y, y0)
    _spec.demand(_ON_LANES, w=y, a=a, y0=y0)
    _lib.require_dense_cuda(g=g)
    gw, ga = torch.empty_like(g), torch.empty_like(a)
    gy0 = None if y0 is None else torch.empty_like(y0)
    if y.shape[0]:
        calls += 1
        lanes, steps = y.shape
        _lib.check(_lib.lib().b200_allpole_bwd(lanes, steps, a.shape[1], _lib.ptr(g), _lib.ptr(a), _lib.ptr(y),
                                               _lib.ptr(y0), _lib.ptr(ga), _lib.ptr(gw), _lib.ptr(gy0),
                                               _lib.stream_ptr(y.device)), "b200_allpole_bwd")
    return ga, gw, (a.new_empty(0) if gy0 is None else gy0)


@_allpole_bwd_op.register_fake
def _(g, a, y, y0):
    return torch.empty_like(a), torch.empty_like(g), (a.new_empty(0) if y0 is None else torch.empty_like(y0))


def _remember(ctx, inputs, output):
    a, _, y0 = inputs
    ctx.save_for_backward(a, output, y0)


def _adjoint(ctx, g):
    a, y, y0 = ctx.saved_tensors
    ga, gw, gy0 = _allpole_bwd_op(g, a, y, y0)
    return ga, gw, (None if y0 is None else gy0)


_allpole_op.register_autograd(_adjoint, setup_context=_remember)


def run(a: torch.Tensor, w: torch.Tensor, y0: torch.Tensor | None) -> torch.Tensor:
    """Run the filter bank; differentiable in ``a``, ``w`` and ``y0``.

    ``a [..., na]`` and ``y0 [..., na]`` broadcast over the leading dims of ``w [..., L]``; they are
    spread onto lanes here, outside the op, so autograd folds lane gradients back.
    """
    rows_w, rows_a, rows_y0 = _spec.lanes(w, 1, a, y0)
    return _allpole_op(rows_a, rows_w, rows_y0).reshape(w.shape)
