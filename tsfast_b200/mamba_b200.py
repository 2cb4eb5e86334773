"""B200 backend of the fused Mamba selective-scan section.

``h_t = exp(softplus(draw_t) A) h_{t-1} + softplus(draw_t) u_t B_t``,
``out_t = (h_t . C_t + Dp u_t) * silu(z_t)``, returning ``(out [B,L,D], h_last [B,D,N])``.

Drop-in for the reference's ``tsfast/models/architectures/mamba/mamba_triton.py`` (and the CPU
``backend_c.py``): the same ``supports(draw, A, Bt, Ct, u, z, Dp, h0)`` / ``run(...)`` protocol and
the same three custom ops (inference, training with state checkpoints, backward) with fake
implementations, under the ``b200scan`` namespace.  ``run`` is differentiable in all eight inputs
and in ``h_last``.  The kernels are ``b200_mamba_fwd`` / ``b200_mamba_bwd`` of ``libb200scan.so``.
The training op's third output holds the states the adjoint restarts from, one per
``b200_mamba_chk_interval()`` steps; its shape is this library's choice (the interface only asks
that the fake implementation agrees with the real one).
"""

from __future__ import annotations

import functools

import torch

from . import _lib, _spec

__all__ = ["supports", "run", "calls"]

calls = 0  # launches through this module since import (the drop-in tests read it)

_CONTRACT = _spec.Contract(
    op="mamba_scan",
    tensors=(_spec.Tensor("draw", ("B", "L", "D")), _spec.Tensor("A", ("D", "N")), _spec.Tensor("Bt", ("B", "L", "N")),
             _spec.Tensor("Ct", ("B", "L", "N")), _spec.Tensor("u", ("B", "L", "D")), _spec.Tensor("z", ("B", "L", "D")),
             _spec.Tensor("Dp", ("D",)), _spec.Tensor("h0", ("B", "D", "N"), optional=True)),
    dtypes=(torch.float32,), ranges={"N": (1, 128)})
_NAMES = ("draw", "A", "Bt", "Ct", "u", "z", "Dp", "h0")


def supports(draw, A, Bt, Ct, u, z, Dp, h0) -> str | None:
    """Reason these tensors cannot be handled, or None when they can."""
    return _spec.explain(_CONTRACT, **dict(zip(_NAMES, (draw, A, Bt, Ct, u, z, Dp, h0))))


@functools.lru_cache(maxsize=None)
def _interval() -> int:
    """Steps between two stored states (a property of the loaded library)."""
    return int(_lib.lib().b200_mamba_chk_interval())


def _slots(steps: int) -> int:
    return -(-steps // _interval())


def _launch_forward(args, keep_states: bool):
    global calls
    args = _spec.dense(*args)
    _spec.demand(_CONTRACT, **dict(zip(_NAMES, args)))
    draw, A = args[0], args[1]
    rows, steps, chans = draw.shape
    n = A.shape[1]
    out = torch.empty_like(draw)
    h_last = draw.new_empty(rows, chans, n)
    states = draw.new_empty(rows, _slots(steps), chans, n) if keep_states else None
    if rows and chans:
        calls += 1
        rc = _lib.lib().b200_mamba_fwd(rows, steps, chans, n, *(_lib.ptr(t) for t in args), _lib.ptr(out),
                                       _lib.ptr(h_last), _lib.ptr(states), _lib.stream_ptr(draw.device))
        _lib.check(rc, "b200_mamba_fwd")
    return out, h_last, states


@torch.library.custom_op("b200scan::mamba_scan", mutates_args=())
def _scan_op(
    draw: torch.Tensor, A: torch.Tensor, Bt: torch.Tensor, Ct: torch.Tensor, u: torch.Tensor, z: torch.Tensor,
    Dp: torch.Tensor, h0: torch.Tensor | None,
) -> tuple[torch.Tensor, torch.Tensor]:
    out, h_last, _ = _launch_forward((draw, A, Bt, Ct, u, z, Dp, h0), keep_states=False)
    return out, h_last


@torch.library.custom_op("b200scan::mamba_scan_train", mutates_args=())
def _scan_train_op(
    draw: torch.Tensor, A: torch.Tensor, Bt: torch.Tensor, Ct: torch.Tensor, u: torch.Tensor, z: torch.Tensor,
    Dp: torch.Tensor, h0: torch.Tensor | None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return _launch_forward((draw, A, Bt, Ct, u, z, Dp, h0), keep_states=True)


@_scan_op.register_fake
def _(draw, A, Bt, Ct, u, z, Dp, h0):
    return torch.empty_like(draw), draw.new_empty(draw.shape[0], draw.shape[2], A.shape[1])


@_scan_train_op.register_fake
def _(draw, A, Bt, Ct, u, z, Dp, h0):
    rows, steps, chans = draw.shape
    return (torch.empty_like(draw), draw.new_empty(rows, chans, A.shape[1]),
            draw.new_empty(rows, _slots(steps), chans, A.shape[1]))


@torch.library.custom_op("b200scan::mamba_scan_bwd", mutates_args=())
def _scan_bwd_op(
    gout: torch.Tensor, ghlast: torch.Tensor | None, chk: torch.Tensor, draw: torch.Tensor, A: torch.Tensor,
    Bt: torch.Tensor, Ct: torch.Tensor, u: torch.Tensor, z: torch.Tensor, Dp: torch.Tensor, h0: torch.Tensor | None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
           torch.Tensor]:
    global calls
    gout, ghlast, chk, draw, A, Bt, Ct, u, z, Dp, h0 = _spec.dense(gout, ghlast, chk, draw, A, Bt, Ct, u, z, Dp, h0)
    _lib.require_dense_cuda(gout=gout, ghlast=ghlast, chk=chk)
    rows, steps, chans = draw.shape
    n = A.shape[1]
    grads = {"draw": torch.empty_like(draw), "A": draw.new_empty(chans, n), "Bt": draw.new_empty(rows, steps, n),
             "Ct": draw.new_empty(rows, steps, n), "u": torch.empty_like(draw), "z": torch.empty_like(draw),
             "Dp": draw.new_empty(chans), "h0": None if h0 is None else draw.new_empty(rows, chans, n)}
    if rows and chans:
        calls += 1
        L_ = _lib.lib()
        ws = _lib.workspace(L_.b200_mamba_bwd_workspace_bytes(rows, steps, chans, n), draw.device)
        inputs = (draw, A, Bt, Ct, u, z, Dp, h0, chk, gout, ghlast)
        outputs = tuple(grads[k] for k in ("draw", "A", "Bt", "Ct", "u", "z", "Dp", "h0"))
        rc = L_.b200_mamba_bwd(rows, steps, chans, n, *(_lib.ptr(t) for t in inputs + outputs), _lib.ptr(ws), ws.numel(),
                               _lib.stream_ptr(draw.device))
        _lib.check(rc, "b200_mamba_bwd")
    else:  # empty batch or no channels: the sums over (batch, time) are empty
        grads["A"].zero_()
        grads["Dp"].zero_()
    if grads["h0"] is None:
        grads["h0"] = gout.new_empty(0)
    return tuple(grads[k] for k in ("draw", "A", "Bt", "Ct", "u", "z", "Dp", "h0"))


@_scan_bwd_op.register_fake
def _(gout, ghlast, chk, draw, A, Bt, Ct, u, z, Dp, h0):
    rows, steps, chans = draw.shape
    n = A.shape[1]
    per_step_n = draw.new_empty(rows, steps, n)
    return (torch.empty_like(draw), torch.empty_like(A), per_step_n, torch.empty_like(per_step_n), torch.empty_like(draw),
            torch.empty_like(draw), torch.empty_like(Dp), (draw.new_empty(0) if h0 is None else draw.new_empty(rows, chans, n)))


def _remember(ctx, inputs, output):
    ctx.save_for_backward(*inputs, output[2])


def _adjoint(ctx, gout, ghlast, _gstates):
    *inputs, states = ctx.saved_tensors
    draw, h0 = inputs[0], inputs[7]
    if gout is None:  # only h_last was used downstream
        gout = torch.zeros_like(draw)
    grads = _scan_bwd_op(gout, ghlast, states, *inputs)
    return grads[:7] + ((None if h0 is None else grads[7]),)


_scan_train_op.register_autograd(_adjoint, setup_context=_remember)


def run(draw, A, Bt, Ct, u, z, Dp, h0):
    """Fused section → ``(out [B, L, D], h_last [B, D, N])``; differentiable in every input and in ``h_last``."""
    needs_grad = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (draw, A, Bt, Ct, u, z, Dp, h0))
    if not needs_grad:
        return _scan_op(draw, A, Bt, Ct, u, z, Dp, h0)
    out, h_last, _states = _scan_train_op(draw, A, Bt, Ct, u, z, Dp, h0)
    return out, h_last
