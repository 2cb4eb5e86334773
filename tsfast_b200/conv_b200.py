"""B200 backend of the Mamba block's causal depthwise convolution + SiLU.

``run(x, tail, weight, bias) = silu(conv1d(cat(tail, x), weight, bias))`` on channel-last
``x [B, L, D]`` with the carried left context ``tail [B, D, K-1]`` and depthwise
``weight [D, 1, K]``.  Drop-in for the reference's
``tsfast/models/architectures/mamba/conv_triton.py`` module: same ``supports`` / ``run`` protocol,
same forward/backward custom-op pair (here ``b200scan::mamba_conv_silu``), float32, ``2 <= K <= 8``.
The strided ``in_proj`` chunk view is read in place as long as its channel stride is 1; the
adjoint kernel also produces the tail gradient (the reference finishes that in PyTorch).
"""

from __future__ import annotations

import torch

from . import _lib, _spec

__all__ = ["supports", "run", "calls"]

calls = 0  # launches through this module since import (the drop-in tests read it)

_WIDTH = {"K": (2, 8)}
_F32 = (torch.float32,)


def _contract(weight_dims):
    return _spec.Contract(
        op="mamba_conv_silu",
        tensors=(_spec.Tensor("x", ("B", "L", "D")), _spec.Tensor("weight", weight_dims),
                 _spec.Tensor("tail", ("B", "D", "Km1")), _spec.Tensor("bias", ("D",), optional=True)),
        dtypes=_F32, ranges=_WIDTH)


_PUBLIC = _contract(("D", 1, "K"))  # the module's depthwise Conv1d weight
_OP = _contract(("D", "K"))         # what the ops take


def _window_mismatch(weight, tail) -> str | None:
    if tail.shape[-1] != weight.shape[-1] - 1:
        return f"tail carries {tail.shape[-1]} steps, a width-{weight.shape[-1]} window needs {weight.shape[-1] - 1}"
    return None


def supports(x, tail, weight, bias) -> str | None:
    """Reason these tensors cannot be handled, or None when they can."""
    return _spec.explain(_PUBLIC, x=x, weight=weight, tail=tail, bias=bias) or _window_mismatch(weight, tail)


def _unit_channel_stride(x):
    """``x`` itself when its channels are adjacent in memory, else a dense copy."""
    return x if x.shape[-1] == 1 or x.stride(-1) == 1 else x.contiguous()


def _guard(x, tail, weight, bias, suffix=""):
    why = _spec.explain(_OP, x=x, weight=weight, tail=tail, bias=bias) or _window_mismatch(weight, tail)
    if why is not None:
        raise RuntimeError(f"b200scan::mamba_conv_silu{suffix}: {why}")


@torch.library.custom_op("b200scan::mamba_conv_silu", mutates_args=())
def _conv_silu_op(x: torch.Tensor, tail: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    global calls
    x = _unit_channel_stride(x)
    tail, weight, bias = _spec.dense(tail, weight, bias)
    _guard(x, tail, weight, bias)
    rows, steps, chans = x.shape
    out = torch.empty(rows, steps, chans, device=x.device, dtype=x.dtype)
    if out.numel():
        calls += 1
        _lib.check(_lib.lib().b200_conv_silu_fwd(rows, steps, chans, weight.shape[1], _lib.ptr(x), x.stride(0), x.stride(1),
                                                 _lib.ptr(tail), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(out),
                                                 _lib.stream_ptr(x.device)), "b200_conv_silu_fwd")
    return out


@_conv_silu_op.register_fake
def _(x, tail, weight, bias):
    return torch.empty(x.shape, device=x.device, dtype=x.dtype)


@torch.library.custom_op("b200scan::mamba_conv_silu_bwd", mutates_args=())
def _conv_silu_bwd_op(
    gy: torch.Tensor, x: torch.Tensor, tail: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    global calls
    x = _unit_channel_stride(x)
    gy, tail, weight, bias = _spec.dense(gy, tail, weight, bias)
    _guard(x, tail, weight, bias, "_bwd")
    rows, steps, chans = x.shape
    gx = torch.empty(rows, steps, chans, device=x.device, dtype=x.dtype)
    gtail, gw = torch.zeros_like(tail), torch.zeros_like(weight)
    gb = None if bias is None else torch.zeros_like(bias)
    if gx.numel():
        calls += 1
        L_ = _lib.lib()
        width = weight.shape[1]
        ws = _lib.workspace(L_.b200_conv_silu_bwd_workspace_bytes(rows, steps, chans, width), x.device)
        _lib.check(L_.b200_conv_silu_bwd(rows, steps, chans, width, _lib.ptr(gy), _lib.ptr(x), x.stride(0), x.stride(1),
                                         _lib.ptr(tail), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(gx), _lib.ptr(gtail),
                                         _lib.ptr(gw), _lib.ptr(gb), _lib.ptr(ws), ws.numel(), _lib.stream_ptr(x.device)),
                   "b200_conv_silu_bwd")
    return gx, gtail, gw, (gx.new_empty(0) if gb is None else gb)


@_conv_silu_bwd_op.register_fake
def _(gy, x, tail, weight, bias):
    return (torch.empty(x.shape, device=x.device, dtype=x.dtype), torch.empty_like(tail), torch.empty_like(weight),
            (gy.new_empty(0) if bias is None else torch.empty_like(bias)))


def _remember(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _adjoint(ctx, gy):
    x, tail, weight, bias = ctx.saved_tensors
    gx, gtail, gw, gb = _conv_silu_bwd_op(gy, x, tail, weight, bias)
    return gx, gtail, gw, (None if bias is None else gb)


_conv_silu_op.register_autograd(_adjoint, setup_context=_remember)


def run(x, tail, weight, bias):
    """Fused causal depthwise conv + SiLU → ``[B, L, D]`` contiguous; differentiable in all inputs."""
    return _conv_silu_op(x, tail.contiguous(), weight.contiguous().squeeze(1), bias)
