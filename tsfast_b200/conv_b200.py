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

from . import _lib

__all__ = ["supports", "run"]


def supports(x, tail, weight, bias) -> str | None:
    """Reason these tensors cannot be handled, or None when they can."""
    if not torch.cuda.is_available():
        return "CUDA not available"
    tensors = {"x": x, "tail": tail, "weight": weight}
    if bias is not None:
        tensors["bias"] = bias
    for name, tt in tensors.items():
        if tt.device.type != "cuda":
            return f"{name} not on CUDA"
        if tt.dtype != torch.float32:
            return f"needs float32, got {name}={tt.dtype}"
    if x.dim() != 3:
        return f"x must be [B, L, D], got {x.dim()} dims"
    B, L, D = x.shape
    if weight.dim() != 3 or weight.shape[0] != D or weight.shape[1] != 1:
        return f"weight.shape {tuple(weight.shape)} is not depthwise [D, 1, K] for D={D}"
    K = weight.shape[-1]
    if not 2 <= K <= 8:
        return f"kernel width {K} outside the supported range [2, 8]"
    if tuple(tail.shape) != (B, D, K - 1):
        return f"tail.shape {tuple(tail.shape)} != {(B, D, K - 1)}"
    if bias is not None and tuple(bias.shape) != (D,):
        return f"bias.shape {tuple(bias.shape)} != {(D,)}"
    return None


def _channel_last(x):
    """x with unit channel stride (a copy only if the view is strided along channels)."""
    return x if x.shape[-1] == 1 or x.stride(-1) == 1 else x.contiguous()


def _check(x, tail, w, bias, name):
    if x.dim() != 3 or w.dim() != 2 or w.shape[0] != x.shape[2] or not 2 <= w.shape[1] <= 8:
        raise RuntimeError(f"b200scan::{name}: expected x [B,L,D] and weight [D,K], 2<=K<=8, got "
                           f"{tuple(x.shape)} and {tuple(w.shape)}")
    for t in (x, tail, w, bias):
        if t is not None and (t.dtype != torch.float32 or t.device.type != "cuda"):
            raise RuntimeError(f"b200scan::{name}: needs float32 CUDA tensors")


@torch.library.custom_op("b200scan::mamba_conv_silu", mutates_args=())
def _conv_silu_op(x: torch.Tensor, tail: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    x = _channel_last(x)
    tail, weight = tail.contiguous(), weight.contiguous()
    bias = bias.contiguous() if bias is not None else None
    _check(x, tail, weight, bias, "mamba_conv_silu")
    B, L, D = x.shape
    out = torch.empty(B, L, D, device=x.device, dtype=x.dtype)
    if out.numel():
        st = _lib.lib().b200_conv_silu_fwd(B, L, D, weight.shape[1], _lib.ptr(x), x.stride(0), x.stride(1), _lib.ptr(tail),
                                           _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(out), _lib.stream_ptr(x.device))
        _lib.check(st, "b200_conv_silu_fwd")
    return out


@_conv_silu_op.register_fake
def _(x, tail, weight, bias):
    return torch.empty(x.shape, device=x.device, dtype=x.dtype)


@torch.library.custom_op("b200scan::mamba_conv_silu_bwd", mutates_args=())
def _conv_silu_bwd_op(
    gy: torch.Tensor, x: torch.Tensor, tail: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    x = _channel_last(x)
    gy, tail, weight = gy.contiguous(), tail.contiguous(), weight.contiguous()
    bias = bias.contiguous() if bias is not None else None
    _check(x, tail, weight, bias, "mamba_conv_silu_bwd")
    B, L, D = x.shape
    K = weight.shape[1]
    gx = torch.empty(B, L, D, device=x.device, dtype=x.dtype)
    gtail = torch.zeros_like(tail)
    gw = torch.zeros_like(weight)
    gb = torch.zeros_like(bias) if bias is not None else None
    if gx.numel():
        L_ = _lib.lib()
        ws = _lib.workspace(L_.b200_conv_silu_bwd_workspace_bytes(B, L, D, K), x.device)
        st = L_.b200_conv_silu_bwd(B, L, D, K, _lib.ptr(gy), _lib.ptr(x), x.stride(0), x.stride(1), _lib.ptr(tail),
                                   _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(gx), _lib.ptr(gtail), _lib.ptr(gw),
                                   _lib.ptr(gb), _lib.ptr(ws), ws.numel(), _lib.stream_ptr(x.device))
        _lib.check(st, "b200_conv_silu_bwd")
    return gx, gtail, gw, (gb if gb is not None else gx.new_empty(0))


@_conv_silu_bwd_op.register_fake
def _(gy, x, tail, weight, bias):
    gb = torch.empty_like(bias) if bias is not None else gy.new_empty(0)
    return torch.empty(x.shape, device=x.device, dtype=x.dtype), torch.empty_like(tail), torch.empty_like(weight), gb


def _conv_setup(ctx, inputs, output):
    x, tail, weight, bias = inputs
    ctx.save_for_backward(x, tail, weight, bias)


def _conv_backward(ctx, gy):
    x, tail, weight, bias = ctx.saved_tensors
    gx, g_tail, gw, gb = _conv_silu_bwd_op(gy, x, tail, weight, bias)
    return gx, g_tail, gw, (gb if bias is not None else None)


_conv_silu_op.register_autograd(_conv_backward, setup_context=_conv_setup)


def run(x, tail, weight, bias):
    """Fused causal depthwise conv + SiLU → ``[B, L, D]`` contiguous; differentiable in all inputs."""
    return _conv_silu_op(x, tail.contiguous(), weight.contiguous().squeeze(1), bias)
