"""dynoNet's linear block (G-block) with numerator, denominator and pair sum fused in one B200 kernel.

tsfast's ``LinearDynamicalOperator.forward`` (``tsfast/models/architectures/dynonet/core.py:199-250``)
runs a grouped ``conv1d`` for the FIR numerators (``[B, I*O, L]`` written), the all-pole scan on that
tensor (read and written again) and a sum over the input channels (read once more).  Here one
kernel, ``b200_gblock_fwd``, does all three per (batch row, output channel): the numerator output
never reaches memory and the per-pair outputs only when the adjoint will need them.

* :func:`linear_block` is the functional form: ``(u, b_coeff, a_coeff, state) -> (y, new_state)``
  with tsfast's tensor layouts and state dict (``{"u": FIR tail, "x": IIR states}``).  It is
  differentiable: the adjoint is ``b200_gblock_bwd`` (the all-pole adjoint of every pair reading the
  output gradient in place, then one kernel for the numerator's input and tap gradients).
* ``tsfast_b200.install(fuse_dynonet=True)`` routes tsfast's own ``LinearDynamicalOperator`` (and so
  its ``DynoNet``) through it.

float32 on CUDA, ``1 <= na <= 4`` and ``nb <= 16``; anything else raises (tsfast's own module is the
place for other shapes: this package has no second path).
"""

from __future__ import annotations

import torch

from . import _lib
from .allpole_b200 import _allpole_bwd_op

__all__ = ["linear_block", "supports"]

_MAX_NA = 4
_SPLIT_BELOW = 296  # (batch row, output) warps under which the forward runs one warp per filter: 2 per SM
_NB_SIZES = (4, 8, 16)


def supports(u: torch.Tensor, b_coeff: torch.Tensor, a_coeff: torch.Tensor) -> str | None:
    """Reason the fused kernel cannot take these tensors, or None when it can."""
    if u.device.type != "cuda":
        return "inputs not on CUDA"
    if any(t.dtype != torch.float32 for t in (u, b_coeff, a_coeff)):
        return "needs float32 tensors"
    if u.dim() != 3 or b_coeff.dim() != 3 or a_coeff.dim() != 3:
        return "expected u [B, L, I], b_coeff [O, I, nb], a_coeff [O, I, na]"
    if not 1 <= a_coeff.shape[-1] <= _MAX_NA:
        return f"na={a_coeff.shape[-1]} outside [1, {_MAX_NA}]"
    if not 1 <= b_coeff.shape[-1] <= _NB_SIZES[-1]:
        return f"nb={b_coeff.shape[-1]} outside [1, {_NB_SIZES[-1]}]"
    return None


def _padded_nb(nb: int) -> int:
    return next(s for s in _NB_SIZES if s >= nb)


def _rows_and_taps(u, tail, b_coeff, NB):
    """The kernels' input rows ``[B, I, pitch]`` (zeros, the carried tail, then ``u[b, :, j]``; one
    kernel, ``b200_gblock_pack_rows``) and the taps zero-padded to ``NB``."""
    B, L, I = u.shape
    O, _, nb = b_coeff.shape
    pitch = (L + NB - 1 + 3) // 4 * 4
    u_c = u.contiguous()
    tail_c = tail.contiguous() if (tail is not None and nb > 1) else None
    _lib.require_dense_cuda(u=u_c, tail=tail_c)
    ub = u.new_empty(B, I, pitch)
    if ub.numel():
        st = _lib.lib().b200_gblock_pack_rows(B, L, I, NB, nb, pitch, _lib.ptr(u_c), _lib.ptr(tail_c), _lib.ptr(ub),
                                              _lib.stream_ptr(u.device))
        _lib.check(st, "b200_gblock_pack_rows")
    if nb == NB:
        taps = b_coeff.clone(memory_format=torch.contiguous_format)  # an op output may not alias an input
    else:
        taps = b_coeff.new_zeros(O, I, NB)
        taps[:, :, :nb] = b_coeff
    return ub, taps, pitch


@torch.library.custom_op("b200scan::dynonet_gblock", mutates_args=())
def _gblock_op(u: torch.Tensor, tail: torch.Tensor | None, b_coeff: torch.Tensor, a_coeff: torch.Tensor,
               x0: torch.Tensor | None, keep_pairs: bool
               ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """``(y [B,O,L], y_pairs [B,I*O,L] or empty, x_last [B,I*O,na], rows, taps)`` for u [B,L,I]; the last
    two are the kernel's input rows and padded taps, handed back so that the adjoint can reuse them."""
    why = supports(u, b_coeff, a_coeff)
    if why is not None:
        raise RuntimeError(f"b200scan::dynonet_gblock: {why}")
    B, L, I = u.shape
    O, _, nb = b_coeff.shape
    na = a_coeff.shape[-1]
    NB = _padded_nb(nb)
    ub, taps, pitch = _rows_and_taps(u, tail, b_coeff, NB)
    a_c = a_coeff.contiguous()
    x0_c = x0.contiguous() if x0 is not None else None
    _lib.require_dense_cuda(ub=ub, taps=taps, a=a_c, x0=x0_c)
    # one warp per (batch row, output) walks all inputs; with too few of those to fill the GPU the
    # kernel runs one warp per filter instead, writes the per-pair outputs only, and they are summed here
    per_pair = I > 1 and B * O < _SPLIT_BELOW
    y = None if per_pair else u.new_empty(B, O, L)
    yp = u.new_empty(B, I * O, L) if (keep_pairs or per_pair) else u.new_empty(0)
    xl = u.new_empty(B, I * O, na)
    if B:
        st = _lib.lib().b200_gblock_fwd(B, L, I, O, na, NB, pitch, _lib.ptr(ub), _lib.ptr(taps), _lib.ptr(a_c),
                                        _lib.ptr(x0_c), _lib.ptr(y), _lib.ptr(yp) if yp.numel() else None,
                                        _lib.ptr(xl), _lib.stream_ptr(u.device))
        _lib.check(st, "b200_gblock_fwd")
    if per_pair:
        y = yp.view(B, I, O, L).sum(1)
        if not keep_pairs:
            yp = u.new_empty(0)
    return y, yp, xl, ub, taps


@_gblock_op.register_fake
def _(u, tail, b_coeff, a_coeff, x0, keep_pairs):
    B, L, I = u.shape
    O, na = b_coeff.shape[0], a_coeff.shape[-1]
    yp = u.new_empty(B, I * O, L) if keep_pairs else u.new_empty(0)
    NB = _padded_nb(b_coeff.shape[-1])
    return (u.new_empty(B, O, L), yp, u.new_empty(B, I * O, na), u.new_empty(B, I, (L + NB - 1 + 3) // 4 * 4),
            b_coeff.new_empty(O, I, NB))


@torch.library.custom_op("b200scan::dynonet_gblock_bwd", mutates_args=())
def _gblock_bwd_op(gy: torch.Tensor, ub: torch.Tensor, taps: torch.Tensor, a_coeff: torch.Tensor,
                   x0: torch.Tensor | None, yp: torch.Tensor, L: int, nb: int
                   ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients of ``sum(y * gy)``, gy [B,O,L], from the forward's rows and padded taps:
    ``(gu [B,L,I], gtail [B,nb-1,I], gb [O,I,nb], ga [O,I,na], gx0 [B,I*O,na] or empty)``."""
    u = ub
    B, I, pitch = ub.shape
    O, _, NB = taps.shape
    na = a_coeff.shape[-1]
    gy_c, a_c, yp_c = gy.contiguous(), a_coeff.contiguous(), yp.contiguous()
    x0_c = x0.contiguous() if x0 is not None else None
    _lib.require_dense_cuda(gy=gy_c, ub=ub, taps=taps, a=a_c, x0=x0_c, y_pairs=yp_c)
    # one warp per (batch row, input) walks all outputs; with too few of those the numerator adjoint
    # runs one warp per filter, writes one input-gradient row per pair, and they are summed here
    per_pair = O > 1 and B * I < _SPLIT_BELOW
    gub = u.new_empty(B, I * O if per_pair else I, pitch)
    gtaps = u.new_empty(B, O, I, NB)
    ga_l = u.new_empty(B, I * O, na)
    gx0 = u.new_empty(B, I * O, na) if x0 is not None else None
    if B:
        nbytes = _lib.lib().b200_gblock_bwd_workspace_bytes(B, L, I, O)
        ws = _lib.workspace(nbytes, u.device)
        st = _lib.lib().b200_gblock_bwd(B, L, I, O, na, NB, pitch, _lib.ptr(gy_c), _lib.ptr(ub), _lib.ptr(taps),
                                        _lib.ptr(a_c), _lib.ptr(yp_c), _lib.ptr(x0_c), _lib.ptr(gub), int(per_pair),
                                        _lib.ptr(gtaps), _lib.ptr(ga_l), _lib.ptr(gx0), _lib.ptr(ws), ws.numel(),
                                        _lib.stream_ptr(u.device))
        _lib.check(st, "b200_gblock_bwd")
    if per_pair:
        gub = gub.view(B, I, O, pitch).sum(2)
    gu = gub[:, :, NB - 1 : NB - 1 + L].transpose(1, 2).clone(memory_format=torch.contiguous_format)
    gtail = gub[:, :, NB - nb : NB - 1].transpose(1, 2).clone(memory_format=torch.contiguous_format)
    gb = gtaps.sum(0)[:, :, :nb].clone(memory_format=torch.contiguous_format)
    ga = ga_l.reshape(B, I, O, na).sum(0).permute(1, 0, 2).clone(memory_format=torch.contiguous_format)
    return gu, gtail, gb, ga, (gx0 if gx0 is not None else u.new_empty(0))


@_gblock_bwd_op.register_fake
def _(gy, ub, taps, a_coeff, x0, yp, L, nb):
    B, I, _ = ub.shape
    O = taps.shape[0]
    gx0 = torch.empty_like(x0) if x0 is not None else ub.new_empty(0)
    return ub.new_empty(B, L, I), ub.new_empty(B, nb - 1, I), taps.new_empty(O, I, nb), torch.empty_like(a_coeff), gx0


def _gblock_setup(ctx, inputs, output):
    u, tail, b_coeff, a_coeff, x0, keep_pairs = inputs
    _, yp, _, ub, taps = output
    ctx.keep_pairs = keep_pairs
    ctx.set_materialize_grads(False)
    ctx.save_for_backward(u, tail, b_coeff, a_coeff, x0, yp, ub, taps)


def _gblock_backward(ctx, gy, gyp, gxl, gub_unused, gtaps_unused):
    u, tail, b_coeff, a_coeff, x0, yp, ub, taps = ctx.saved_tensors
    if not ctx.keep_pairs:
        raise RuntimeError("b200scan::dynonet_gblock was run without keeping the per-pair outputs; "
                           "call linear_block under autograd so that it keeps them")
    B, L, I = u.shape
    if gyp is None and gxl is None:  # the usual case: only y is used downstream
        if gy is None:
            gy = u.new_zeros(B, b_coeff.shape[0], L)
        gu, gtail, gb, ga, gx0 = _gblock_bwd_op(gy, ub, taps, a_coeff, x0, yp, L, b_coeff.shape[-1])
        return gu, (gtail if tail is not None else None), gb, ga, (gx0 if x0 is not None else None), None
    return _gblock_backward_general(u, tail, b_coeff, a_coeff, x0, yp, gy, gyp, gxl)


def _gblock_backward_general(u, tail, b_coeff, a_coeff, x0, yp, gy, gyp, gxl):
    """Gradients when the per-pair outputs or the new state are differentiated too: the per-pair
    upstream gradient is built explicitly, then the all-pole adjoint and PyTorch's grouped
    convolution gradients."""
    B, L, I = u.shape
    O, _, nb = b_coeff.shape
    na = a_coeff.shape[-1]
    P = I * O
    if gy is None:
        gy = u.new_zeros(B, O, L)
    # upstream gradient of every pair: the output channel's gradient, plus what arrives through
    # the per-pair outputs and through the new state (x_last[k] = y_pairs[L-1-k])
    g_pairs = gy.unsqueeze(1).expand(B, I, O, L).reshape(B, P, L).clone()
    if gyp is not None and gyp.numel():
        g_pairs += gyp
    gx0_direct = None
    if gxl is not None:
        n_in = min(na, L)
        g_pairs[..., L - n_in :] += gxl[..., :n_in].flip(-1)
        if L < na and x0 is not None:  # the oldest entries of x_last are x0[: na - L]
            gx0_direct = torch.zeros_like(x0)
            gx0_direct[..., : na - L] = gxl[..., L:]
    a_pairs = a_coeff.permute(1, 0, 2).reshape(1, P, na).expand(B, P, na).reshape(B * P, na)
    y0 = x0.reshape(B * P, na) if x0 is not None else None
    ga_l, gw, gy0 = _allpole_bwd_op(g_pairs.reshape(B * P, L), a_pairs, yp.reshape(B * P, L), y0)
    ga = ga_l.reshape(B, I, O, na).sum(0).permute(1, 0, 2)
    # numerator: w = conv1d(cat(tail, u)^T, flipped taps, groups=I)
    ubuf = u if nb == 1 else torch.cat((tail if tail is not None else u.new_zeros(B, nb - 1, I), u), dim=1)
    ubuf_t = ubuf.transpose(1, 2)
    weight = b_coeff.permute(1, 0, 2).reshape(P, 1, nb).flip(-1)
    gw3 = gw.reshape(B, P, L)
    gub = torch.nn.grad.conv1d_input(ubuf_t.shape, weight, gw3, groups=I).transpose(1, 2)
    gweight = torch.nn.grad.conv1d_weight(ubuf_t, weight.shape, gw3, groups=I)
    gb = gweight.flip(-1).reshape(I, O, nb).permute(1, 0, 2)
    gu = gub[:, nb - 1 :]
    gtail = gub[:, : nb - 1] if tail is not None else None
    gx0 = None
    if x0 is not None:
        gx0 = gy0.reshape(B, P, na)
        if gx0_direct is not None:
            gx0 = gx0 + gx0_direct
    return gu, gtail, gb, ga, gx0, None


_gblock_op.register_autograd(_gblock_backward, setup_context=_gblock_setup)


def linear_block(u: torch.Tensor, b_coeff: torch.Tensor, a_coeff: torch.Tensor, state: dict | None = None):
    """``(y [B, L, O], new_state)`` of the G-block for ``u [B, L, I]``.

    ``state`` is tsfast's ``{"u": [B, nb-1, I] input tail, "x": [B, I*O, na] filter states}`` or
    None for zero initial conditions; ``new_state`` has the same form, so chunked calls continue a
    sequence exactly (``dynonet/core.py:214-252``).
    """
    match state:
        case {"u": tail, "x": x0}:
            pass
        case None:
            tail = x0 = None
        case _:
            raise TypeError(f"expected state dict {{'u': tensor, 'x': tensor}}, got {type(state)}")
    nb = b_coeff.shape[-1]
    keep = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (u, tail, b_coeff, a_coeff, x0))
    y, _, x_last, _, _ = _gblock_op(u, tail, b_coeff, a_coeff, x0, keep)
    B, L, I = u.shape
    if nb > 1:
        ubuf = torch.cat((tail if tail is not None else u.new_zeros(B, nb - 1, I), u[:, max(0, L - (nb - 1)) :]), dim=1)
        new_tail = ubuf[:, ubuf.shape[1] - (nb - 1) :]
    else:
        new_tail = u.new_zeros(B, 0, I)
    return y.transpose(1, 2), {"u": new_tail, "x": x_last}
