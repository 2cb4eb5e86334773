"""B200 backend of the fused Mamba selective-scan section.

``h_t = exp(softplus(draw_t) A) h_{t-1} + softplus(draw_t) u_t B_t``,
``out_t = (h_t . C_t + Dp u_t) * silu(z_t)``, returning ``(out [B,L,D], h_last [B,D,N])``.

Drop-in for the reference's ``tsfast/models/architectures/mamba/mamba_triton.py`` (and the CPU
``backend_c.py``): the same ``supports(draw, A, Bt, Ct, u, z, Dp, h0)`` / ``run(...)`` protocol and
the same three custom ops (inference, training with state checkpoints, backward) with fake
implementations, under the ``b200scan`` namespace.  ``run`` is differentiable in all eight inputs
and in ``h_last``.  The kernels are ``b200_mamba_fwd`` / ``b200_mamba_bwd`` of ``libb200scan.so``;
the checkpoint interval (8 steps, as in the reference) is the library's: ``b200_mamba_chk_interval()``.
"""

from __future__ import annotations

import torch

from . import _lib

__all__ = ["supports", "run"]

_MAX_N = 128
_FAKE_CHK = 8  # checkpoint interval assumed by the fake (shape-only) implementations; checked against the library


def _chk_interval() -> int:
    k = int(_lib.lib().b200_mamba_chk_interval())
    if k != _FAKE_CHK:
        raise RuntimeError(f"libb200scan checkpoints every {k} steps, this module was written for {_FAKE_CHK}")
    return k


def supports(draw, A, Bt, Ct, u, z, Dp, h0) -> str | None:
    """Reason these tensors cannot be handled, or None when they can."""
    if not torch.cuda.is_available():
        return "CUDA not available"
    tensors = {"draw": draw, "A": A, "Bt": Bt, "Ct": Ct, "u": u, "z": z, "Dp": Dp}
    if h0 is not None:
        tensors["h0"] = h0
    for name, tt in tensors.items():
        if tt.device.type != "cuda":
            return f"{name} not on CUDA"
        if tt.dtype != torch.float32:
            return f"needs float32, got {name}={tt.dtype}"
    if draw.dim() != 3:
        return f"draw must be [B, L, D], got {draw.dim()} dims"
    B, L, D = draw.shape
    N = A.shape[-1]
    if tuple(A.shape) != (D, N):
        return f"A.shape {tuple(A.shape)} incompatible with draw {tuple(draw.shape)}"
    if not 1 <= N <= _MAX_N:
        return f"d_state={N} outside the supported range [1, {_MAX_N}]"
    if tuple(u.shape) != (B, L, D) or tuple(z.shape) != (B, L, D):
        return f"u/z shapes {tuple(u.shape)}/{tuple(z.shape)} != {(B, L, D)}"
    if tuple(Bt.shape) != (B, L, N) or tuple(Ct.shape) != (B, L, N):
        return f"Bt/Ct shapes {tuple(Bt.shape)}/{tuple(Ct.shape)} != {(B, L, N)}"
    if tuple(Dp.shape) != (D,):
        return f"Dp.shape {tuple(Dp.shape)} != {(D,)}"
    if h0 is not None and tuple(h0.shape) != (B, D, N):
        return f"h0.shape {tuple(h0.shape)} != {(B, D, N)}"
    return None


def _contig(*ts):
    return [t.contiguous() if t is not None else None for t in ts]


def _forward(draw, A, Bt, Ct, u, z, Dp, h0, store_chk: bool):
    reason = supports(draw, A, Bt, Ct, u, z, Dp, h0)
    if reason is not None:
        raise RuntimeError(f"b200scan::mamba_scan: {reason}")
    B, L, D = draw.shape
    N = A.shape[-1]
    out = torch.empty_like(draw)
    h_last = torch.empty(B, D, N, device=draw.device, dtype=draw.dtype)
    chk = None
    if store_chk:
        chk = torch.empty(B, -(-L // _chk_interval()), D, N, device=draw.device, dtype=draw.dtype)
    if B and D:
        st = _lib.lib().b200_mamba_fwd(B, L, D, N, *(map(_lib.ptr, (draw, A, Bt, Ct, u, z, Dp, h0, out, h_last, chk))),
                                       _lib.stream_ptr(draw.device))
        _lib.check(st, "b200_mamba_fwd")
    return out, h_last, chk


@torch.library.custom_op("b200scan::mamba_scan", mutates_args=())
def _scan_op(
    draw: torch.Tensor, A: torch.Tensor, Bt: torch.Tensor, Ct: torch.Tensor, u: torch.Tensor, z: torch.Tensor,
    Dp: torch.Tensor, h0: torch.Tensor | None,
) -> tuple[torch.Tensor, torch.Tensor]:
    out, h_last, _ = _forward(*_contig(draw, A, Bt, Ct, u, z, Dp, h0), store_chk=False)
    return out, h_last


@torch.library.custom_op("b200scan::mamba_scan_train", mutates_args=())
def _scan_train_op(
    draw: torch.Tensor, A: torch.Tensor, Bt: torch.Tensor, Ct: torch.Tensor, u: torch.Tensor, z: torch.Tensor,
    Dp: torch.Tensor, h0: torch.Tensor | None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return _forward(*_contig(draw, A, Bt, Ct, u, z, Dp, h0), store_chk=True)


def _fake_outs(draw, A, with_chk: bool):
    B, L, D = draw.shape
    N = A.shape[-1]
    out = torch.empty_like(draw)
    h_last = draw.new_empty(B, D, N)
    if not with_chk:
        return out, h_last
    return out, h_last, draw.new_empty(B, -(-L // _FAKE_CHK), D, N)


@_scan_op.register_fake
def _(draw, A, Bt, Ct, u, z, Dp, h0):
    return _fake_outs(draw, A, with_chk=False)


@_scan_train_op.register_fake
def _(draw, A, Bt, Ct, u, z, Dp, h0):
    return _fake_outs(draw, A, with_chk=True)


@torch.library.custom_op("b200scan::mamba_scan_bwd", mutates_args=())
def _scan_bwd_op(
    gout: torch.Tensor, ghlast: torch.Tensor | None, chk: torch.Tensor, draw: torch.Tensor, A: torch.Tensor,
    Bt: torch.Tensor, Ct: torch.Tensor, u: torch.Tensor, z: torch.Tensor, Dp: torch.Tensor, h0: torch.Tensor | None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
           torch.Tensor]:
    gout, ghlast, chk, draw, A, Bt, Ct, u, z, Dp, h0 = _contig(gout, ghlast, chk, draw, A, Bt, Ct, u, z, Dp, h0)
    _lib.require_dense_cuda(gout=gout, ghlast=ghlast, chk=chk)
    B, L, D = draw.shape
    N = A.shape[-1]
    new = lambda *s: torch.empty(*s, device=draw.device, dtype=draw.dtype)  # noqa: E731
    gdraw, gu, gz = torch.empty_like(draw), torch.empty_like(draw), torch.empty_like(draw)
    gA, gBt, gCt, gDp = new(D, N), new(B, L, N), new(B, L, N), new(D)
    gh0 = new(B, D, N) if h0 is not None else None
    if B and D:
        L_ = _lib.lib()
        ws = _lib.workspace(L_.b200_mamba_bwd_workspace_bytes(B, L, D, N), draw.device)
        st = L_.b200_mamba_bwd(
            B, L, D, N,
            *(map(_lib.ptr, (draw, A, Bt, Ct, u, z, Dp, h0, chk, gout, ghlast, gdraw, gA, gBt, gCt, gu, gz, gDp, gh0, ws))),
            ws.numel(), _lib.stream_ptr(draw.device))
        _lib.check(st, "b200_mamba_bwd")
    else:
        gA.zero_(), gDp.zero_()
    return gdraw, gA, gBt, gCt, gu, gz, gDp, (gh0 if gh0 is not None else gout.new_empty(0))


@_scan_bwd_op.register_fake
def _(gout, ghlast, chk, draw, A, Bt, Ct, u, z, Dp, h0):
    B, L, D = draw.shape
    N = A.shape[-1]
    return (torch.empty_like(draw), draw.new_empty(D, N), draw.new_empty(B, L, N), draw.new_empty(B, L, N),
            torch.empty_like(draw), torch.empty_like(draw), draw.new_empty(D),
            (draw.new_empty(B, D, N) if h0 is not None else draw.new_empty(0)))


def _scan_setup(ctx, inputs, output):
    draw, A, Bt, Ct, u, z, Dp, h0 = inputs
    ctx.save_for_backward(draw, A, Bt, Ct, u, z, Dp, h0, output[2])


def _scan_backward(ctx, gout, ghlast, gchk):
    draw, A, Bt, Ct, u, z, Dp, h0, chk = ctx.saved_tensors
    if gout is None:
        gout = torch.zeros_like(draw)
    gdraw, gA, gBt, gCt, gu, gz, gDp, gh0 = _scan_bwd_op(gout, ghlast, chk, draw, A, Bt, Ct, u, z, Dp, h0)
    return gdraw, gA, gBt, gCt, gu, gz, gDp, (gh0 if h0 is not None else None)


_scan_train_op.register_autograd(_scan_backward, setup_context=_scan_setup)


def run(draw, A, Bt, Ct, u, z, Dp, h0):
    """Fused section → ``(out [B, L, D], h_last [B, D, N])``; differentiable in every input and in ``h_last``."""
    inputs = (draw, A, Bt, Ct, u, z, Dp) + ((h0,) if h0 is not None else ())
    if not torch.is_grad_enabled() or not any(t.requires_grad for t in inputs):
        return _scan_op(draw, A, Bt, Ct, u, z, Dp, h0)
    out, h_last, _chk = _scan_train_op(draw, A, Bt, Ct, u, z, Dp, h0)
    return out, h_last
