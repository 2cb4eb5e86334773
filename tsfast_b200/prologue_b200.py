"""Parameter prologues of tsfast's LRU and S5 layers on B200: one launch forward, one for the adjoint.

Between the stored parameters and the scan sit a few lines of parameter-sized math:
``LRU.eigenvalues()`` and the ``gamma`` scaling of ``B`` (``architectures/lru.py:79-83, 97-99``) and
``S5.discretize()`` (``architectures/s5.py:154-170``).  In PyTorch each is a dozen tiny kernels forward
and twice that in the backward pass, per layer and step.  This module computes

* ``lru_prologue(nu_log, theta_log, gamma_log, B_re, B_im) -> (lam [n] complex64, W [2n, d])``
* ``s5_discretize(Lambda_re, Lambda_im, log_step, B_re, B_im, *, discretization, clip_eigs, step_rescale)
  -> (lam_bar [p] complex64, W [2p, d])``

where ``W`` is the input-projection weight with interleaved (re, im) rows, the operand
``proj_b200.packed_in_proj(u, W)`` multiplies by.  Both are custom ops on ``libb200scan.so`` with
adjoints for every parameter and fake implementations; ``install(fuse_projections=True)`` routes
``LRU.forward`` and ``S5.forward`` through them.
"""

from __future__ import annotations

import torch

from . import _lib

__all__ = ["lru_prologue", "s5_discretize", "supports", "calls"]

calls = 0  # launches through this module since import (the drop-in tests read it)
_MODES = {"zoh": 0, "bilinear": 1}


def supports(*params: torch.Tensor) -> str | None:
    """Reason the kernels cannot take these parameters, or None when they can."""
    if not all(p.is_cuda and p.dtype == torch.float32 for p in params):
        return "needs float32 CUDA parameters"
    return None


def _demand(name: str, vecs, mats) -> tuple[int, int]:
    why = supports(*vecs, *mats)
    if why is not None:
        raise RuntimeError(f"b200scan::{name}: {why}")
    n = vecs[0].numel()
    d = mats[0].shape[1] if mats[0].dim() == 2 else -1
    if any(v.dim() != 1 or v.numel() != n for v in vecs) or any(tuple(m.shape) != (n, d) for m in mats):
        raise RuntimeError(f"b200scan::{name}: expected vectors [n] and matrices [n, d], got "
                           f"{[tuple(t.shape) for t in (*vecs, *mats)]}")
    return n, d


def _c(*ts):
    return tuple(t.contiguous() for t in ts)


# ------------------------------------------------------------------------------- LRU
@torch.library.custom_op("b200scan::lru_prologue", mutates_args=())
def _lru_op(nu_log: torch.Tensor, theta_log: torch.Tensor, gamma_log: torch.Tensor, B_re: torch.Tensor,
            B_im: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    global calls
    n, d = _demand("lru_prologue", (nu_log, theta_log, gamma_log), (B_re, B_im))
    nu_log, theta_log, gamma_log, B_re, B_im = _c(nu_log, theta_log, gamma_log, B_re, B_im)
    lam = torch.empty(n, dtype=torch.complex64, device=B_re.device)
    W = torch.empty(2 * n, d, dtype=torch.float32, device=B_re.device)
    calls += 1
    _lib.check(_lib.lib().b200_lru_prologue_fwd(n, d, _lib.ptr(nu_log), _lib.ptr(theta_log), _lib.ptr(gamma_log), _lib.ptr(B_re),
                                                _lib.ptr(B_im), _lib.ptr(lam), _lib.ptr(W), _lib.stream_ptr(B_re.device)),
               "b200_lru_prologue_fwd")
    return lam, W


@_lru_op.register_fake
def _(nu_log, theta_log, gamma_log, B_re, B_im):
    n, d = B_re.shape
    return nu_log.new_empty(n, dtype=torch.complex64), B_re.new_empty(2 * n, d)


@torch.library.custom_op("b200scan::lru_prologue_bwd", mutates_args=())
def _lru_bwd_op(glam: torch.Tensor | None, gW: torch.Tensor | None, nu_log: torch.Tensor, theta_log: torch.Tensor,
                gamma_log: torch.Tensor, B_re: torch.Tensor,
                B_im: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    global calls
    n, d = _demand("lru_prologue_bwd", (nu_log, theta_log, gamma_log), (B_re, B_im))
    nu_log, theta_log, gamma_log, B_re, B_im = _c(nu_log, theta_log, gamma_log, B_re, B_im)
    glam = None if glam is None else glam.contiguous()
    gW = None if gW is None else gW.contiguous()
    outs = (torch.empty_like(nu_log), torch.empty_like(nu_log), torch.empty_like(nu_log), torch.empty_like(B_re),
            torch.empty_like(B_re))
    calls += 1
    _lib.check(_lib.lib().b200_lru_prologue_bwd(n, d, _lib.ptr(nu_log), _lib.ptr(theta_log), _lib.ptr(gamma_log), _lib.ptr(B_re),
                                                _lib.ptr(B_im), _lib.ptr(glam), _lib.ptr(gW), *(_lib.ptr(t) for t in outs),
                                                _lib.stream_ptr(B_re.device)), "b200_lru_prologue_bwd")
    return outs


@_lru_bwd_op.register_fake
def _(glam, gW, nu_log, theta_log, gamma_log, B_re, B_im):
    return (torch.empty_like(nu_log), torch.empty_like(nu_log), torch.empty_like(nu_log), torch.empty_like(B_re),
            torch.empty_like(B_re))


def _lru_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _lru_adjoint(ctx, glam, gW):
    return _lru_bwd_op(glam, gW, *ctx.saved_tensors)


_lru_op.register_autograd(_lru_adjoint, setup_context=_lru_setup)


def lru_prologue(nu_log, theta_log, gamma_log, B_re, B_im):
    """``(lam [n] complex64, W [2n, d])``: the LRU eigenvalues and the gamma-scaled, interleaved ``B``."""
    return _lru_op(nu_log, theta_log, gamma_log, B_re, B_im)


# ------------------------------------------------------------------------------- S5
@torch.library.custom_op("b200scan::s5_discretize", mutates_args=())
def _s5_op(Lambda_re: torch.Tensor, Lambda_im: torch.Tensor, log_step: torch.Tensor, B_re: torch.Tensor, B_im: torch.Tensor,
           mode: int, clip_eigs: bool, step_rescale: float) -> tuple[torch.Tensor, torch.Tensor]:
    global calls
    p, d = _demand("s5_discretize", (Lambda_re, Lambda_im, log_step), (B_re, B_im))
    Lambda_re, Lambda_im, log_step, B_re, B_im = _c(Lambda_re, Lambda_im, log_step, B_re, B_im)
    lam_bar = torch.empty(p, dtype=torch.complex64, device=B_re.device)
    W = torch.empty(2 * p, d, dtype=torch.float32, device=B_re.device)
    calls += 1
    _lib.check(_lib.lib().b200_s5_discretize_fwd(p, d, int(mode), int(clip_eigs), float(step_rescale), _lib.ptr(Lambda_re),
                                                 _lib.ptr(Lambda_im), _lib.ptr(log_step), _lib.ptr(B_re), _lib.ptr(B_im),
                                                 _lib.ptr(lam_bar), _lib.ptr(W), _lib.stream_ptr(B_re.device)),
               "b200_s5_discretize_fwd")
    return lam_bar, W


@_s5_op.register_fake
def _(Lambda_re, Lambda_im, log_step, B_re, B_im, mode, clip_eigs, step_rescale):
    p, d = B_re.shape
    return Lambda_re.new_empty(p, dtype=torch.complex64), B_re.new_empty(2 * p, d)


@torch.library.custom_op("b200scan::s5_discretize_bwd", mutates_args=())
def _s5_bwd_op(glam: torch.Tensor | None, gW: torch.Tensor | None, Lambda_re: torch.Tensor, Lambda_im: torch.Tensor,
               log_step: torch.Tensor, B_re: torch.Tensor, B_im: torch.Tensor, mode: int, clip_eigs: bool,
               step_rescale: float) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    global calls
    p, d = _demand("s5_discretize_bwd", (Lambda_re, Lambda_im, log_step), (B_re, B_im))
    Lambda_re, Lambda_im, log_step, B_re, B_im = _c(Lambda_re, Lambda_im, log_step, B_re, B_im)
    glam = None if glam is None else glam.contiguous()
    gW = None if gW is None else gW.contiguous()
    outs = (torch.empty_like(Lambda_re), torch.empty_like(Lambda_re), torch.empty_like(Lambda_re), torch.empty_like(B_re),
            torch.empty_like(B_re))
    calls += 1
    _lib.check(_lib.lib().b200_s5_discretize_bwd(p, d, int(mode), int(clip_eigs), float(step_rescale), _lib.ptr(Lambda_re),
                                                 _lib.ptr(Lambda_im), _lib.ptr(log_step), _lib.ptr(B_re), _lib.ptr(B_im),
                                                 _lib.ptr(glam), _lib.ptr(gW), *(_lib.ptr(t) for t in outs),
                                                 _lib.stream_ptr(B_re.device)), "b200_s5_discretize_bwd")
    return outs


@_s5_bwd_op.register_fake
def _(glam, gW, Lambda_re, Lambda_im, log_step, B_re, B_im, mode, clip_eigs, step_rescale):
    return (torch.empty_like(Lambda_re), torch.empty_like(Lambda_re), torch.empty_like(Lambda_re), torch.empty_like(B_re),
            torch.empty_like(B_re))


def _s5_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs[:5])
    ctx.flags = inputs[5:]


def _s5_adjoint(ctx, glam, gW):
    return (*_s5_bwd_op(glam, gW, *ctx.saved_tensors, *ctx.flags), None, None, None)


_s5_op.register_autograd(_s5_adjoint, setup_context=_s5_setup)


def s5_discretize(Lambda_re, Lambda_im, log_step, B_re, B_im, *, discretization: str = "zoh", clip_eigs: bool = False,
                  step_rescale: float = 1.0):
    """``(lam_bar [p] complex64, W [2p, d])``: S5's discretised eigenvalues and interleaved ``B_bar``."""
    if discretization not in _MODES:
        raise ValueError(f"unknown discretization {discretization!r}")
    return _s5_op(Lambda_re, Lambda_im, log_step, B_re, B_im, _MODES[discretization], bool(clip_eigs), float(step_rescale))
