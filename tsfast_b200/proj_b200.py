"""Projections around the scans on B200's tensor cores.

tsfast's LRU and S5 layers enter and leave complex state space through two real GEMMs
(``complex_in_proj`` / ``real_out_proj``, ``tsfast/models/_core/scan.py:272-313``) and its Mamba layer
produces ``draw, B_t, C_t`` for the fused section with two more (``x_proj`` / ``dt_proj``,
``architectures/mamba/core.py:150-152``).  With the scans at HBM speed these products, run as float32
SIMT GEMMs over hundreds of thousands of tokens, are most of a training step.  This module runs them
on ``b200_proj_gemm`` / ``b200_proj_wgrad``: ``tcgen05`` TF32 MMAs fed by TMA with every operand split
into a TF32 head and tail, so the result is float32-faithful (no precision is traded, unlike
``allow_tf32``).

* ``linear(a, w, bias=None)`` – ``a [..., K] @ w [N, K]^T + bias``, differentiable in all three; the
  input gradient runs on the same kernel, the weight gradient (a reduction over all tokens) on the
  token-major variant, both deterministic;
* ``complex_in_proj(u, W_re, W_im)`` / ``real_out_proj(x, W_re, W_im)`` – drop-ins for tsfast's;
* ``readout(x, C_re, C_im, u, D)`` – ``Re(x C^T) + u D^T`` in one pass over the output;
* ``supports(a, w)`` – reason the kernel cannot take these tensors, or None.

``tsfast_b200.install(fuse_projections=True)`` points tsfast's LRU, S5 and Mamba modules at them.
"""

from __future__ import annotations

import torch

from . import _lib, glue_b200

__all__ = ["linear", "complex_in_proj", "packed_in_proj", "real_out_proj", "readout", "supports", "calls"]

calls = 0  # launches through this module since import (the drop-in tests read it)


def supports(a: torch.Tensor, w: torch.Tensor) -> str | None:
    """Reason ``linear(a, w)`` cannot run on the tensor-core kernel, or None when it can."""
    if not torch.cuda.is_available():
        return "no CUDA device is visible to this process"
    if a.device.type != "cuda" or w.device.type != "cuda":
        return "the kernels only read CUDA memory"
    if a.dtype != torch.float32 or w.dtype != torch.float32:
        return f"needs float32 operands, got {a.dtype} and {w.dtype}"
    if w.dim() != 2 or a.dim() < 1 or a.shape[-1] != w.shape[1]:
        return f"shapes {tuple(a.shape)} and {tuple(w.shape)} do not form a [..., K] x [N, K]^T product"
    if w.shape[0] < 1 or w.shape[1] < 1:
        return "empty weight"
    return None


def _rows(a: torch.Tensor) -> torch.Tensor:
    """``a`` as a 2-D matrix the kernel can read in place: unit column stride, row pitch a multiple of 4
    floats, 16-byte aligned base.  A view that does not qualify is copied into a buffer that does (its
    row pitch rounded up to 4 floats)."""
    a2 = a.reshape(-1, a.shape[-1])
    rows, k = a2.shape
    if a2.stride(1) == 1 and a2.stride(0) % 4 == 0 and a2.stride(0) >= k and a2.data_ptr() % 16 == 0:
        return a2
    if rows <= 1 and a2.is_contiguous() and a2.data_ptr() % 16 == 0:
        return a2.as_strided((rows, k), ((k + 3) // 4 * 4, 1))
    buf = torch.empty(rows, (k + 3) // 4 * 4, device=a.device, dtype=a.dtype)
    view = buf[:, :k]
    view.copy_(a2)
    return view


def _gemm(a1, b1, a2=None, b2=None, bias=None):
    global calls
    L_ = _lib.lib()
    m, k1 = a1.shape
    n = b1.shape[0]
    k2 = 0 if a2 is None else a2.shape[1]
    npad = (n + 3) // 4 * 4
    buf = torch.empty(m, npad, device=a1.device, dtype=torch.float32)
    out = buf[:, :n]
    if m == 0:
        return out
    ws = _lib.workspace(L_.b200_proj_gemm_workspace_bytes(n, k1, k2), a1.device)
    calls += 1
    rc = L_.b200_proj_gemm(m, n, k1, _lib.ptr(a1), a1.stride(0), _lib.ptr(b1), b1.stride(0), k2, _lib.ptr(a2),
                           0 if a2 is None else a2.stride(0), _lib.ptr(b2), 0 if b2 is None else b2.stride(0),
                           _lib.ptr(bias), _lib.ptr(buf), buf.stride(0), _lib.ptr(ws), ws.numel(), _lib.stream_ptr(a1.device))
    _lib.check(rc, "b200_proj_gemm")
    return out


def _wgrad(g, a):
    """``g [M, N]^T @ a [M, K]`` -> ``[N, K]``."""
    global calls
    L_ = _lib.lib()
    m, n = g.shape
    k = a.shape[1]
    dw = torch.empty(n, k, device=g.device, dtype=torch.float32)
    ws = _lib.workspace(L_.b200_proj_wgrad_workspace_bytes(m, n, k), g.device)
    calls += 1
    rc = L_.b200_proj_wgrad(m, n, k, _lib.ptr(g), g.stride(0), _lib.ptr(a), a.stride(0), _lib.ptr(dw), dw.stride(0),
                            _lib.ptr(ws), ws.numel(), _lib.stream_ptr(g.device))
    _lib.check(rc, "b200_proj_wgrad")
    return dw


def _guard(name, *pairs):
    for a, w in pairs:
        why = supports(a, w)
        if why is not None:
            raise RuntimeError(f"b200scan::{name}: {why}")


@torch.library.custom_op("b200scan::proj_gemm", mutates_args=())
def _proj_gemm_op(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    """``a [M, K] @ w [N, K]^T (+ bias [N])`` -> ``[M, N]``."""
    _guard("proj_gemm", (a, w))
    return _gemm(_rows(a), w.contiguous(), bias=None if bias is None else bias.contiguous())


@_proj_gemm_op.register_fake
def _(a, w, bias):
    n = w.shape[0]
    return a.new_empty(a.shape[0], (n + 3) // 4 * 4)[:, :n]


@torch.library.custom_op("b200scan::proj_gemm2", mutates_args=())
def _proj_gemm2_op(a1: torch.Tensor, w1: torch.Tensor, a2: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """``a1 @ w1^T + a2 @ w2^T`` in one pass over the output (readout plus feed-through)."""
    _guard("proj_gemm2", (a1, w1), (a2, w2))
    if a1.shape[0] != a2.shape[0] or w1.shape[0] != w2.shape[0]:
        raise RuntimeError("b200scan::proj_gemm2: the two products must have the same output shape")
    return _gemm(_rows(a1), w1.contiguous(), _rows(a2), w2.contiguous())


@_proj_gemm2_op.register_fake
def _(a1, w1, a2, w2):
    n = w1.shape[0]
    return a1.new_empty(a1.shape[0], (n + 3) // 4 * 4)[:, :n]


@torch.library.custom_op("b200scan::proj_wgrad", mutates_args=())
def _proj_wgrad_op(g: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
    """``g [M, N]^T @ a [M, K]`` -> ``[N, K]``: the weight gradient, reduced over all M tokens."""
    if g.dim() != 2 or a.dim() != 2 or g.shape[0] != a.shape[0]:
        raise RuntimeError(f"b200scan::proj_wgrad: {tuple(g.shape)} and {tuple(a.shape)} do not share a token axis")
    for t in (g, a):
        if t.device.type != "cuda" or t.dtype != torch.float32:
            raise RuntimeError("b200scan::proj_wgrad: needs float32 CUDA tensors")
    return _wgrad(_rows(g), _rows(a))


@_proj_wgrad_op.register_fake
def _(g, a):
    return g.new_empty(g.shape[1], a.shape[1])


def _input_grad(g: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``g [M, N] @ w [N, K]``: the same kernel with the transposed weight as its [rows = outputs] operand."""
    return _proj_gemm_op(g, w.t().contiguous(), None)


def _remember(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _adjoint(ctx, g):
    a, w, bias = ctx.saved_tensors
    need = ctx.needs_input_grad
    ga = _input_grad(g, w) if need[0] else None
    gw = _proj_wgrad_op(g, a) if need[1] else None
    gb = glue_b200.column_sums(g) if (bias is not None and need[2]) else None
    return ga, gw, gb


def _adjoint2(ctx, g):
    a1, w1, a2, w2 = ctx.saved_tensors
    need = ctx.needs_input_grad
    return (_input_grad(g, w1) if need[0] else None, _proj_wgrad_op(g, a1) if need[1] else None,
            _input_grad(g, w2) if need[2] else None, _proj_wgrad_op(g, a2) if need[3] else None)


_proj_gemm_op.register_autograd(_adjoint, setup_context=_remember)
_proj_gemm2_op.register_autograd(_adjoint2, setup_context=_remember)


def linear(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``a [..., K] @ w [N, K]^T + bias`` -> ``[..., N]`` (float32 CUDA), the contract of ``F.linear``."""
    return _proj_gemm_op(a.reshape(-1, a.shape[-1]), w, bias).reshape(*a.shape[:-1], w.shape[0])


def complex_in_proj(u: torch.Tensor, W_re: torch.Tensor, W_im: torch.Tensor) -> torch.Tensor:
    """``u @ (W_re + i W_im)^T`` for real ``u [..., d]`` and ``W [n, d]`` -> complex ``[..., n]``.

    The weight rows are interleaved (re, im) so that the real GEMM result already has
    ``view_as_complex``'s memory layout, as in tsfast's function of the same name."""
    n, d = W_re.shape
    w = torch.stack((W_re, W_im), dim=1).reshape(2 * n, d)
    return torch.view_as_complex(linear(u, w).unflatten(-1, (n, 2)))


def packed_in_proj(u: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
    """``complex_in_proj`` for a weight that already has the interleaved (re, im) row order ``[2n, d]``
    (what ``prologue_b200`` produces): real ``u [..., d]`` -> complex ``[..., n]``."""
    return torch.view_as_complex(linear(u, W).unflatten(-1, (W.shape[0] // 2, 2)))


def _readout_weight(W_re, W_im):
    out, n = W_re.shape
    return torch.stack((W_re, -W_im), dim=-1).reshape(out, 2 * n)


def real_out_proj(x: torch.Tensor, W_re: torch.Tensor, W_im: torch.Tensor) -> torch.Tensor:
    """``Re(x @ (W_re + i W_im)^T)`` for complex ``x [..., n]`` and ``W [out, n]`` -> real ``[..., out]``."""
    return linear(torch.view_as_real(x).flatten(-2), _readout_weight(W_re, W_im))


def readout(x: torch.Tensor, C_re: torch.Tensor, C_im: torch.Tensor, u: torch.Tensor, D: torch.Tensor) -> torch.Tensor:
    """``Re(x C^T) + u D^T``: the LRU layer's output map (``architectures/lru.py:107``), one pass over ``y``."""
    xr = torch.view_as_real(x).flatten(-2)
    y = _proj_gemm2_op(xr.reshape(-1, xr.shape[-1]), _readout_weight(C_re, C_im), u.reshape(-1, u.shape[-1]), D)
    return y.reshape(*u.shape[:-1], D.shape[0])
