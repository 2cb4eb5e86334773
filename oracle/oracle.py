"""TEST INFRASTRUCTURE: ctypes binding of ``liboracle.so`` on numpy arrays.

Every wrapper takes and returns numpy arrays (float32/float64, or complex64/complex128 for the
complex diagonal scans) in the layouts of the reference ops: diagonal ``lam [M,N]``,
``v [M,L,N]``; selective ``lam, v [B,L,N]``; Mamba ``draw/u/z [B,L,D]``, ``A [D,N]``,
``Bt/Ct [B,L,N]``; all-pole ``a [lanes,na]``, ``w [lanes,L]``.  The precision of the oracle run
follows the dtype of the arrays handed in.
"""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = None


def build(force: bool = False) -> Path:
    """Compile ``liboracle.so`` with the Makefile beside this file (no-op when up to date)."""
    if force:
        subprocess.run(["make", "-C", str(_HERE), "clean"], check=True, capture_output=True)
    subprocess.run(["make", "-C", str(_HERE)], check=True, capture_output=True)
    return _HERE / "liboracle.so"


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = _HERE / "liboracle.so"
        if not path.exists():
            build()
        _LIB = ctypes.CDLL(str(path))
        _LIB.oracle_num_threads.restype = ctypes.c_int
    return _LIB


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(ctypes.c_int(n))


def _real_dtype(x: np.ndarray):
    return {np.dtype("float32"): np.float32, np.dtype("complex64"): np.float32,
            np.dtype("float64"): np.float64, np.dtype("complex128"): np.float64}[x.dtype]


def _sfx(x: np.ndarray) -> str:
    return "f32" if _real_dtype(x) is np.float32 else "f64"


def _c(x):
    return None if x is None else np.ascontiguousarray(x)


def _p(x):
    return ctypes.c_void_p(None if x is None else x.ctypes.data)


def _call(name, sfx, ints, ptrs):
    fn = getattr(lib(), f"oracle_{name}_{sfx}")
    fn.restype = None
    fn(*[ctypes.c_int64(i) for i in ints[0]], *[ctypes.c_int(i) for i in ints[1]], *[_p(p) for p in ptrs])


# ------------------------------------------------------------------ S1 / S2
def _diag_like(name, lam, v, x0):
    lam, v, x0 = _c(lam), _c(v), _c(x0)
    M, L, N = v.shape
    out = np.empty_like(v)
    _call(name, _sfx(v), ((M, L, N), (int(np.iscomplexobj(v)),)), (lam, v, x0, out))
    return out


def _diag_like_bwd(name, g, lam, out, x0):
    g, lam, out, x0 = _c(g), _c(lam), _c(out), _c(x0)
    M, L, N = out.shape
    glam = np.empty_like(lam)
    gv = np.empty_like(out)
    gx0 = np.empty_like(x0) if x0 is not None else None
    _call(name, _sfx(out), ((M, L, N), (int(np.iscomplexobj(out)),)), (g, lam, out, x0, glam, gv, gx0))
    return glam, gv, gx0


def diag_fwd(lam, v, x0=None):
    """S1 forward: ``lam [M,N]`` constant over time."""
    return _diag_like("diag_fwd", lam, v, x0)


def diag_bwd(g, lam, out, x0=None):
    """S1 adjoint → ``(glam [M,N], gv [M,L,N], gx0 [M,N] | None)``."""
    return _diag_like_bwd("diag_bwd", g, lam, out, x0)


def sel_fwd(lam, v, x0=None):
    """S2 forward: ``lam [B,L,N]`` time-varying."""
    return _diag_like("sel_fwd", lam, v, x0)


def sel_bwd(g, lam, out, x0=None):
    """S2 adjoint → ``(glam [B,L,N], gv [B,L,N], gx0 [B,N] | None)``."""
    return _diag_like_bwd("sel_bwd", g, lam, out, x0)


# ------------------------------------------------------------------ S3
def mamba_fwd(draw, A, Bt, Ct, u, z, Dp, h0=None):
    draw, A, Bt, Ct, u, z, Dp, h0 = map(_c, (draw, A, Bt, Ct, u, z, Dp, h0))
    B, L, D = draw.shape
    N = A.shape[-1]
    assert N <= 256
    out = np.empty_like(draw)
    hlast = np.empty((B, D, N), dtype=draw.dtype)
    _call("mamba_fwd", _sfx(draw), ((B, L, D, N), ()), (draw, A, Bt, Ct, u, z, Dp, h0, out, hlast))
    return out, hlast


def mamba_bwd(draw, A, Bt, Ct, u, z, Dp, h0, gout, ghlast=None):
    """S3 adjoint → dict with gdraw, gA, gBt, gCt, gu, gz, gDp, gh0 (None without h0)."""
    draw, A, Bt, Ct, u, z, Dp, h0, gout, ghlast = map(_c, (draw, A, Bt, Ct, u, z, Dp, h0, gout, ghlast))
    B, L, D = draw.shape
    N = A.shape[-1]
    dt = draw.dtype
    r = dict(gdraw=np.empty_like(draw), gA=np.empty((D, N), dt), gBt=np.empty((B, L, N), dt),
             gCt=np.empty((B, L, N), dt), gu=np.empty_like(draw), gz=np.empty_like(draw),
             gDp=np.empty((D,), dt), gh0=(np.empty((B, D, N), dt) if h0 is not None else None))
    _call("mamba_bwd", _sfx(draw), ((B, L, D, N), ()),
          (draw, A, Bt, Ct, u, z, Dp, h0, gout, ghlast, r["gdraw"], r["gA"], r["gBt"], r["gCt"],
           r["gu"], r["gz"], r["gDp"], r["gh0"]))
    return r


# ------------------------------------------------------------------ S4
def allpole_fwd(a, w, y0=None):
    a, w, y0 = _c(a), _c(w), _c(y0)
    lanes, L = w.shape
    na = a.shape[-1]
    assert 1 <= na <= 16
    y = np.empty_like(w)
    _call("allpole_fwd", _sfx(w), ((lanes, L, na), ()), (a, w, y0, y))
    return y


def allpole_bwd(g, a, y, y0=None):
    """S4 adjoint → ``(grad_a [lanes,na], gw [lanes,L], grad_y0 [lanes,na] | None)``."""
    g, a, y, y0 = _c(g), _c(a), _c(y), _c(y0)
    lanes, L = y.shape
    na = a.shape[-1]
    ga = np.empty_like(a)
    gw = np.empty_like(y)
    gy0 = np.empty_like(y0) if y0 is not None else None
    _call("allpole_bwd", _sfx(y), ((lanes, L, na), ()), (g, a, y, y0, ga, gw, gy0))
    return ga, gw, gy0


# ------------------------------------------------------------------ dynoNet G-block (FIR + all-pole + pair sum)
def gblock_fwd(u, b_coeff, a_coeff, u_tail=None, x0=None):
    """``LinearDynamicalOperator.forward`` of tsfast/models/architectures/dynonet/core.py:199-250.

    u [B,L,I], b_coeff [O,I,nb], a_coeff [O,I,na], u_tail [B,nb-1,I] or None, x0 [B,I*O,na] or None
    (pair index j*O + i, newest output first).  Returns ``(y [B,L,O], y_pairs [B,I*O,L],
    x_last [B,I*O,na], new_tail [B,nb-1,I])``: the numerator is the causal FIR
    ``w_t = sum_k b_k u_{t-k}`` on ``cat(u_tail, u)`` (:214-220), the denominator the all-pole
    recurrence (:228-231), ``x_last`` the last ``na`` outputs reversed, padded from ``x0`` when the
    chunk is shorter than ``na`` (:240-246), and the output the sum over inputs (:250).
    """
    u, b_coeff, a_coeff = _c(u), _c(b_coeff), _c(a_coeff)
    B, L, I = u.shape
    O, _, nb = b_coeff.shape
    na = a_coeff.shape[-1]
    P = I * O
    dt = u.dtype
    tail = np.zeros((B, nb - 1, I), dt) if u_tail is None else np.asarray(u_tail, dt)
    ubuf = np.concatenate((tail, u), axis=1)  # [B, L+nb-1, I]
    w = np.zeros((B, P, L), dt)
    for j in range(I):
        for i in range(O):
            acc = np.zeros((B, L), dt)
            for k in range(nb):
                acc += b_coeff[i, j, k] * ubuf[:, nb - 1 - k : nb - 1 - k + L, j]
            w[:, j * O + i] = acc
    a_pairs = np.ascontiguousarray(np.broadcast_to(a_coeff.transpose(1, 0, 2).reshape(1, P, na), (B, P, na))).reshape(B * P, na)
    y0 = None if x0 is None else np.ascontiguousarray(np.asarray(x0, dt)).reshape(B * P, na)
    yp = allpole_fwd(a_pairs, w.reshape(B * P, L), y0).reshape(B, P, L)
    y = yp.reshape(B, I, O, L).sum(1).transpose(0, 2, 1)
    x0z = np.zeros((B, P, na), dt) if x0 is None else np.asarray(x0, dt)
    hist = np.concatenate((x0z[..., ::-1], yp), axis=-1)  # oldest .. newest
    x_last = np.ascontiguousarray(hist[..., ::-1][..., :na])
    new_tail = ubuf[:, ubuf.shape[1] - (nb - 1) :]
    return np.ascontiguousarray(y), yp, x_last, np.ascontiguousarray(new_tail)


def gblock_bwd(gy, u, b_coeff, a_coeff, y_pairs, u_tail=None, x0=None):
    """Adjoint of ``gblock_fwd`` for an upstream gradient on ``y`` only: returns
    ``(gu [B,L,I], gb [O,I,nb], ga [O,I,na], gu_tail [B,nb-1,I], gx0 [B,I*O,na] | None)``."""
    gy, u, b_coeff, a_coeff, y_pairs = _c(gy), _c(u), _c(b_coeff), _c(a_coeff), _c(y_pairs)
    B, L, I = u.shape
    O, _, nb = b_coeff.shape
    na = a_coeff.shape[-1]
    P = I * O
    dt = u.dtype
    g_pairs = np.ascontiguousarray(np.broadcast_to(gy.transpose(0, 2, 1)[:, None], (B, I, O, L))).reshape(B * P, L)
    a_pairs = np.ascontiguousarray(np.broadcast_to(a_coeff.transpose(1, 0, 2).reshape(1, P, na), (B, P, na))).reshape(B * P, na)
    y0 = None if x0 is None else np.ascontiguousarray(np.asarray(x0, dt)).reshape(B * P, na)
    ga_l, gw, gy0 = allpole_bwd(g_pairs, a_pairs, y_pairs.reshape(B * P, L), y0)
    gw = gw.reshape(B, I, O, L)
    tail = np.zeros((B, nb - 1, I), dt) if u_tail is None else np.asarray(u_tail, dt)
    ubuf = np.concatenate((tail, u), axis=1)
    gubuf = np.zeros_like(ubuf)
    gb = np.zeros_like(b_coeff)
    for j in range(I):
        for i in range(O):
            for k in range(nb):
                seg = slice(nb - 1 - k, nb - 1 - k + L)
                gb[i, j, k] = np.sum(gw[:, j, i] * ubuf[:, seg, j])
                gubuf[:, seg, j] += b_coeff[i, j, k] * gw[:, j, i]
    ga = ga_l.reshape(B, I, O, na).sum(0).transpose(1, 0, 2)
    gx0 = None if gy0 is None else gy0.reshape(B, P, na)
    return np.ascontiguousarray(gubuf[:, nb - 1 :]), gb, np.ascontiguousarray(ga), np.ascontiguousarray(gubuf[:, : nb - 1]), gx0


# ------------------------------------------------------------------ Mamba causal conv + SiLU
def conv_fwd(x, tail, w, bias=None):
    """``silu(conv1d(cat(tail, x)))`` depthwise and causal: x [B,L,D], tail [B,D,K-1], w [D,K], bias [D]."""
    x, tail, w, bias = _c(x), _c(tail), _c(w), _c(bias)
    B, L, D = x.shape
    K = w.shape[-1]
    out = np.empty_like(x)
    _call("conv_fwd", _sfx(x), ((B, L, D, K), ()), (x, tail, w, bias, out))
    return out


def conv_bwd(gy, x, tail, w, bias=None):
    """Adjoint → ``(gx [B,L,D], gtail [B,D,K-1], gw [D,K], gb [D] | None)``."""
    gy, x, tail, w, bias = _c(gy), _c(x), _c(tail), _c(w), _c(bias)
    B, L, D = x.shape
    K = w.shape[-1]
    gx, gtail, gw = np.empty_like(x), np.empty_like(tail), np.empty_like(w)
    gb = np.empty_like(bias) if bias is not None else None
    _call("conv_bwd", _sfx(x), ((B, L, D, K), ()), (gy, x, tail, w, bias, gx, gtail, gw, gb))
    return gx, gtail, gw, gb
