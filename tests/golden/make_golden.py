"""Generate the golden fixtures in this folder by running the reference (tsfast) itself.

Run where the reference checkout is importable, e.g.::

    CXX=/usr/bin/g++ CC=/usr/bin/gcc PYTHONPATH=<tsfast checkout> python tests/golden/make_golden.py

Every case draws float32 inputs from a seeded generator, then evaluates the reference twice:

* ``ref64_*``: the reference's pure-PyTorch path (``use_backend("reference")``: the doubling scans
  of ``tsfast/models/_core/scan.py``, the unfused Mamba section of
  ``tsfast/models/architectures/mamba/core.py:159-173`` and the companion-matrix
  ``linear_recurrence`` of ``tsfast/models/architectures/dynonet/core.py``) in float64 /
  complex128 on the same values, gradients by the reference's own registered adjoints;
* ``c32_*``: the reference's generated-C++ CPU backends in float32 where one exists
  (``diagonal_c``, ``selective_c``, ``mamba/backend_c``), to record the float32 noise floor.

Only the forward output of the float32 runs is kept.  Inputs and results go to one compressed
``.npz`` per scan.  The fixtures are small (about 4 MB in total) and committed; tests read them without needing the reference.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

os.environ.setdefault("CXX", "/usr/bin/g++")
os.environ.setdefault("CC", "/usr/bin/gcc")

import tsfast.models._core.scan as scan  # noqa: E402
from tsfast.models import use_backend  # noqa: E402
from tsfast.models.architectures.dynonet import linear_recurrence  # noqa: E402
from tsfast.models.architectures.mamba import backend_c as mamba_c  # noqa: E402

HERE = Path(__file__).resolve().parent


def _np(t):
    return None if t is None else t.detach().cpu().numpy()


def _to64(t):
    if t is None:
        return None
    return t.to(torch.complex128 if t.is_complex() else torch.float64)


def _leaf(t):
    return None if t is None else t.clone().requires_grad_()


# ------------------------------------------------------------------ S1 / S2
def _diag_inputs(gen, kind, v_shape, lam_shape, cplx, with_x0, c1_style=False):
    M, L, N = v_shape
    if kind == "diag":
        if c1_style:  # the BASELINE config-1 distribution
            r = torch.rand(*lam_shape, generator=gen) * 0.099 + 0.9
            th = torch.rand(*lam_shape, generator=gen) * (np.pi / 10)
            lam = (r * torch.exp(1j * th)).to(torch.complex64)
        else:
            lam = torch.rand(*lam_shape, generator=gen) * 0.85
            if cplx:
                lam = lam * torch.exp(1j * torch.rand(*lam_shape, generator=gen) * 3.0)
    else:
        lam = torch.rand(*v_shape, generator=gen) * 0.9 + 0.05
        if cplx:
            lam = lam * torch.exp(1j * torch.rand(*v_shape, generator=gen) * 3.0)
    v = torch.randn(*v_shape, generator=gen)
    g = torch.randn(*v_shape, generator=gen)
    x0 = torch.randn(M, N, generator=gen) if with_x0 else None
    if cplx:
        v = v + 1j * torch.randn(*v_shape, generator=gen)
        g = g + 1j * torch.randn(*v_shape, generator=gen)
        if with_x0:
            x0 = x0 + 1j * torch.randn(M, N, generator=gen)
        lam, v, g = lam.to(torch.complex64), v.to(torch.complex64), g.to(torch.complex64)
        x0 = None if x0 is None else x0.to(torch.complex64)
    return lam, v, x0, g


def _run_diag(fn, backend, lam, v, x0, g):
    lam_, v_, x0_ = _leaf(lam), _leaf(v), _leaf(x0)
    with use_backend(backend):
        out = fn(lam_, v_, x0_)
        out.backward(g)
    return out, lam_.grad, v_.grad, (None if x0 is None else x0_.grad)


def make_diag(kind):
    fn = scan.diagonal_recurrence if kind == "diag" else scan.selective_recurrence
    ALL = [(False, True), (False, False), (True, True), (True, False)]  # (complex, with_x0)
    if kind == "diag":
        cases = [((2, 7, 3), (3,), ALL), ((3, 1, 6), (6,), ALL), ((2, 257, 8), (2, 8), [(True, True), (False, False)]),
                 ((2, 50, 16), (16,), [(False, True), (True, False)]), ((1, 260, 24), (24,), [(True, True), (False, False)]),
                 ((1, 40, 100), (100,), [(False, True), (True, False)])]
    else:
        cases = [((2, 7, 3), None, ALL), ((2, 1, 3), None, ALL),
                 ((2, 257, 8), None, [(False, True), (True, False)]),
                 ((1, 130, 36), None, [(True, True), (False, False)])]
    store = {}
    names = []
    idx = 0
    for v_shape, lam_shape, variants in cases:
        for cplx, with_x0 in variants:
            gen = torch.Generator().manual_seed(1000 + idx)
            lam, v, x0, g = _diag_inputs(gen, kind, v_shape, lam_shape, cplx, with_x0)
            name = f"case{idx}"
            idx += 1
            names.append(name)
            r64 = _run_diag(fn, "reference", _to64(lam), _to64(v), _to64(x0), _to64(g))
            store.update({f"{name}_lam": _np(lam), f"{name}_v": _np(v), f"{name}_g": _np(g)})
            if x0 is not None:
                store[f"{name}_x0"] = _np(x0)
            for lbl, t in zip(("out", "glam", "gv", "gx0"), r64):
                if t is not None:
                    store[f"{name}_ref64_{lbl}"] = _np(t)
            if not (kind == "sel" and cplx):  # selective_c is float32-only
                c32 = _run_diag(fn, "c", lam, v, x0, g)
                store[f"{name}_c32_out"] = _np(c32[0])
    if kind == "diag":  # one case with the config-1 value distribution (complex, carry-in)
        gen = torch.Generator().manual_seed(0)
        lam, v, x0, g = _diag_inputs(gen, kind, (2, 100, 32), (32,), True, True, c1_style=True)
        x0 = (x0 * (0.1**0.5)).to(torch.complex64)
        name = f"case{idx}"
        names.append(name)
        r64 = _run_diag(fn, "reference", _to64(lam), _to64(v), _to64(x0), _to64(g))
        c32 = _run_diag(fn, "c", lam, v, x0, g)
        store.update({f"{name}_lam": _np(lam), f"{name}_v": _np(v), f"{name}_g": _np(g), f"{name}_x0": _np(x0)})
        for lbl, t in zip(("out", "glam", "gv", "gx0"), r64):
            store[f"{name}_ref64_{lbl}"] = _np(t)
        store[f"{name}_c32_out"] = _np(c32[0])
    store["names"] = np.array(names)
    np.savez_compressed(HERE / f"{kind}.npz", **store)
    print(kind, len(names), "cases")


# ------------------------------------------------------------------ S3
def _mamba_generic(draw, A, Bt, Ct, u, z, Dp, h0):
    """The unfused section exactly as MambaLayer._ssm spells it (mamba/core.py:159-173)."""
    Bsz, L, D = draw.shape
    N = A.shape[-1]
    delta = F.softplus(draw)
    lam = torch.exp(delta.unsqueeze(-1) * A)
    v = (delta * u).unsqueeze(-1) * Bt.unsqueeze(-2)
    h0f = None if h0 is None else h0.reshape(Bsz, D * N)
    with use_backend("reference"):
        h = scan.selective_recurrence(lam.flatten(-2), v.flatten(-2), h0f)
    y = (h.view(Bsz, L, D, N) * Ct.unsqueeze(-2)).sum(-1)
    return (y + Dp * u) * F.silu(z), h[..., -1, :].reshape(Bsz, D, N)


def make_mamba():
    ALL = [(True, True), (True, False), (False, True), (False, False)]  # (with_h0, with_glast)
    cases = [((2, 19, 20, 12), ALL), ((2, 33, 8, 16), ALL), ((1, 1, 4, 4), ALL), ((2, 8, 16, 5), ALL),
             ((2, 70, 33, 16), [(True, True), (False, False)])]
    store, names, idx = {}, [], 0
    for (Bsz, L, D, N), variants in cases:
        for with_h0, with_glast in variants:
            gen = torch.Generator().manual_seed(2000 + idx)
            rn = lambda *s: torch.randn(*s, generator=gen)  # noqa: E731
            draw = rn(Bsz, L, D) * 0.5 - 1.0
            A = -torch.exp(rn(D, N) * 0.5)
            Bt, Ct, u, z = rn(Bsz, L, N), rn(Bsz, L, N), rn(Bsz, L, D), rn(Bsz, L, D)
            Dp = rn(D)
            h0 = rn(Bsz, D, N) if with_h0 else None
            gout = rn(Bsz, L, D)
            ghl = rn(Bsz, D, N) if with_glast else None
            name = f"case{idx}"
            idx += 1
            names.append(name)
            ins = dict(draw=draw, A=A, Bt=Bt, Ct=Ct, u=u, z=z, Dp=Dp)
            for k, t in ins.items():
                store[f"{name}_{k}"] = _np(t)
            store[f"{name}_gout"] = _np(gout)
            if with_h0:
                store[f"{name}_h0"] = _np(h0)
            if with_glast:
                store[f"{name}_ghlast"] = _np(ghl)
            for tag, fn, cast in (("ref64", _mamba_generic, _to64), ("c32", mamba_c.run, lambda t: t)):
                leaves = [_leaf(cast(t)) for t in (draw, A, Bt, Ct, u, z, Dp)]
                h0_ = _leaf(cast(h0))
                out, hl = fn(*leaves, h0_)
                loss = (out * cast(gout)).sum()
                if with_glast:
                    loss = loss + (hl * cast(ghl)).sum()
                loss.backward()
                store[f"{name}_{tag}_out"] = _np(out)
                store[f"{name}_{tag}_hlast"] = _np(hl)
                if tag == "c32":
                    continue
                for k, t in zip(("gdraw", "gA", "gBt", "gCt", "gu", "gz", "gDp"), leaves):
                    store[f"{name}_{tag}_{k}"] = _np(t.grad)
                if with_h0:
                    store[f"{name}_{tag}_gh0"] = _np(h0_.grad)
    store["names"] = np.array(names)
    np.savez_compressed(HERE / "mamba.npz", **store)
    print("mamba", len(names), "cases")


# ------------------------------------------------------------------ S4
def _companion(a):
    na = a.shape[-1]
    shift = torch.eye(na, dtype=a.dtype)[:-1].expand(a.shape[0], na - 1, na)
    return torch.cat((-a.unsqueeze(1), shift), dim=1)


def _allpole_ref(a, w, y0):
    """Companion-matrix scan of the same filter, as tests/test_scan_allpole_backend.py:48-51."""
    x = linear_recurrence(_companion(a), F.pad(w.unsqueeze(-1), (0, a.shape[-1] - 1)), y0)
    return x[..., 0]


def make_allpole():
    cases = [(3, 5, 7, 3), (2, 4, 1, 2), (2, 4, 2, 4), (1, 1, 513, 1), (4, 8, 100, 8), (2, 3, 300, 16),
             (2, 6, 200, 4)]
    store, names, idx = {}, [], 0
    for (Bsz, P, L, na) in cases:
        for with_y0 in (True, False):
            gen = torch.Generator().manual_seed(3000 + idx)
            lanes = Bsz * P
            if (Bsz, P, L, na) == (2, 6, 200, 4):  # the config-4 pole distribution
                r = torch.rand(lanes, 2, generator=gen) * 0.45 + 0.5
                th = torch.rand(lanes, 2, generator=gen) * np.pi
                a = torch.zeros(lanes, 4, dtype=torch.float64)
                for i in range(lanes):
                    p = np.poly1d([1.0])
                    for k in range(2):
                        p = p * np.poly1d([1.0, -2 * float(r[i, k]) * np.cos(float(th[i, k])), float(r[i, k]) ** 2])
                    a[i] = torch.tensor(p.coeffs[1:])
                a = a.float()
            else:
                a = torch.randn(lanes, na, generator=gen) * (0.25 if na <= 8 else 0.1)
            w = torch.randn(lanes, L, generator=gen)
            g = torch.randn(lanes, L, generator=gen)
            y0 = torch.randn(lanes, na, generator=gen) if with_y0 else None
            name = f"case{idx}"
            idx += 1
            names.append(name)
            a_, w_, y0_ = _leaf(_to64(a)), _leaf(_to64(w)), _leaf(_to64(y0))
            y = _allpole_ref(a_, w_, y0_)
            y.backward(_to64(g))
            store.update({f"{name}_a": _np(a), f"{name}_w": _np(w), f"{name}_g": _np(g),
                          f"{name}_ref64_y": _np(y), f"{name}_ref64_ga": _np(a_.grad), f"{name}_ref64_gw": _np(w_.grad)})
            if with_y0:
                store[f"{name}_y0"] = _np(y0)
                store[f"{name}_ref64_gy0"] = _np(y0_.grad)
    store["names"] = np.array(names)
    np.savez_compressed(HERE / "allpole.npz", **store)
    print("allpole", len(names), "cases")


# ------------------------------------------------------------------ DeepLRU caller stack
def make_lru():
    """A small reference DeepLRU (tsfast/models/architectures/lru.py) in float64: parameters,
    input, output, carried states, and the gradient of sum(y * g) w.r.t. every parameter."""
    from tsfast.models.architectures.lru import DeepLRU

    torch.manual_seed(42)
    model = DeepLRU(2, 3, d_model=8, d_state=6, n_layers=2, r_min=0.5, r_max=0.98, max_phase=1.0,
                    return_state=True).double()
    with use_backend("reference"):
        gen = torch.Generator().manual_seed(4000)
        u = torch.randn(3, 40, 2, generator=gen, dtype=torch.float64)
        g = torch.randn(3, 40, 3, generator=gen, dtype=torch.float64)
        y, states = model(u)
        (y * g).sum().backward()
    store = {"u": _np(u), "g": _np(g), "y": _np(y)}
    for i, s in enumerate(states):
        store[f"state{i}"] = _np(s)
    for k, v in model.state_dict().items():
        store[f"param/{k}"] = _np(v)
    for k, v in model.named_parameters():
        store[f"grad/{k}"] = _np(v.grad)
    np.savez_compressed(HERE / "deeplru.npz", **store)
    print("deeplru", len(store), "arrays")


# ------------------------------------------------------------------ Mamba causal conv + SiLU
def make_conv():
    """The eager conv section of MambaLayer (mamba/core.py:38-58) in float64, gradients by autograd."""
    from tsfast.models.architectures.mamba.core import _causal_depthwise_silu

    cases = [(2, 19, 20, 4, True), (2, 3, 8, 4, True), (1, 1, 5, 2, False), (3, 70, 33, 8, True), (2, 40, 16, 3, False)]
    store, names = {}, []
    for idx, (Bsz, L, D, K, with_bias) in enumerate(cases):
        gen = torch.Generator().manual_seed(5000 + idx)
        rn = lambda *s: torch.randn(*s, generator=gen)  # noqa: E731
        x, tail, w = rn(Bsz, L, D), rn(Bsz, D, K - 1), rn(D, 1, K) * 0.5
        bias = rn(D) if with_bias else None
        gy = rn(Bsz, L, D)
        name = f"case{idx}"
        names.append(name)
        leaves = [_leaf(_to64(t)) for t in (x, tail, w)]
        b_ = _leaf(_to64(bias))
        y = _causal_depthwise_silu(leaves[0], leaves[1], leaves[2], b_ if b_ is not None else torch.zeros(D, dtype=torch.float64))
        y.backward(_to64(gy))
        store.update({f"{name}_x": _np(x), f"{name}_tail": _np(tail), f"{name}_w": _np(w[:, 0]), f"{name}_gy": _np(gy),
                      f"{name}_ref64_out": _np(y), f"{name}_ref64_gx": _np(leaves[0].grad),
                      f"{name}_ref64_gtail": _np(leaves[1].grad), f"{name}_ref64_gw": _np(leaves[2].grad[:, 0])})
        if with_bias:
            store[f"{name}_bias"] = _np(bias)
            store[f"{name}_ref64_gb"] = _np(b_.grad)
    store["names"] = np.array(names)
    np.savez_compressed(HERE / "conv.npz", **store)
    print("conv", len(names), "cases")


# ------------------------------------------------------------------ dynoNet G-block
def make_gblock():
    """The reference's ``LinearDynamicalOperator`` (tsfast/models/architectures/dynonet/core.py:
    144-254) in float64 on its CPU path: output, new state, and the gradient of ``sum(y * g)``
    w.r.t. the input, both coefficient tensors and the carried state."""
    from tsfast.models.architectures.dynonet.core import LinearDynamicalOperator

    # (B, L, I, O, nb, na, with_state)
    cases = [(2, 50, 1, 3, 8, 2, False), (2, 130, 3, 2, 8, 2, True), (1, 1100, 2, 2, 4, 4, True),
             (2, 33, 2, 1, 5, 3, True), (1, 3, 1, 1, 8, 4, True), (2, 64, 4, 4, 16, 1, False),
             (3, 257, 2, 3, 8, 4, True)]
    store, names = {}, []
    for idx, (Bsz, L, I, O, nb, na, with_state) in enumerate(cases):
        gen = torch.Generator().manual_seed(5000 + idx)
        op = LinearDynamicalOperator(I, O, nb=nb, na=na, backend="scan").double()
        with torch.no_grad():
            op.b_coeff.copy_((torch.randn(O, I, nb, generator=gen) * 0.3).double())  # float32 values
            op.a_coeff.copy_((torch.randn(O, I, na, generator=gen) * 0.2).double())
        u = torch.randn(Bsz, L, I, generator=gen)
        g = torch.randn(Bsz, L, O, generator=gen)
        tail = torch.randn(Bsz, nb - 1, I, generator=gen) if with_state else None
        x0 = torch.randn(Bsz, I * O, na, generator=gen) if with_state else None
        u_, tail_, x0_ = _leaf(_to64(u)), _leaf(_to64(tail)), _leaf(_to64(x0))
        state = {"u": tail_, "x": x0_} if with_state else None
        y, new_state = op(u_, state=state, return_state=True)
        (y * _to64(g)).sum().backward()
        name = f"case{idx}"
        names.append(name)
        store.update({f"{name}_u": _np(u), f"{name}_g": _np(g), f"{name}_b": _np(op.b_coeff.float()),
                      f"{name}_a": _np(op.a_coeff.float()), f"{name}_ref64_y": _np(y),
                      f"{name}_ref64_tail": _np(new_state["u"]), f"{name}_ref64_xlast": _np(new_state["x"]),
                      f"{name}_ref64_gu": _np(u_.grad), f"{name}_ref64_gb": _np(op.b_coeff.grad),
                      f"{name}_ref64_ga": _np(op.a_coeff.grad)})
        if with_state:
            store.update({f"{name}_tail": _np(tail), f"{name}_x0": _np(x0),
                          f"{name}_ref64_gtail": _np(tail_.grad), f"{name}_ref64_gx0": _np(x0_.grad)})
    store["names"] = np.array(names)
    np.savez_compressed(HERE / "gblock.npz", **store)
    print("gblock", len(names), "cases")


def make_dynonet():
    """A small reference DynoNet (tsfast/models/architectures/dynonet/core.py:257-346) in float64:
    parameters, input, output, and the gradient of ``sum(y * g)`` w.r.t. every parameter."""
    from tsfast.models.architectures.dynonet.core import DynoNet

    torch.manual_seed(11)
    net = DynoNet(2, 1, n_channels=4, nb=8, na=2, hidden_size=16, hidden_layers=1, bypass=True).double()
    with torch.no_grad():
        for n_, p_ in net.named_parameters():
            if n_.endswith("a_coeff"):
                p_.copy_((torch.randn(p_.shape) * 0.2).double())  # poles away from the origin; float32 values
            else:
                p_.copy_(p_.float().double())
    gen = torch.Generator().manual_seed(12)
    u = torch.randn(3, 700, 2, generator=gen)
    g = torch.randn(3, 700, 1, generator=gen)
    y = net(_to64(u))
    (y * _to64(g)).sum().backward()
    store = {"u": _np(u), "g": _np(g), "ref64_y": _np(y)}
    for n_, p_ in net.named_parameters():
        store[f"param_{n_}"] = _np(p_.float())
        store[f"grad_{n_}"] = _np(p_.grad)
    np.savez_compressed(HERE / "dynonet.npz", **store)
    print("dynonet", len(list(net.named_parameters())), "parameters")


if __name__ == "__main__":
    torch.set_num_threads(4)
    which = sys.argv[1:] or ["diag", "sel", "mamba", "allpole", "lru", "conv", "gblock", "dynonet"]
    if "diag" in which:
        make_diag("diag")
    if "sel" in which:
        make_diag("sel")
    if "mamba" in which:
        make_mamba()
    if "allpole" in which:
        make_allpole()
    if "lru" in which:
        make_lru()
    if "conv" in which:
        make_conv()
    if "gblock" in which:
        make_gblock()
    if "dynonet" in which:
        make_dynonet()
