"""GPU parity of the fused Mamba selective-scan section (S3) through the C-ABI: golden vectors
from the reference's unfused float64 path, the float64 CPU oracle at the odd shapes the reference
tests (L not a multiple of the checkpoint interval, L below it, ragged channel block, d_state
not a power of two; reference tests/test_mamba.py:276-298), carried state and its gradients, and a
full-size run checked on a slice.  Bound: max|a-b|/max|b| < 1e-4 per tensor."""

import numpy as np
import pytest
import torch

from conftest import load_golden, rel_err

pytestmark = pytest.mark.gpu
REL = 1e-4
GRADS = ("gdraw", "gA", "gBt", "gCt", "gu", "gz", "gDp", "gh0")


def _err(a, b):
    """rel_err with a floor on the reference scale: a gradient that is exactly zero in float64
    (e.g. grad_A for L=1 from a zero state) comes out as float32 rounding residue (~1e-9)."""
    a, b = np.asarray(a), np.asarray(b)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-4)) if a.size else 0.0


def _dev(x):
    return None if x is None else torch.from_numpy(np.array(x, copy=True)).cuda()


def _run(ins, gout, ghlast):
    """ins: draw, A, Bt, Ct, u, z, Dp, h0 (numpy).  Returns out, hlast and the gradient dict."""
    from tsfast_b200 import mamba_b200 as mb

    d = [_dev(x) for x in ins]
    out, hlast, chk = mb._scan_train_op(*d)
    out2, hlast2 = mb._scan_op(*d)
    assert torch.equal(out, out2) and torch.equal(hlast, hlast2)  # inference path == training path
    g = mb._scan_bwd_op(_dev(gout), _dev(ghlast), chk, *d)
    torch.cuda.synchronize()
    r = {k: v.cpu().numpy() for k, v in zip(GRADS, g)}
    if ins[7] is None:
        r["gh0"] = None
    return out.cpu().numpy(), hlast.cpu().numpy(), r


def test_golden():
    for c in load_golden("mamba"):
        ins = [getattr(c, k) for k in ("draw", "A", "Bt", "Ct", "u", "z", "Dp", "h0")]
        out, hlast, r = _run(ins, c.gout, c.ghlast)
        assert rel_err(out, c.ref64_out) < REL, (c.name, "out")
        assert rel_err(hlast, c.ref64_hlast) < REL, (c.name, "hlast")
        for k in GRADS:
            ref = getattr(c, f"ref64_{k}")
            if ref is not None:
                assert _err(r[k], ref) < REL, (c.name, k)


def _case(rng, B, L, D, N, with_h0, with_glast, s4d=False):
    f = lambda *s: rng.standard_normal(s).astype(np.float32)  # noqa: E731
    draw = (f(B, L, D) * 0.5 - (3.0 if s4d else 1.0)).astype(np.float32)
    A = (-np.broadcast_to(np.arange(1, N + 1, dtype=np.float32), (D, N)).copy() if s4d
         else -np.exp(f(D, N) * 0.5)).astype(np.float32)
    ins = [draw, A, f(B, L, N), f(B, L, N), f(B, L, D), f(B, L, D), (np.ones(D, np.float32) if s4d else f(D)),
           f(B, D, N) if with_h0 else None]
    return ins, f(B, L, D), (f(B, D, N) if with_glast else None)


_SHAPES = [(2, 19, 20, 12), (2, 5, 8, 16), (3, 64, 33, 16), (1, 1, 4, 4), (2, 37, 16, 5), (2, 100, 40, 3),
           (2, 50, 12, 24), (1, 48, 8, 64), (1, 33, 6, 128), (2, 130, 70, 16), (4, 256, 128, 16), (2, 17, 1, 1)]


@pytest.mark.parametrize("with_h0,with_glast", [(True, True), (False, False), (True, False), (False, True)])
@pytest.mark.parametrize("B,L,D,N", _SHAPES)
def test_matches_oracle(oracle, B, L, D, N, with_h0, with_glast):
    rng = np.random.default_rng(B * 7919 + L * 31 + D * 7 + N)
    ins, gout, ghl = _case(rng, B, L, D, N, with_h0, with_glast)
    out, hlast, r = _run(ins, gout, ghl)
    d = lambda x: None if x is None else x.astype(np.float64)  # noqa: E731
    ro, rh = oracle.mamba_fwd(*map(d, ins))
    rr = oracle.mamba_bwd(*map(d, ins), d(gout), d(ghl))
    assert rel_err(out, ro) < REL and rel_err(hlast, rh) < REL
    for k in GRADS:
        if rr[k] is not None:
            assert _err(r[k], rr[k]) < REL, k


def test_bitwise_repeat():
    rng = np.random.default_rng(4)
    ins, gout, ghl = _case(rng, 3, 90, 48, 16, True, True)
    a, b = _run(ins, gout, ghl), _run(ins, gout, ghl)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    for k in GRADS:
        assert np.array_equal(a[2][k], b[2][k]), k


def test_run_autograd_chunked_state(oracle):
    """run(): three chunks with the state handed over give the same output as one pass and the
    gradient flows through the carried state (reference tests/test_mamba.py:179-230)."""
    from tsfast_b200 import mamba_b200 as mb

    rng = np.random.default_rng(8)
    ins, gout, _ = _case(rng, 2, 96, 24, 16, True, False)
    t = [(_dev(x).requires_grad_() if x is not None else None) for x in ins]
    out_full, h_full = mb.run(*t)
    (out_full * _dev(gout)).sum().backward()
    full_grads = [x.grad.clone() for x in t]
    for x in t:
        x.grad = None
    h, outs = t[7], []
    for lo, hi in ((0, 40), (40, 41), (41, 96)):
        sl = [t[0][:, lo:hi], t[1], t[2][:, lo:hi], t[3][:, lo:hi], t[4][:, lo:hi], t[5][:, lo:hi], t[6], h]
        o, h = mb.run(*sl)
        outs.append(o)
    out_chunks = torch.cat(outs, 1)
    assert rel_err(out_chunks.detach().cpu().numpy(), out_full.detach().cpu().numpy()) < 1e-5
    assert rel_err(h.detach().cpu().numpy(), h_full.detach().cpu().numpy()) < 1e-5
    (out_chunks * _dev(gout)).sum().backward()
    for name, x, gf in zip(("draw", "A", "Bt", "Ct", "u", "z", "Dp", "h0"), t, full_grads):
        assert rel_err(x.grad.cpu().numpy(), gf.cpu().numpy()) < 1e-4, name
    with torch.no_grad():
        o2, _ = mb.run(*t)
    assert torch.equal(o2, out_full)


def test_config3_full_size_slice(oracle):
    """C3 (B=32, T=2048, D=512, N=16, S4D-real A, D=1): full-size launch, checked against the
    float64 oracle on one batch row (the rows are independent) for every output."""
    rng = np.random.default_rng(0)
    B, L, D, N = 32, 2048, 512, 16
    ins, gout, _ = _case(rng, B, L, D, N, False, False, s4d=True)
    out, hlast, r = _run(ins, gout, None)
    b = 5
    sl = [ins[0][b : b + 1], ins[1], ins[2][b : b + 1], ins[3][b : b + 1], ins[4][b : b + 1], ins[5][b : b + 1],
          ins[6], None]
    d = lambda x: None if x is None else x.astype(np.float64)  # noqa: E731
    ro, rh = oracle.mamba_fwd(*map(d, sl))
    rr = oracle.mamba_bwd(*map(d, sl), d(gout[b : b + 1]), None)
    assert rel_err(out[b : b + 1], ro) < REL and rel_err(hlast[b : b + 1], rh) < REL
    for k in ("gdraw", "gu", "gz", "gBt", "gCt"):
        assert rel_err(r[k][b : b + 1], rr[k]) < REL, k
    assert np.isfinite(r["gA"]).all() and np.isfinite(r["gDp"]).all()
