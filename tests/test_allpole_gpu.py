"""GPU parity of the all-pole IIR scan (S4) through the C-ABI: golden vectors from the reference's
companion-matrix scan, the float64 CPU oracle at the shapes of the reference's
tests/test_scan_allpole_backend.py:21-28 (incl. L=1, L<na, single lane, every order 1..16), and
size-independent residual checks at the full benchmark size.  Bound: max|a-b|/max|b| < 1e-4."""

import numpy as np
import pytest
import torch

from conftest import load_golden, rel_err

pytestmark = pytest.mark.gpu
REL = 1e-4


def _dev(x):
    return None if x is None else torch.from_numpy(np.array(x, copy=True)).cuda()


def _run(a, w, y0, g):
    from tsfast_b200 import allpole_b200 as ap

    a_d, w_d, y0_d, g_d = _dev(a), _dev(w), _dev(y0), _dev(g)
    y = ap._allpole_op(a_d, w_d, y0_d)
    ga, gw, gy0 = ap._allpole_bwd_op(g_d, a_d, y, y0_d)
    torch.cuda.synchronize()
    return y.cpu().numpy(), ga.cpu().numpy(), gw.cpu().numpy(), (gy0.cpu().numpy() if y0 is not None else None)


def test_golden():
    for c in load_golden("allpole"):
        y, ga, gw, gy0 = _run(c.a, c.w, c.y0, c.g)
        assert rel_err(y, c.ref64_y) < REL, (c.name, "y")
        assert rel_err(gw, c.ref64_gw) < REL, (c.name, "gw")
        assert rel_err(ga, c.ref64_ga) < REL, (c.name, "ga")
        if c.y0 is not None:
            assert rel_err(gy0, c.ref64_gy0) < REL, (c.name, "gy0")


def _stable_a(rng, lanes, na):
    """Monic denominator from random poles inside the unit circle (radius <= 0.9)."""
    a = np.zeros((lanes, na))
    for i in range(lanes):
        poles = []
        while len(poles) < na:
            r, th = rng.uniform(0.2, 0.9), rng.uniform(0, np.pi)
            if na - len(poles) >= 2:
                poles += [r * np.exp(1j * th), r * np.exp(-1j * th)]
            else:
                poles.append(rng.uniform(-0.9, 0.9))
        a[i] = np.real(np.poly(poles))[1:]
    return a.astype(np.float32)


_SHAPES = [(32 * 8, 200, 2), (4 * 32, 100, 8), (15, 7, 3), (8, 1, 2), (8, 2, 4), (1, 513, 1), (3, 1024, 4),
           (5, 1500, 4), (2, 2051, 6), (7, 512, 16), (3, 40, 16), (2, 3, 16)]
_SHAPES += [(3, 530, na) for na in range(1, 17)]


@pytest.mark.parametrize("with_y0", [True, False])
@pytest.mark.parametrize("lanes,L,na", _SHAPES)
def test_matches_oracle(oracle, lanes, L, na, with_y0):
    rng = np.random.default_rng(lanes * 1000 + L * 17 + na)
    a = _stable_a(rng, lanes, na)
    w = rng.standard_normal((lanes, L)).astype(np.float32)
    g = rng.standard_normal((lanes, L)).astype(np.float32)
    y0 = rng.standard_normal((lanes, na)).astype(np.float32) if with_y0 else None
    y, ga, gw, gy0 = _run(a, w, y0, g)
    d = lambda x: None if x is None else x.astype(np.float64)  # noqa: E731
    ry = oracle.allpole_fwd(d(a), d(w), d(y0))
    rga, rgw, rgy0 = oracle.allpole_bwd(d(g), d(a), ry, d(y0))
    assert rel_err(y, ry) < REL
    assert rel_err(gw, rgw) < REL
    assert rel_err(ga, rga) < REL
    if with_y0:
        assert rel_err(gy0, rgy0) < REL


def test_zero_coefficients_and_bitwise_repeat(oracle):
    """a = 0 (dynoNet's initialisation: a nilpotent companion matrix) is the identity filter; two
    launches on the same inputs give identical bits."""
    rng = np.random.default_rng(3)
    a = np.zeros((6, 4), dtype=np.float32)
    w = rng.standard_normal((6, 700)).astype(np.float32)
    g = rng.standard_normal((6, 700)).astype(np.float32)
    r1 = _run(a, w, None, g)
    assert np.array_equal(r1[0], w) and np.array_equal(r1[2], g)
    a = _stable_a(rng, 6, 4)
    y0 = rng.standard_normal((6, 4)).astype(np.float32)
    r1, r2 = _run(a, w, y0, g), _run(a, w, y0, g)
    for x, y in zip(r1, r2):
        assert np.array_equal(x, y)


def test_unstable_pole_overflows_without_fault():
    """An unstable filter runs to non-finite values and the context stays usable
    (reference tests/test_dynonet.py:165-174); zero input through it stays exactly zero."""
    from tsfast_b200 import allpole_b200 as ap

    a = torch.tensor([[-3.0]], device="cuda")
    y = ap.run(a, torch.ones(1, 2000, device="cuda"), None)
    torch.cuda.synchronize()
    assert not torch.isfinite(y).all()
    z = ap.run(a, torch.zeros(1, 2000, device="cuda"), None)
    assert torch.count_nonzero(z).item() == 0


def test_unaligned_length_and_views(oracle):
    """L not a multiple of 4 or a sliced buffer takes the 4-byte copy path."""
    from tsfast_b200 import allpole_b200 as ap

    rng = np.random.default_rng(9)
    a = _stable_a(rng, 5, 3)
    w = rng.standard_normal((5, 1027)).astype(np.float32)
    y = ap._allpole_op(_dev(a), _dev(w), None).cpu().numpy()
    assert rel_err(y, oracle.allpole_fwd(a.astype(np.float64), w.astype(np.float64), None)) < REL
    big = torch.zeros(5 * 1024 + 1, device="cuda")
    wv = big[1:].view(5, 1024)
    wv.copy_(_dev(w[:, :1024]))
    y = ap._allpole_op(_dev(a), wv, None).cpu().numpy()
    assert rel_err(y, oracle.allpole_fwd(a.astype(np.float64), w[:, :1024].astype(np.float64), None)) < REL


def test_run_broadcast_and_autograd(oracle):
    """run(): a [P,na] broadcast over batch, gradients folded by autograd; per-batch a keeps its
    batch axis (reference tests/test_scan_allpole_backend.py:79-97); no-grad equals grad path."""
    from tsfast_b200 import allpole_b200 as ap

    rng = np.random.default_rng(1)
    Bn, P, L, na = 4, 6, 128, 3
    a0 = _stable_a(rng, P, na)
    a = _dev(a0).requires_grad_()
    w = torch.randn(Bn, P, L, device="cuda", requires_grad=True)
    y0 = torch.randn(Bn, P, na, device="cuda", requires_grad=True)
    gy = torch.randn(Bn, P, L, device="cuda")
    y = ap.run(a, w, y0)
    ga, gw, gy0 = torch.autograd.grad(y, (a, w, y0), gy)
    d = lambda t: t.detach().cpu().numpy().astype(np.float64)  # noqa: E731
    al = np.broadcast_to(a0.astype(np.float64), (Bn, P, na)).reshape(-1, na)
    ry = oracle.allpole_fwd(al, d(w).reshape(-1, L), d(y0).reshape(-1, na))
    rga, rgw, rgy0 = oracle.allpole_bwd(d(gy).reshape(-1, L), al, ry, d(y0).reshape(-1, na))
    assert rel_err(d(y).reshape(-1, L), ry) < REL
    assert rel_err(d(ga), rga.reshape(Bn, P, na).sum(0)) < REL
    assert rel_err(d(gw).reshape(-1, L), rgw) < REL
    assert rel_err(d(gy0).reshape(-1, na), rgy0) < REL
    with torch.no_grad():
        assert torch.equal(ap.run(a, w, y0), y)
    ab = _dev(np.broadcast_to(a0, (Bn, P, na)).copy()).requires_grad_()
    (gab,) = torch.autograd.grad(ap.run(ab, w, y0), (ab,), gy)
    assert gab.shape == ab.shape and rel_err(d(gab).reshape(-1, na), rga) < REL


def test_config4_full_size_properties():
    """C4 (128 x 128 lanes, T=8192, order 4 from two conjugate pole pairs): the defining difference
    equation holds at every step of the output and of the adjoint (size-independent check)."""
    from tsfast_b200 import allpole_b200 as ap

    rng = np.random.default_rng(0)
    P, Bn, L = 128, 128, 8192
    a0 = np.zeros((P, 4))
    for i in range(P):
        poles = []
        for _ in range(2):
            r, th = rng.uniform(0.5, 0.95), rng.uniform(0, np.pi)
            poles += [r * np.exp(1j * th), r * np.exp(-1j * th)]
        a0[i] = np.real(np.poly(poles))[1:]
    a = _dev(np.broadcast_to(a0.astype(np.float32), (Bn, P, 4)).reshape(-1, 4).copy())
    gen = torch.Generator(device="cuda").manual_seed(0)
    w = torch.randn(Bn * P, L, device="cuda", generator=gen)
    y = ap._allpole_op(a, w, None)

    def residual(out, inp, reverse):
        o = out.flip(-1) if reverse else out
        i_ = inp.flip(-1) if reverse else inp
        pred = i_[:, 4:].clone()
        for k in range(4):
            pred -= a[:, k : k + 1] * o[:, 3 - k : L - 1 - k]
        return (o[:, 4:] - pred).abs().max().item()

    # a state error e at a segment seam shows up as a residual of about sum|a_k| * e
    amp = 1.0 + a.abs().sum(1).max().item()
    assert residual(y, w, False) < 1e-5 * amp * y.abs().max().item()
    g = torch.randn(Bn * P, L, device="cuda", generator=gen)
    ga, gw, _ = ap._allpole_bwd_op(g, a, y, None)
    assert residual(gw, g, True) < 1e-5 * amp * gw.abs().max().item()
    assert torch.isfinite(ga).all()
