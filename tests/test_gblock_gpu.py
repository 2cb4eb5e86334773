"""GPU parity of the fused dynoNet G-block (FIR numerator + all-pole denominator + pair sum) through
the C-ABI: golden vectors from the reference's LinearDynamicalOperator
(tsfast/models/architectures/dynonet/core.py:144-254), the float64 CPU oracle at ragged and
multi-tile shapes, chunked continuation (tests/test_dynonet.py's stateful equivalence), and the
module mirror.  Bound: max|a-b|/max|b| < 1e-4."""

import numpy as np
import pytest
import torch

from conftest import load_golden, rel_err

pytestmark = pytest.mark.gpu
REL = 1e-4


def _dev(x, grad=False):
    if x is None:
        return None
    t = torch.from_numpy(np.array(x, copy=True)).cuda()
    return t.requires_grad_() if grad else t


def _np(t):
    return None if t is None else t.detach().cpu().numpy()


def _run(u, b, a, tail, x0, g=None):
    """Forward (and, with g, the gradients of sum(y*g)) through tsfast_b200.dynonet_b200.linear_block."""
    from tsfast_b200 import dynonet_b200 as dn

    grad = g is not None
    u_d, b_d, a_d, tail_d, x0_d = (_dev(t, grad) for t in (u, b, a, tail, x0))
    state = {"u": tail_d, "x": x0_d} if tail is not None else None
    y, new_state = dn.linear_block(u_d, b_d, a_d, state)
    out = {"y": _np(y), "tail": _np(new_state["u"]), "xlast": _np(new_state["x"])}
    if grad:
        (y * _dev(g)).sum().backward()
        out.update(gu=_np(u_d.grad), gb=_np(b_d.grad), ga=_np(a_d.grad))
        if tail is not None:
            out.update(gtail=_np(tail_d.grad), gx0=_np(x0_d.grad))
    torch.cuda.synchronize()
    return out


@pytest.fixture(params=["per_row", "per_filter"])
def warp_split(request, monkeypatch):
    """Both work splits must pass: a warp per (batch row, channel) walking the other channel axis,
    and (chosen for blocks too small to fill the GPU) a warp per filter with the sum done outside."""
    from tsfast_b200 import dynonet_b200 as dn

    monkeypatch.setattr(dn, "_SPLIT_BELOW", 0 if request.param == "per_row" else 10**9)
    return request.param


def test_golden(warp_split):
    for c in load_golden("gblock"):
        r = _run(c.u, c.b, c.a, c.tail, c.x0, c.g)
        keys = ["y", "tail", "xlast", "gu", "gb", "ga"] + (["gtail", "gx0"] if c.tail is not None else [])
        for k in keys:
            assert rel_err(r[k], getattr(c, "ref64_" + k)) < REL, (c.name, k)


def test_golden_without_autograd_matches(warp_split):
    """The inference path (no per-pair outputs kept) gives the same numbers."""
    for c in load_golden("gblock"):
        with torch.no_grad():
            r = _run(c.u, c.b, c.a, c.tail, c.x0)
        assert rel_err(r["y"], c.ref64_y) < REL, c.name
        assert rel_err(r["xlast"], c.ref64_xlast) < REL, c.name


# (B, L, I, O, nb, na, with_state): ragged lengths, L not a multiple of 4 (4-byte copies), several
# 1024-step tiles, the tile boundary inside the last na steps, every supported order and tap size
SHAPES = [(2, 1, 1, 1, 8, 2, True), (1, 2, 2, 2, 4, 4, True), (3, 1023, 2, 3, 8, 2, False),
          (2, 1024, 3, 2, 8, 3, True), (2, 1025, 1, 4, 8, 4, True), (1, 2050, 2, 2, 16, 1, True),
          (2, 3000, 4, 4, 8, 2, True), (1, 777, 5, 3, 3, 2, True), (2, 96, 8, 8, 1, 2, False),
          (1, 1026, 2, 2, 12, 4, True)]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s[:6])) + ("s" if s[6] else ""))
def test_matches_oracle(oracle, warp_split, shape):
    Bsz, L, I, O, nb, na, with_state = shape
    rng = np.random.default_rng(sum(p * q for p, q in zip(shape[:6], (7, 11, 13, 17, 19, 23))))
    u = rng.standard_normal((Bsz, L, I)).astype(np.float32)
    b = (rng.standard_normal((O, I, nb)) * 0.3).astype(np.float32)
    a = (rng.standard_normal((O, I, na)) * (0.5 / na)).astype(np.float32)
    g = rng.standard_normal((Bsz, L, O)).astype(np.float32)
    tail = rng.standard_normal((Bsz, nb - 1, I)).astype(np.float32) if with_state else None
    x0 = rng.standard_normal((Bsz, I * O, na)).astype(np.float32) if with_state else None
    f64 = lambda t: None if t is None else t.astype(np.float64)
    y, yp, xl, nt = oracle.gblock_fwd(f64(u), f64(b), f64(a), f64(tail), f64(x0))
    gu, gb, ga, gt, gx0 = oracle.gblock_bwd(f64(g), f64(u), f64(b), f64(a), yp, f64(tail), f64(x0))
    r = _run(u, b, a, tail, x0, g)
    for k, ref in (("y", y), ("xlast", xl), ("tail", nt), ("gu", gu), ("gb", gb), ("ga", ga)):
        assert rel_err(r[k], ref) < REL, (shape, k)
    if with_state:
        assert rel_err(r["gtail"], gt) < REL, (shape, "gtail")
        assert rel_err(r["gx0"], gx0) < REL, (shape, "gx0")


def test_chunked_rollout_equals_full_sequence(warp_split):
    """Feeding the returned state back continues the sequence (reference tests/test_dynonet.py stateful checks)."""
    from tsfast_b200 import dynonet_b200 as dn

    torch.manual_seed(0)
    Bsz, L, I, O, nb, na = 2, 2500, 2, 3, 8, 2
    u = torch.randn(Bsz, L, I, device="cuda")
    b = torch.randn(O, I, nb, device="cuda") * 0.3
    a = torch.randn(O, I, na, device="cuda") * 0.2
    with torch.no_grad():
        full, _ = dn.linear_block(u, b, a, None)
        parts, state = [], None
        for lo, hi in ((0, 1), (1, 700), (700, 1724), (1724, 2500)):
            y, state = dn.linear_block(u[:, lo:hi], b, a, state)
            parts.append(y)
    torch.cuda.synchronize()
    assert rel_err(torch.cat(parts, 1).cpu().numpy(), full.cpu().numpy()) < 1e-5


def test_gradient_through_the_new_state(warp_split):
    """A loss on the returned filter state as well: the general adjoint against the reference's
    formulation (grouped conv1d, all-pole op, slices) differentiated by autograd."""
    import torch.nn.functional as F

    from tsfast_b200 import allpole_b200, dynonet_b200 as dn

    torch.manual_seed(1)
    Bsz, L, I, O, nb, na = 2, 300, 2, 3, 8, 3
    mk = lambda *s: torch.randn(*s, device="cuda")
    u0, b0, a0 = mk(Bsz, L, I), mk(O, I, nb) * 0.3, mk(O, I, na) * 0.15
    tail0, x00, gy, gx = mk(Bsz, nb - 1, I), mk(Bsz, I * O, na), mk(Bsz, L, O), mk(Bsz, I * O, na)

    def grads(fused):
        u, b, a, tail, x0 = (t.clone().requires_grad_() for t in (u0, b0, a0, tail0, x00))
        if fused:
            y, st = dn.linear_block(u, b, a, {"u": tail, "x": x0})
            xl = st["x"]
        else:
            P = I * O
            w = F.conv1d(torch.cat((tail, u), 1).transpose(1, 2), b.permute(1, 0, 2).reshape(P, 1, nb).flip(-1), groups=I)
            yp = allpole_b200.run(a.permute(1, 0, 2).reshape(P, na), w, x0)
            y = yp.view(Bsz, I, O, L).sum(1).transpose(1, 2)
            xl = yp[..., L - na :].flip(-1)
        ((y * gy).sum() + (xl * gx).sum()).backward()
        return [t.grad.cpu().numpy() for t in (u, b, a, tail, x0)]

    for got, ref, name in zip(grads(True), grads(False), ("gu", "gb", "ga", "gtail", "gx0")):
        assert rel_err(got, ref) < 1e-4, name


def test_module_mirror_loads_reference_state_dict_names():
    from mirrors import LinearDynamicalOperator

    op = LinearDynamicalOperator(2, 3, nb=8, na=2).cuda()
    assert set(op.state_dict()) == {"b_coeff", "a_coeff"}
    assert op.b_coeff.shape == (3, 2, 8) and op.a_coeff.shape == (3, 2, 2)
    u = torch.randn(2, 40, 2, device="cuda")
    y, st = op(u, return_state=True)
    assert y.shape == (2, 40, 3) and st["u"].shape == (2, 7, 2) and st["x"].shape == (2, 6, 2)
    y.sum().backward()
    assert op.b_coeff.grad is not None and op.a_coeff.grad is not None


def test_dynonet_matches_reference_model():
    """The DynoNet mirror with the reference model's parameters (loaded by name) reproduces its
    float64 output and parameter gradients (fixture from tsfast's DynoNet, dynonet/core.py:257-346)."""
    from pathlib import Path

    from mirrors import DynoNet

    z = np.load(Path(__file__).parent / "golden" / "dynonet.npz")
    net = DynoNet(2, 1, n_channels=4, nb=8, na=2, hidden_size=16, hidden_layers=1, bypass=True)
    sd = {k[len("param_"):]: torch.from_numpy(z[k]) for k in z.files if k.startswith("param_")}
    assert set(sd) == set(net.state_dict())
    net.load_state_dict(sd)
    net.cuda()
    y = net(_dev(z["u"]))
    (y * _dev(z["g"])).sum().backward()
    torch.cuda.synchronize()
    assert rel_err(_np(y), z["ref64_y"]) < REL
    for name, p_ in net.named_parameters():
        assert rel_err(_np(p_.grad), z["grad_" + name]) < 2e-4, name


def test_unsupported_shapes_raise():
    from tsfast_b200 import dynonet_b200 as dn

    u = torch.randn(1, 8, 1, device="cuda")
    with pytest.raises(RuntimeError):
        dn.linear_block(u, torch.randn(1, 1, 8, device="cuda"), torch.randn(1, 1, 5, device="cuda"), None)
    with pytest.raises(RuntimeError):
        dn.linear_block(u, torch.randn(1, 1, 17, device="cuda"), torch.randn(1, 1, 2, device="cuda"), None)
    with pytest.raises(RuntimeError):
        dn.linear_block(u.cpu(), torch.randn(1, 1, 8), torch.randn(1, 1, 2), None)


def test_full_size_residuals():
    """At the benchmark size (B=128, T=8192, 8 x 16 filters, nb=8, na=4) the outputs satisfy the
    defining equations: every pair's output run back through its denominator gives the numerator
    output (grouped conv1d of the input), the block output is the sum over inputs, and the new
    state is the last na outputs of every pair."""
    import torch.nn.functional as F

    from tsfast_b200 import dynonet_b200 as dn

    torch.manual_seed(4)
    Bsz, L, I, O, nb, na = 128, 8192, 8, 16, 8, 4
    P = I * O
    u = torch.randn(Bsz, L, I, device="cuda")
    b = torch.randn(O, I, nb, device="cuda") * 0.3
    r, th = torch.rand(O, I, 2, device="cuda") * 0.45 + 0.5, torch.rand(O, I, 2, device="cuda") * 3.14159
    c1, d1 = -2 * r[..., 0] * torch.cos(th[..., 0]), r[..., 0] ** 2
    c2, d2 = -2 * r[..., 1] * torch.cos(th[..., 1]), r[..., 1] ** 2
    a = torch.stack((c1 + c2, d1 + d2 + c1 * c2, c1 * d2 + c2 * d1, d1 * d2), -1)  # two conjugate pole pairs
    with torch.no_grad():
        y, yp, xl, _, _ = dn._gblock_op(u, None, b, a, None, True)
        y_inf = dn._gblock_op(u, None, b, a, None, False)[0]
        w = F.conv1d(torch.cat((u.new_zeros(Bsz, nb - 1, I), u), 1).transpose(1, 2),
                     b.permute(1, 0, 2).reshape(P, 1, nb).flip(-1), groups=I)
        a_p = a.permute(1, 0, 2).reshape(1, P, na)
        res = yp.clone()
        for k in range(1, na + 1):  # y_t + sum_k a_k y_{t-k} = w_t with a zero start
            res[..., k:] += a_p[..., k - 1 : k] * yp[..., :-k]
        # rounding of the na + 1 terms is relative to the outputs, which these poles amplify
        bound = 1e-5 * float(yp.abs().max()) * (1 + float(a.abs().sum(-1).max()))
        err = float((res - w).abs().max())
        assert err < bound, (err, bound, float(w.abs().max()))
        assert torch.equal(y, y_inf)
        ysum = yp.view(Bsz, I, O, L).sum(1)
        assert float((y - ysum).abs().max()) < 1e-5 * float(ysum.abs().max())
        assert torch.equal(xl, yp[..., L - na :].flip(-1))
