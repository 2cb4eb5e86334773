"""GPU parity of the Mamba causal depthwise conv + SiLU through the C-ABI: golden vectors from the
reference's eager definition (float64), the float64 CPU oracle over kernel widths 2..8, ragged
channel counts, sequences shorter than the kernel and strided chunk views, bitwise repeatability,
and autograd through `run`.  Bound: max|a-b|/max|b| < 1e-4 per tensor."""

import numpy as np
import pytest
import torch

from conftest import load_golden, rel_err

pytestmark = pytest.mark.gpu
REL = 1e-4


def _dev(x):
    return None if x is None else torch.from_numpy(np.array(x, copy=True)).cuda()


def _run(x, tail, w, bias, gy):
    from tsfast_b200 import conv_b200 as cv

    xd, td, wd, bd, gd = (_dev(t) for t in (x, tail, w, bias, gy))
    out = cv._conv_silu_op(xd, td, wd, bd)
    gx, gt, gw, gb = cv._conv_silu_bwd_op(gd, xd, td, wd, bd)
    torch.cuda.synchronize()
    return tuple(t.cpu().numpy() for t in (out, gx, gt, gw)) + ((gb.cpu().numpy() if bias is not None else None),)


def test_golden():
    for c in load_golden("conv"):
        out, gx, gt, gw, gb = _run(c.x, c.tail, c.w, c.bias, c.gy)
        assert rel_err(out, c.ref64_out) < REL, (c.name, "out")
        assert rel_err(gx, c.ref64_gx) < REL, (c.name, "gx")
        assert rel_err(gt, c.ref64_gtail) < REL, (c.name, "gtail")
        assert rel_err(gw, c.ref64_gw) < REL, (c.name, "gw")
        if c.bias is not None:
            assert rel_err(gb, c.ref64_gb) < REL, (c.name, "gb")


_SHAPES = [(2, 200, 64, 4), (3, 65, 20, 4), (1, 1, 8, 4), (2, 2, 12, 8), (2, 129, 33, 3), (1, 500, 512, 4), (4, 64, 256, 2)]
_SHAPES += [(2, 70, 16, K) for K in range(2, 9)]
# whole segments only: a segment that is first and last at once, several tiles per CTA of the persistent adjoint
_SHAPES += [(1, 32, 8, 4), (2, 96, 300, 8), (3, 160, 130, 5), (700, 64, 256, 4)]


@pytest.mark.parametrize("with_bias", [True, False])
@pytest.mark.parametrize("B,L,D,K", _SHAPES)
def test_matches_oracle(oracle, B, L, D, K, with_bias):
    rng = np.random.default_rng(B * 100003 + L * 101 + D * 7 + K)
    f = lambda *s: rng.standard_normal(s).astype(np.float32)  # noqa: E731
    x, tail, w, gy = f(B, L, D), f(B, D, K - 1), f(D, K) * 0.5, f(B, L, D)
    bias = f(D) if with_bias else None
    got = _run(x, tail, w, bias, gy)
    d = lambda t: None if t is None else t.astype(np.float64)  # noqa: E731
    ro = oracle.conv_fwd(d(x), d(tail), d(w), d(bias))
    rgx, rgt, rgw, rgb = oracle.conv_bwd(d(gy), d(x), d(tail), d(w), d(bias))
    for name, a, b in zip(("out", "gx", "gtail", "gw"), got, (ro, rgx, rgt, rgw)):
        assert rel_err(a, b) < REL, name
    if with_bias:
        assert rel_err(got[4], rgb) < REL


def test_strided_chunk_view_run_autograd_and_repeat(oracle):
    """x as the first half of a wider projection (read in place, stride 2D along time), through
    `run` with weight [D,1,K], gradients by autograd; two runs are bitwise identical."""
    from tsfast_b200 import conv_b200 as cv

    torch.manual_seed(0)
    B, L, D, K = 3, 150, 48, 4
    proj = torch.randn(B, L, 2 * D, device="cuda", requires_grad=True)
    tail = torch.randn(B, D, K - 1, device="cuda", requires_grad=True)
    w = (torch.randn(D, 1, K, device="cuda") * 0.5).requires_grad_()
    bias = torch.randn(D, device="cuda", requires_grad=True)
    gy = torch.randn(B, L, D, device="cuda")
    x = proj.chunk(2, dim=-1)[0]
    assert not x.is_contiguous() and cv.supports(x, tail, w, bias) is None
    y = cv.run(x, tail, w, bias)
    grads = torch.autograd.grad(y, (proj, tail, w, bias), gy)
    y2 = cv.run(x, tail, w, bias)
    grads2 = torch.autograd.grad(y2, (proj, tail, w, bias), gy)
    assert torch.equal(y, y2) and all(torch.equal(a, b) for a, b in zip(grads, grads2))
    d = lambda t: t.detach().cpu().numpy().astype(np.float64)  # noqa: E731
    xn = d(proj)[:, :, :D].copy()
    ro = oracle.conv_fwd(xn, d(tail), d(w)[:, 0], d(bias))
    rgx, rgt, rgw, rgb = oracle.conv_bwd(d(gy), xn, d(tail), d(w)[:, 0], d(bias))
    assert rel_err(d(y), ro) < REL
    assert rel_err(d(grads[0])[:, :, :D], rgx) < REL and np.abs(d(grads[0])[:, :, D:]).max() == 0.0
    assert rel_err(d(grads[1]), rgt) < REL and rel_err(d(grads[2])[:, 0], rgw) < REL and rel_err(d(grads[3]), rgb) < REL


def test_config3_shape_against_torch_conv():
    """The Mamba benchmark shape (B=32, T=2048, D=512, K=4): cross-check with cuDNN's grouped conv1d
    in float32 (an independent implementation) on the output and the input gradient."""
    import torch.nn.functional as F

    from tsfast_b200 import conv_b200 as cv

    torch.manual_seed(1)
    B, L, D, K = 32, 2048, 512, 4
    x = torch.randn(B, L, D, device="cuda", requires_grad=True)
    tail = torch.randn(B, D, K - 1, device="cuda")
    w = torch.randn(D, 1, K, device="cuda") * 0.5
    bias = torch.randn(D, device="cuda")
    gy = torch.randn(B, L, D, device="cuda")
    y = cv.run(x, tail, w, bias)
    (gx,) = torch.autograd.grad(y, (x,), gy)
    xr = x.detach().clone().requires_grad_()
    yr = F.silu(F.conv1d(torch.cat((tail, xr.mT), dim=-1), w, bias, groups=D)).mT
    (gxr,) = torch.autograd.grad(yr, (xr,), gy)
    assert (y - yr).abs().max().item() < 1e-4 * yr.abs().max().item()
    assert (gx - gxr).abs().max().item() < 1e-4 * gxr.abs().max().item()
