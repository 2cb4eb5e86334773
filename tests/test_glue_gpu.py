"""LayerNorm and the gated residual (glue_b200) against PyTorch in float64, values and gradients.

Tolerance ``max|a-b| / max|b| < 1e-5`` (these are float32 elementwise / row-reduction kernels); the
weight / bias gradients of LayerNorm, sums over hundreds of thousands of rows, must also repeat bit
for bit (fixed-order partial sums).  Widths cover one to sixteen features per lane and ragged ones.
"""

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

TOL = 1e-5


def _rel(a, b):
    return (a.double() - b.double()).abs().max().item() / (b.double().abs().max().item() + 1e-30)


@pytest.mark.parametrize("shape", [(4, 50, 128), (1000, 32), (3, 7, 100), (257, 512), (2, 1), (5, 33, 20), (100000, 128)])
@pytest.mark.parametrize("affine", [True, False])
def test_layer_norm_matches_float64(shape, affine):
    from tsfast_b200 import glue_b200 as gl

    torch.manual_seed(sum(shape))
    d = shape[-1]
    x = (torch.randn(*shape, device="cuda") * 3 + 1.5).requires_grad_()
    w = torch.randn(d, device="cuda").requires_grad_() if affine else None
    b = torch.randn(d, device="cuda").requires_grad_() if affine else None
    y = gl.layer_norm(x, w, b, 1e-5)
    g = torch.randn_like(y)
    (y * g).sum().backward()
    x64 = x.detach().double().requires_grad_()
    w64 = w.detach().double().requires_grad_() if affine else None
    b64 = b.detach().double().requires_grad_() if affine else None
    y64 = F.layer_norm(x64, (d,), w64, b64, 1e-5)
    (y64 * g.double()).sum().backward()
    assert _rel(y, y64) < TOL
    assert _rel(x.grad, x64.grad) < TOL
    if affine:
        assert _rel(w.grad, w64.grad) < TOL and _rel(b.grad, b64.grad) < TOL
        first = (w.grad.clone(), b.grad.clone())
        w.grad = b.grad = x.grad = None
        (gl.layer_norm(x, w, b, 1e-5) * g).sum().backward()
        assert torch.equal(w.grad, first[0]) and torch.equal(b.grad, first[1])


def test_layer_norm_refuses_what_it_cannot_take():
    from tsfast_b200 import glue_b200 as gl

    assert gl.supports_norm(torch.zeros(4, 600, device="cuda"), (600,)) is not None
    assert gl.supports_norm(torch.zeros(4, 8, 8, device="cuda"), (8, 8)) is not None
    assert gl.supports_norm(torch.zeros(4, 8), (8,)) is not None
    assert gl.supports_norm(torch.zeros(4, 8, device="cuda"), (8,)) is None


@pytest.mark.parametrize("shape", [(6, 40, 128), (1000, 30), (3, 5)])
def test_glu_residual_and_gate_residual(shape):
    from tsfast_b200 import glue_b200 as gl

    torch.manual_seed(1)
    d = shape[-1]
    u = torch.randn(*shape, device="cuda", requires_grad=True)
    z = torch.randn(*shape[:-1], 2 * d, device="cuda", requires_grad=True)
    y = gl.glu_residual(u, z)
    g = torch.randn_like(y)
    (y * g).sum().backward()
    u64, z64 = (t.detach().double().requires_grad_() for t in (u, z))
    y64 = u64 + F.glu(z64, dim=-1)
    (y64 * g.double()).sum().backward()
    assert _rel(y, y64) < TOL and _rel(u.grad, u64.grad) < TOL and _rel(z.grad, z64.grad) < TOL

    a = torch.randn(*shape, device="cuda", requires_grad=True)
    b = torch.randn(*shape, device="cuda", requires_grad=True)
    u.grad = None
    y2 = gl.gate_residual(u, a, b)
    (y2 * g).sum().backward()
    a64, b64 = (t.detach().double().requires_grad_() for t in (a, b))
    u64.grad = None
    y264 = u64 + a64 * torch.sigmoid(b64)
    (y264 * g.double()).sum().backward()
    assert _rel(y2, y264) < TOL
    for t, r in ((u, u64), (a, a64), (b, b64)):
        assert _rel(t.grad, r.grad) < TOL


def test_opcheck():
    from tsfast_b200 import glue_b200 as gl

    x = torch.randn(9, 24, device="cuda", requires_grad=True)
    w = torch.randn(24, device="cuda", requires_grad=True)
    torch.library.opcheck(gl._ln_op, (x, w, None, 1e-5), test_utils=("test_schema", "test_faketensor"))
    z = torch.randn(9, 48, device="cuda", requires_grad=True)
    torch.library.opcheck(gl._glu_res_op, (x, z), test_utils=("test_schema", "test_faketensor"))


@pytest.mark.parametrize("M,D", [(1, 1), (5, 3), (1000, 128), (70001, 256), (4097, 512), (300, 1024), (9, 260), (333, 2000)])
def test_column_sums_match_float64(M, D):
    """Bias gradient of the linear layers: column sums in one pass, reproducible, any width."""
    from tsfast_b200 import glue_b200
    g = torch.randn(M, D, device="cuda")
    got = glue_b200.column_sums(g)
    want = g.double().sum(0)
    assert torch.allclose(got.double(), want, rtol=1e-5, atol=1e-5 * float(want.abs().max() + 1))
    assert torch.equal(got, glue_b200.column_sums(g))
    # a strided view (the half of a wider matrix) and an expanded gradient
    wide = torch.randn(M, 2 * D, device="cuda")
    half = wide[:, D:]
    assert torch.allclose(glue_b200.column_sums(half).double(), half.double().sum(0), rtol=1e-5,
                          atol=1e-5 * float(half.abs().max() * M**0.5 + 1))
    ones = torch.ones(1, D, device="cuda").expand(M, D)
    assert torch.allclose(glue_b200.column_sums(ones), torch.full((D,), float(M), device="cuda"))


def test_linear_bias_gradient_uses_the_column_sum_kernel():
    from tsfast_b200 import glue_b200, proj_b200

    a = torch.randn(3000, 64, device="cuda", requires_grad=True)
    w = torch.randn(96, 64, device="cuda", requires_grad=True)
    b = torch.randn(96, device="cuda", requires_grad=True)
    g = torch.randn(3000, 96, device="cuda")
    before = glue_b200.calls
    proj_b200.linear(a, w, b).backward(g)
    assert glue_b200.calls == before + 1
    assert torch.allclose(b.grad.double(), g.double().sum(0), rtol=1e-5, atol=1e-4)
