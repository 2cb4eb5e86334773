"""The tensor-core projection GEMM (b200_proj_gemm) and the two boundary-projection functions built on it.

Oracle: the same products in float64 (``torch.matmul`` on float64 copies, which is what the reference's
``complex_in_proj`` / ``real_out_proj`` compute, ``tsfast/models/_core/scan.py:272-313``).  Tolerance:
``max|a-b| / max|b| < 1e-5`` per tensor, the float32-faithful bound of the split-TF32 arithmetic (a plain
TF32 GEMM sits at about 1e-3 and would fail); PyTorch's own float32 GEMM error is printed beside ours.
Shapes cover ragged M, N and K (partial tiles and blocks), one to many K-blocks, strided row pitches, the
bias and two-product forms, the token-major weight-gradient kernel and the projection functions with autograd.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-5


def _rel(a, b):
    return (a.double() - b.double()).abs().max().item() / (b.double().abs().max().item() + 1e-30)


@pytest.fixture(autouse=True)
def _no_tf32():
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32 = prev


@pytest.mark.parametrize("M,N,K", [(128, 128, 32), (1000, 512, 128), (257, 64, 32), (4096, 128, 512), (77, 200, 96),
                                   (1, 24, 64), (130, 136, 160), (500, 512, 16), (333, 34, 64), (64, 7, 2), (300, 48, 50)])
def test_single_product_matches_float64(M, N, K):
    from tsfast_b200 import proj_b200 as pj

    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda")
    w = torch.randn(N, K, device="cuda") / K**0.5
    got = pj.linear(a, w)
    want = a.double() @ w.double().t()
    torch.cuda.synchronize()
    err, torch_err = _rel(got, want), _rel(a @ w.t(), want)
    print(f"[{M}x{N}x{K}] b200 {err:.2e}  torch float32 {torch_err:.2e}")
    assert got.shape == (M, N)
    assert err < TOL


def test_values_spanning_many_magnitudes():
    """The head/tail split must hold for operands of very different sizes in one product."""
    from tsfast_b200 import proj_b200 as pj

    torch.manual_seed(0)
    a = torch.randn(512, 128, device="cuda") * torch.logspace(-6, 6, 128, device="cuda")
    w = torch.randn(64, 128, device="cuda") * torch.logspace(6, -6, 128, device="cuda")
    assert _rel(pj.linear(a, w), a.double() @ w.double().t()) < TOL


def test_strided_rows_are_read_in_place():
    """A column slice of a wider matrix (row pitch > K) goes through without a copy and is exact."""
    from tsfast_b200 import proj_b200 as pj

    torch.manual_seed(1)
    wide = torch.randn(300, 256, device="cuda")
    a = wide[:, 64:192]
    w = torch.randn(96, 128, device="cuda")
    assert pj._rows(a).data_ptr() == a.data_ptr()
    assert _rel(pj.linear(a, w), a.double() @ w.double().t()) < TOL


def test_two_products_in_one_pass():
    from tsfast_b200 import proj_b200 as pj

    torch.manual_seed(2)
    a1, w1 = torch.randn(700, 256, device="cuda"), torch.randn(128, 256, device="cuda") / 16
    a2, w2 = torch.randn(700, 64, device="cuda"), torch.randn(128, 64, device="cuda") / 8
    got = pj._proj_gemm2_op(a1, w1, a2, w2)
    want = a1.double() @ w1.double().t() + a2.double() @ w2.double().t()
    assert _rel(got, want) < TOL


def test_bias_and_wrong_operands():
    from tsfast_b200 import proj_b200 as pj

    torch.manual_seed(4)
    a, w, b = torch.randn(90, 20, device="cuda"), torch.randn(33, 20, device="cuda"), torch.randn(33, device="cuda")
    want = a.double() @ w.double().t() + b.double()
    assert _rel(pj.linear(a, w, b), want) < TOL
    assert "float32" in pj.supports(a.double(), w)
    with pytest.raises(RuntimeError, match="product"):
        pj.linear(a, w[:, :8].contiguous())


@pytest.mark.parametrize("M,N,K", [(4096, 512, 128), (1000, 128, 512), (77, 48, 16), (31, 130, 200), (100000, 64, 32)])
def test_weight_gradient_kernel(M, N, K):
    """dW = G^T A over the token axis (both operands read token-major in place), against float64."""
    from tsfast_b200 import proj_b200 as pj

    torch.manual_seed(M + K)
    g, a = torch.randn(M, N, device="cuda"), torch.randn(M, K, device="cuda")
    got = pj._proj_wgrad_op(g, a)
    want = g.double().t() @ a.double()
    err, torch_err = _rel(got, want), _rel(g.t() @ a, want)
    print(f"wgrad [{M}x{N}x{K}] b200 {err:.2e}  torch float32 {torch_err:.2e}")
    assert err < TOL
    assert torch.equal(got, pj._proj_wgrad_op(g, a))  # slices are added in a fixed order


def test_linear_autograd_matches_float64():
    from tsfast_b200 import proj_b200 as pj

    torch.manual_seed(5)
    a = torch.randn(6, 70, 96, device="cuda", requires_grad=True)
    w = torch.randn(40, 96, device="cuda", requires_grad=True)
    b = torch.randn(40, device="cuda", requires_grad=True)
    y = pj.linear(a, w, b)
    g = torch.randn_like(y)
    (y * g).sum().backward()
    a64, w64, b64 = (t.detach().double().requires_grad_() for t in (a, w, b))
    y64 = torch.nn.functional.linear(a64, w64, b64)
    (y64 * g.double()).sum().backward()
    assert _rel(y, y64) < TOL
    for name, t, r in (("a", a, a64), ("w", w, w64), ("b", b, b64)):
        assert _rel(t.grad, r.grad) < TOL, name


def test_projection_functions_with_autograd():
    """complex_in_proj / real_out_proj against the float64 complex formulas, values and gradients."""
    from tsfast_b200 import proj_b200 as pj

    torch.manual_seed(3)
    Bn, L, d, n, o = 3, 50, 64, 48, 32
    u = torch.randn(Bn, L, d, device="cuda", requires_grad=True)
    B_re, B_im = (torch.randn(n, d, device="cuda", requires_grad=True) for _ in range(2))
    C_re, C_im = (torch.randn(o, 2 * 16, device="cuda", requires_grad=True) for _ in range(2))
    v = pj.complex_in_proj(u, B_re, B_im)
    x = v[..., :32]  # any complex sequence will do for the readout
    y = pj.real_out_proj(x.contiguous(), C_re, C_im)
    D = torch.randn(o, d, device="cuda", requires_grad=True)
    y2 = pj.readout(x.contiguous(), C_re, C_im, u, D)
    assert _rel(y2, y.double() + u.double() @ D.double().t()) < TOL
    g_v, g_y = torch.randn_like(v), torch.randn_like(y)
    (torch.view_as_real(v) * torch.view_as_real(g_v)).sum().backward(retain_graph=True)
    (y * g_y).sum().backward()
    got = [t.grad.clone() for t in (u, B_re, B_im, C_re, C_im)]

    u64, Br, Bi, Cr, Ci = (t.detach().double().requires_grad_() for t in (u, B_re, B_im, C_re, C_im))
    v64 = u64.to(torch.complex128) @ torch.complex(Br, Bi).mT
    y64 = (v64[..., :32] @ torch.complex(Cr, Ci).mT).real
    (torch.view_as_real(v64) * torch.view_as_real(g_v).double()).sum().backward(retain_graph=True)
    (y64 * g_y.double()).sum().backward()
    assert _rel(torch.view_as_real(v), torch.view_as_real(v64)) < TOL
    assert _rel(y, y64) < TOL
    for name, a, b in zip(("u", "B_re", "B_im", "C_re", "C_im"), got, (u64, Br, Bi, Cr, Ci)):
        assert _rel(a, b.grad) < 2e-5, name


def test_status_word_is_clean_and_graph_capture_works():
    from tsfast_b200 import _lib, proj_b200 as pj

    a, w = torch.randn(640, 128, device="cuda"), torch.randn(256, 128, device="cuda")
    L_ = _lib.lib()
    ws = _lib.workspace(L_.b200_proj_gemm_workspace_bytes(256, 128, 0), a.device)
    out = torch.empty(640, 256, device="cuda")
    rc = L_.b200_proj_gemm(640, 256, 128, a.data_ptr(), 128, w.data_ptr(), 128, 0, None, 0, None, 0, None, out.data_ptr(), 256,
                           ws.data_ptr(), ws.numel(), _lib.stream_ptr(a.device))
    assert rc == 0 and _lib.workspace_status(ws) == 0
    want = pj.linear(a, w)
    assert torch.equal(out, want)
    g = torch.cuda.CUDAGraph()
    static_a = a.clone()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        pj.linear(static_a, w)
    torch.cuda.current_stream().wait_stream(s)
    with torch.cuda.graph(g):
        static_out = pj.linear(static_a, w)
    static_a.copy_(a * 2)
    g.replay()
    torch.cuda.synchronize()
    assert _rel(static_out, 2 * want) < 1e-6
