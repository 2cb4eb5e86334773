"""The LRU layer as one op (lru_b200) against the same math in float64 PyTorch: output, carried
state and the gradient of every argument, with and without an initial state, and when only the
carried state is used downstream.  Tolerance ``max|a-b| / max|b| < 1e-4`` (float32 scan over
hundreds of steps, TF32x3 GEMMs)."""

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-4


def _rel(a, b):
    a, b = a.detach(), b.detach()
    if a.is_complex():
        a, b = torch.view_as_real(a), torch.view_as_real(b)
    return (a.double() - b.double()).abs().max().item() / (b.double().abs().max().item() + 1e-30)


def _reference(u, lam, W_in, C_ro, D, x0):
    """lru.py:97-110 with the packed weights: sequential recurrence in float64 / complex128."""
    B, L, d = u.shape
    n = lam.numel()
    v = torch.view_as_complex((u @ W_in.T).reshape(B, L, n, 2).contiguous())
    x = torch.zeros(B, n, dtype=lam.dtype, device=u.device) if x0 is None else x0
    xs = []
    for t in range(L):
        x = lam * x + v[:, t]
        xs.append(x)
    xs = torch.stack(xs, dim=1)
    y = torch.view_as_real(xs).flatten(-2) @ C_ro.T + u @ D.T
    return y, xs[:, -1]


@pytest.mark.parametrize("B,L,d,n,out,with_x0", [(2, 37, 5, 6, 3, False), (3, 300, 16, 24, 16, True), (4, 130, 128, 64, 128, True),
                                                (1, 1, 4, 3, 2, True)])
def test_lru_layer_matches_float64(B, L, d, n, out, with_x0):
    from tsfast_b200 import lru_b200

    gen = torch.Generator(device="cuda").manual_seed(B * 1000 + L)
    r = lambda *s: torch.randn(*s, device="cuda", generator=gen)  # noqa: E731
    lam = (torch.rand(n, device="cuda", generator=gen) * 0.09 + 0.9) * torch.exp(1j * torch.rand(n, device="cuda", generator=gen) * 0.3)
    args32 = [r(B, L, d), lam.to(torch.complex64), r(2 * n, d) / d**0.5, r(out, 2 * n) / n**0.5, r(out, d) / d**0.5,
              (r(B, n) + 1j * r(B, n)).to(torch.complex64) if with_x0 else None]
    args64 = [None if t is None else t.to(torch.complex128 if t.is_complex() else torch.float64) for t in args32]
    for t in (*args32, *args64):
        if t is not None:
            t.requires_grad_()
    gy, gs = r(B, L, out), (r(B, n) + 1j * r(B, n)).to(torch.complex64)

    y, s = lru_b200.lru_layer(*args32)
    ry, rs = _reference(*args64)
    assert _rel(y, ry) < TOL and _rel(s, rs) < TOL
    torch.autograd.backward([y, s], [gy, gs])
    torch.autograd.backward([ry, rs], [gy.double(), gs.to(torch.complex128)])
    for i, (a, b) in enumerate(zip(args32, args64)):
        if a is not None:
            assert _rel(a.grad, b.grad) < TOL, i

    # only the carried state feeds the loss
    for t in (*args32, *args64):
        if t is not None:
            t.grad = None
    _, s = lru_b200.lru_layer(*args32)
    _, rs = _reference(*args64)
    s.backward(gs)
    rs.backward(gs.to(torch.complex128))
    for i, (a, b) in enumerate(zip(args32, args64)):
        if a is not None and b.grad is not None:
            scale = b.grad.abs().max().item()
            got = a.grad if a.grad is not None else torch.zeros_like(a)
            assert (got.to(b.grad.dtype) - b.grad).abs().max().item() <= TOL * max(scale, 1e-6) + 1e-9, i


def test_fake_kernel_and_repeatability():
    from tsfast_b200 import lru_b200

    u = torch.randn(2, 50, 8, device="cuda")
    lam = torch.polar(torch.full((6,), 0.95, device="cuda"), torch.linspace(0, 0.3, 6, device="cuda"))
    W, C, D = torch.randn(12, 8, device="cuda"), torch.randn(4, 12, device="cuda"), torch.randn(4, 8, device="cuda")
    torch.library.opcheck(lru_b200._lru_op, (u, lam, W, C, D, None), test_utils=("test_schema", "test_faketensor"))
    a, b = lru_b200.lru_layer(u, lam, W, C, D), lru_b200.lru_layer(u, lam, W, C, D)
    assert torch.equal(a[0], b[0]) and torch.equal(torch.view_as_real(a[1]), torch.view_as_real(b[1]))
