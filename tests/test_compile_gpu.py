"""The custom ops compose with torch.compile without graph breaks, forward and backward (the
reference checks the same for its ops: tests/test_scan_dispatch.py:102-112, tests/test_mamba.py:
331-344, tests/test_dynonet.py:246-265).  `aot_eager` keeps code generation out of the test: what
is verified is tracing through the fake implementations and the registered adjoints."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(fn, args, grads_of):
    for a in grads_of:
        a.grad = None
    eager = fn(*args)
    eager.sum().backward()
    want = [a.grad.clone() for a in grads_of]
    for a in grads_of:
        a.grad = None
    compiled = torch.compile(fn, fullgraph=True, backend="aot_eager")
    got = compiled(*args)
    got.sum().backward()
    assert torch.allclose(got, eager, rtol=1e-5, atol=1e-6)
    for a, w in zip(grads_of, want):
        assert torch.allclose(a.grad, w, rtol=1e-4, atol=1e-5)


def test_diagonal_and_selective_ops_fullgraph():
    import tsfast_b200 as tb

    torch.manual_seed(0)
    lam = (torch.rand(12, device="cuda") * 0.9).requires_grad_()
    v = torch.randn(3, 50, 12, device="cuda", requires_grad=True)
    x0 = torch.randn(3, 12, device="cuda", requires_grad=True)
    _check(lambda l, v_, x: tb.diagonal_recurrence(l, v_, x) * 2.0, (lam, v, x0), (lam, v, x0))
    a = (torch.rand(3, 50, 12, device="cuda") * 0.9).requires_grad_()
    _check(lambda a_, v_: tb.selective_recurrence(torch.sigmoid(a_), v_).tanh(), (a, v), (a, v))


def test_mamba_and_allpole_ops_fullgraph():
    from tsfast_b200 import allpole_b200, mamba_b200

    torch.manual_seed(1)
    r = lambda *s: torch.randn(*s, device="cuda")  # noqa: E731
    B, L, D, N = 2, 40, 24, 16
    ins = [(r(B, L, D) * 0.5 - 1).requires_grad_(), (-torch.exp(r(D, N) * 0.3)).requires_grad_(), r(B, L, N).requires_grad_(),
           r(B, L, N).requires_grad_(), r(B, L, D).requires_grad_(), r(B, L, D).requires_grad_(), r(D).requires_grad_(),
           r(B, D, N).requires_grad_()]

    def f(*t):
        out, hl = mamba_b200.run(*t)
        return out.sum(-1) + hl.sum()

    _check(f, ins, ins)
    a, w, y0 = (r(5, 3) * 0.2).requires_grad_(), r(4, 5, 90).requires_grad_(), r(4, 5, 3).requires_grad_()
    _check(lambda a_, w_, y_: allpole_b200.run(a_, w_, y_), (a, w, y0), (a, w, y0))


def test_non_contiguous_inputs_are_densified_inside_the_ops():
    """Strided views (a transposed batch, an expanded lam) must give what their dense copies give
    (reference: `.contiguous()` inside every op, _core/scan.py:102-103,122-125)."""
    import tsfast_b200 as tb

    torch.manual_seed(2)
    v = torch.randn(40, 3, 16, device="cuda").transpose(0, 1)  # [3, 40, 16], non-contiguous
    lam = (torch.rand(1, 16, device="cuda") * 0.9).expand(3, 16)  # stride-0 batch axis
    assert not v.is_contiguous() and not lam.is_contiguous()
    assert torch.equal(tb.diagonal_recurrence(lam, v), tb.diagonal_recurrence(lam.contiguous(), v.contiguous()))
    a = (torch.rand(40, 3, 16, device="cuda") * 0.9).transpose(0, 1)
    assert torch.equal(tb.selective_recurrence(a, v), tb.selective_recurrence(a.contiguous(), v.contiguous()))
