"""Parameter prologues of the LRU and S5 layers (prologue_b200) against the reference's formulas in
float64 through autograd: values and the gradient of every parameter.

The formulas restated here are ``LRU.eigenvalues`` + the gamma scaling (``architectures/lru.py:79-83,
97-99``) and ``S5.discretize`` (``architectures/s5.py:154-170``).  Tolerance ``max|a-b| / max|b| < 2e-5``
(float32 exp / sincos chains against float64)."""

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 2e-5


def _rel(a, b):
    a, b = a.detach().cpu(), b.detach().cpu()
    if a.is_complex():
        a, b = torch.view_as_real(a), torch.view_as_real(b)
    return (a.double() - b.double()).abs().max().item() / (b.double().abs().max().item() + 1e-30)


def _lru_ref(nu_log, theta_log, gamma_log, B_re, B_im):
    lam_abs = torch.exp(-torch.exp(nu_log))
    phase = torch.exp(theta_log)
    lam = torch.complex(lam_abs * torch.cos(phase), lam_abs * torch.sin(phase))
    g = torch.exp(gamma_log).unsqueeze(-1)
    n, d = B_re.shape
    return lam, torch.stack((g * B_re, g * B_im), dim=1).reshape(2 * n, d)


def _s5_ref(L_re, L_im, log_step, B_re, B_im, discretization, clip_eigs, step_rescale):
    lam_re = torch.clamp(L_re, max=-1e-4) if clip_eigs else L_re
    lam = torch.complex(lam_re, L_im)
    step = step_rescale * torch.exp(log_step)
    B_tilde = torch.complex(B_re, B_im)
    if discretization == "zoh":
        lam_bar = torch.exp(lam * step)
        B_bar = ((lam_bar - 1) / lam).unsqueeze(-1) * B_tilde
    else:
        bl = 1 / (1 - (step / 2) * lam)
        lam_bar = bl * (1 + (step / 2) * lam)
        B_bar = (bl * step).unsqueeze(-1) * B_tilde
    p, d = B_re.shape
    return lam_bar, torch.stack((B_bar.real, B_bar.imag), dim=1).reshape(2 * p, d)


def _check(fn32, fn64, params32):
    gen = torch.Generator(device="cuda").manual_seed(7)
    p32 = [t.clone().requires_grad_() for t in params32]
    p64 = [t.double().clone().requires_grad_() for t in params32]
    lam, W = fn32(*p32)
    rlam, rW = fn64(*p64)
    assert _rel(lam, rlam) < TOL and _rel(W, rW) < TOL
    glam = torch.randn(lam.shape, device="cuda", generator=gen) + 1j * torch.randn(lam.shape, device="cuda", generator=gen)
    gW = torch.randn(W.shape, device="cuda", generator=gen)
    for pick in ((glam, gW), (glam, None), (None, gW)):
        for t in (*p32, *p64):
            t.grad = None
        lam, W = fn32(*p32)
        rlam, rW = fn64(*p64)
        outs, routs, gs, rgs = [], [], [], []
        if pick[0] is not None:
            outs.append(lam), routs.append(rlam), gs.append(glam.to(torch.complex64)), rgs.append(glam.to(torch.complex128))
        if pick[1] is not None:
            outs.append(W), routs.append(rW), gs.append(gW), rgs.append(gW.double())
        torch.autograd.backward(outs, gs)
        torch.autograd.backward(routs, rgs)
        for i, (a, b) in enumerate(zip(p32, p64)):
            ga = a.grad if a.grad is not None else torch.zeros_like(a)
            gb = b.grad if b.grad is not None else torch.zeros_like(b)
            scale = gb.abs().max().item()
            assert (ga.double() - gb).abs().max().item() <= TOL * max(scale, 1e-3) + 1e-7, (i, pick[0] is None, pick[1] is None)


@pytest.mark.parametrize("n,d", [(1, 1), (7, 3), (64, 40), (256, 128), (300, 5)])
def test_lru_prologue_values_and_gradients(n, d):
    from tsfast_b200 import prologue_b200

    gen = torch.Generator(device="cuda").manual_seed(n * 1000 + d)
    u1, u2 = torch.rand(n, device="cuda", generator=gen), torch.rand(n, device="cuda", generator=gen)
    nu_log = torch.log(-0.5 * torch.log(u1 * (0.999**2 - 0.9**2) + 0.9**2))
    theta_log = torch.log(0.314 * u2 + 1e-3)
    gamma_log = 0.5 * torch.log(1 - torch.exp(-torch.exp(nu_log)).square())
    B_re, B_im = torch.randn(n, d, device="cuda", generator=gen), torch.randn(n, d, device="cuda", generator=gen)
    _check(prologue_b200.lru_prologue, _lru_ref, [nu_log, theta_log, gamma_log, B_re, B_im])


@pytest.mark.parametrize("clip", [False, True])
@pytest.mark.parametrize("disc", ["zoh", "bilinear"])
@pytest.mark.parametrize("p,d", [(1, 1), (9, 4), (128, 64), (200, 33)])
def test_s5_discretize_values_and_gradients(p, d, disc, clip):
    from tsfast_b200 import prologue_b200

    gen = torch.Generator(device="cuda").manual_seed(p * 100 + d)
    L_re = -0.5 - torch.rand(p, device="cuda", generator=gen)
    if clip and p > 2:
        L_re[::3] = 0.01  # above the clip: the value is clamped and the gradient is cut
    L_im = torch.randn(p, device="cuda", generator=gen) * 3
    log_step = torch.log(torch.rand(p, device="cuda", generator=gen) * 0.099 + 0.001)
    B_re, B_im = torch.randn(p, d, device="cuda", generator=gen), torch.randn(p, d, device="cuda", generator=gen)

    def ours(*ps):
        return prologue_b200.s5_discretize(*ps, discretization=disc, clip_eigs=clip, step_rescale=0.7)

    def ref(*ps):
        return _s5_ref(*ps, disc, clip, 0.7)

    _check(ours, ref, [L_re, L_im, log_step, B_re, B_im])


def test_fake_kernels_and_compile():
    from tsfast_b200 import prologue_b200

    n, d = 16, 8
    ps = [torch.randn(n, device="cuda") * 0.1 - 1 for _ in range(3)] + [torch.randn(n, d, device="cuda") for _ in range(2)]
    torch.library.opcheck(prologue_b200._lru_op, tuple(ps), test_utils=("test_schema", "test_faketensor"))
    torch.library.opcheck(prologue_b200._s5_op, (*ps, 0, True, 1.0), test_utils=("test_schema", "test_faketensor"))

    @torch.compile(fullgraph=True)
    def f(*q):
        lam, W = prologue_b200.lru_prologue(*q)
        return lam.abs().sum() + W.sum()

    assert torch.allclose(f(*ps), (lambda lw: lw[0].abs().sum() + lw[1].sum())(prologue_b200.lru_prologue(*ps)))
