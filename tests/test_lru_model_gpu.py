"""The DeepLRU caller stack on the B200 scan against the reference's own DeepLRU.

`tests/golden/deeplru.npz` holds a small reference model (float64, `use_backend("reference")`):
parameters, input, output, carried states and every parameter gradient.  The mirror in
`tests/mirrors.py` loads that state_dict unchanged and must reproduce all of it in float32
(bound 1e-4 relative, TF32 off as in the reference's model-level parity tests,
tests/test_lru.py:157-170), and a chunked rollout with the carried state must equal one pass."""

import numpy as np
import pytest
import torch

from conftest import GOLDEN, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture
def golden_model():
    from mirrors import DeepLRU

    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    d = dict(np.load(GOLDEN / "deeplru.npz"))
    model = DeepLRU(2, 3, d_model=8, d_state=6, n_layers=2, return_state=True)
    sd = {k[len("param/"):]: torch.from_numpy(v).float() for k, v in d.items() if k.startswith("param/")}
    model.load_state_dict(sd, strict=True)  # same parameter names and shapes as tsfast's DeepLRU
    return model.cuda(), d


def test_matches_reference_model(golden_model):
    model, d = golden_model
    u = torch.from_numpy(d["u"]).float().cuda()
    g = torch.from_numpy(d["g"]).float().cuda()
    y, states = model(u)
    (y * g).sum().backward()
    assert rel_err(y.detach().cpu().numpy(), d["y"]) < 1e-4
    for i, s in enumerate(states):
        assert rel_err(s.detach().cpu().numpy(), d[f"state{i}"]) < 1e-4
    for k, p in model.named_parameters():
        assert rel_err(p.grad.cpu().numpy(), d[f"grad/{k}"]) < 2e-4, k


def test_chunked_rollout_equals_one_pass(golden_model):
    model, d = golden_model
    u = torch.from_numpy(d["u"]).float().cuda()
    with torch.no_grad():
        y_full, _ = model(u)
        y1, st = model(u[:, :17])
        y2, st = model(u[:, 17:18], st)
        y3, _ = model(u[:, 18:], st)
    assert rel_err(torch.cat((y1, y2, y3), 1).cpu().numpy(), y_full.cpu().numpy()) < 1e-5


def test_config5_shape_gradient_is_a_descent_direction():
    """The C5 architecture (4 blocks, width 128, 256 complex states) on a reduced batch: the
    gradient through the whole stack matches a central finite difference along itself (5 %), and a
    data-parallel step with a small learning rate lowers the loss."""
    from tsfast_b200.dist import dp_train_step
    from mirrors import DeepLRU

    torch.backends.cuda.matmul.allow_tf32 = False
    torch.manual_seed(0)
    model = DeepLRU(1, 1, d_model=128, d_state=256, n_layers=4, r_min=0.5, r_max=0.99, max_phase=0.5).cuda()
    x = torch.randn(8, 2000, 1, device="cuda") * 0.1
    yt = torch.tanh(torch.cumsum(x, 1) * 0.05)
    loss_of = lambda: torch.nn.functional.mse_loss(model(x), yt)  # noqa: E731
    params = list(model.parameters())
    loss0 = loss_of()
    grads = torch.autograd.grad(loss0, params)
    gnorm = torch.sqrt(sum((g.double() ** 2).sum() for g in grads)).item()
    assert np.isfinite(gnorm) and gnorm > 0
    eps = 1e-2 / gnorm
    with torch.no_grad():
        for sign, store in ((+1, "p"), (-2, "m")):
            for p, g in zip(params, grads):
                p.add_(g, alpha=sign * eps)
            if store == "p":
                lp = loss_of().item()
            else:
                lm = loss_of().item()
        for p, g in zip(params, grads):
            p.add_(g, alpha=eps)  # back to the start
    fd = (lp - lm) / (2 * eps)
    assert abs(fd - gnorm**2) < 0.05 * gnorm**2, (fd, gnorm**2)
    opt = torch.optim.SGD(model.parameters(), lr=0.05 / gnorm**2 * loss0.item())
    dp_train_step(model, opt, torch.nn.functional.mse_loss, x, yt)
    assert loss_of().item() < loss0.item()
