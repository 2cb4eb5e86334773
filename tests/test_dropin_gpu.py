"""The drop-in shown on a GPU with tsfast's OWN modules and its OWN test files.

After ``tsfast_b200.install()`` tsfast's DeepLRU, DeepS5, DeepMamba and DynoNet (imported from the
unmodified reference copy that ``oracle/make_ref.py`` places under ``oracle/_ref``) run on CUDA under
``use_backend("auto")`` and are compared with the same modules under ``use_backend("reference")``
in float64: outputs, every parameter gradient, a three-chunk stateful roll-out with gradient through
the carried state, ``torch.compile(fullgraph=True)`` and tsfast's ``GraphedStatefulModel``.  Launch
counters on the B200 modules prove that these kernels, not tsfast's Triton ones, were entered.
The last test runs tsfast's hot-path test files unmodified in a child pytest with the backend
installed from a plugin and requires that none fails.

Tolerances: model outputs and parameter gradients ``max|a-b|/max|b| < 1e-3`` against the float64
reference path, the bound tsfast's own model-level backend tests use
(``tests/test_scan_selective_backends.py:69-95``); scan-level checks stay at ``1e-4`` elsewhere.
"""

import copy
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from conftest import ROOT, import_tsfast_models, reference_checkout

pytestmark = pytest.mark.gpu

MODEL_TOL = 1e-3


def _rel(a, b):
    return (a.double() - b.double()).abs().max().item() / (b.double().abs().max().item() + 1e-30)


@pytest.fixture(scope="module")
def tsfast_installed():
    m = import_tsfast_models()
    import tsfast_b200

    tsfast_b200.install()
    prev = torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    yield m
    torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = prev
    tsfast_b200.uninstall()


def _launches():
    from tsfast_b200 import allpole_b200, conv_b200, mamba_b200
    from tsfast_b200.scan_backends import diagonal_b200, selective_b200

    return {"diag": diagonal_b200.calls, "sel": selective_b200.calls, "ssm": mamba_b200.calls,
            "conv": conv_b200.calls, "allpole": allpole_b200.calls}


def _build(m, family):
    torch.manual_seed(0)
    if family == "lru":
        return m.DeepLRU(3, 2, d_model=32, d_state=48, n_layers=2, return_state=True), "diag"
    if family == "s5":
        return m.DeepS5(3, 2, d_model=32, d_state=32, n_layers=2, return_state=True), "diag"
    if family == "mamba":
        return m.DeepMamba(3, 2, d_model=32, d_state=16, n_layers=2, return_state=True), "ssm"
    return m.DynoNet(3, 2, n_channels=4, nb=4, na=2, return_state=True), "allpole"


def _chunked(model, u, cuts):
    """Roll the model over ``u`` in chunks, handing the state over; gradient flows through it."""
    outs, state, lo = [], None, 0
    for hi in list(cuts) + [u.shape[1]]:
        y, state = model(u[:, lo:hi], state=state)
        outs.append(y)
        lo = hi
    return torch.cat(outs, dim=1)


@pytest.mark.parametrize("family", ["lru", "s5", "mamba", "dynonet"])
def test_tsfast_models_on_b200_kernels_match_float64_reference(tsfast_installed, family):
    m = tsfast_installed
    from tsfast.models import use_backend

    model32, counter = _build(m, family)
    if family == "dynonet":  # dynoNet starts with a = 0; give the poles something to do
        torch.manual_seed(1)
        with torch.no_grad():
            for name, p in model32.named_parameters():
                if name.endswith("a_coeff"):
                    p.normal_(0, 0.2)
    model64 = copy.deepcopy(model32).double()
    model32, model64 = model32.cuda(), model64.cuda()
    torch.manual_seed(2)
    u = torch.randn(4, 96, 3, device="cuda")
    cuts = (40, 43)  # second chunk is shorter than the conv window / filter order of some models

    before = _launches()[counter]
    with use_backend("auto"):
        got = _chunked(model32, u, cuts)
        (got**2).mean().backward()
    assert _launches()[counter] > before, f"the B200 {counter} backend was never entered"
    with use_backend("reference"):
        want = _chunked(model64, u.double(), cuts)
        (want**2).mean().backward()

    assert _rel(got, want) < MODEL_TOL
    worst = ("", 0.0)
    for (name, p), q in zip(model32.named_parameters(), model64.parameters()):
        assert p.grad is not None, name
        r = _rel(p.grad, q.grad)
        if r > worst[1]:
            worst = (name, r)
    assert worst[1] < MODEL_TOL, f"{family}: worst parameter gradient {worst}"
    with use_backend("auto"), torch.no_grad():  # inference path equals the autograd path
        again = _chunked(model32, u, cuts)
    assert _rel(again, got) < 1e-6


@pytest.mark.parametrize("family", ["lru", "s5", "mamba"])
def test_projections_on_tensor_cores_match_float64_reference(tsfast_installed, family):
    """install(fuse_projections=True) + accelerate_linears(model): tsfast's own model with every GEMM of the
    step (boundary projections, encoder/decoder, GLU, Mamba's in/x/dt/out projections) on the tcgen05
    kernel, against the float64 reference path: output and every parameter gradient."""
    m = tsfast_installed
    import tsfast_b200
    from tsfast.models import use_backend
    from tsfast_b200 import prologue_b200, proj_b200

    torch.manual_seed(0)
    if family == "lru":
        model32 = m.DeepLRU(3, 2, d_model=64, d_state=96, n_layers=2, return_state=True)
    elif family == "s5":
        model32 = m.DeepS5(3, 2, d_model=64, d_state=64, n_layers=2, return_state=True)
    else:
        model32 = m.DeepMamba(3, 2, d_model=64, d_state=16, n_layers=2, return_state=True)
    model64 = copy.deepcopy(model32).double().cuda()
    model32 = model32.cuda()
    u = torch.randn(4, 200, 3, device="cuda")
    tsfast_b200.install(fuse_projections=True)
    n_lin = tsfast_b200.accelerate_linears(model32)
    assert n_lin >= 2
    before, before_prologue = proj_b200.calls, prologue_b200.calls
    try:
        with use_backend("auto"):
            got = _chunked(model32, u, (90,))
            (got**2).mean().backward()
        used = proj_b200.calls - before
        assert used >= 6 * n_lin // 2, f"only {used} launches of the projection kernels"
        if family in ("lru", "s5"):  # eigenvalues / discretisation: one launch forward and one backward per layer and chunk
            assert prologue_b200.calls - before_prologue >= 2 * 2, "the parameter prologue kernels did not run"
        with use_backend("reference"):
            want = _chunked(model64, u.double(), (90,))
            (want**2).mean().backward()
        assert _rel(got, want) < MODEL_TOL
        for (name, p), q in zip(model32.named_parameters(), model64.parameters()):
            assert p.grad is not None, name
            assert _rel(p.grad, q.grad) < MODEL_TOL, name
    finally:
        assert tsfast_b200.restore_linears(model32) == n_lin
        tsfast_b200.uninstall()
        tsfast_b200.install()  # the module fixture keeps the scan backends installed
    with use_backend("auto"), torch.no_grad():
        before = proj_b200.calls
        model32(u)
        assert proj_b200.calls == before, "the projections were not restored"


@pytest.mark.parametrize("kw", [dict(discretization="bilinear"), dict(clip_eigs=True), dict(conj_sym=False),
                                dict(step_rescale=0.5, discretization="bilinear", clip_eigs=True),
                                dict(C_init="complex_normal", conj_sym=False, step_rescale=2.0)])
def test_s5_layer_variants_through_the_fused_path(tsfast_installed, kw):
    """tsfast's S5 layer in its other configurations (bilinear map, clipped eigenvalues, full state
    without conjugate symmetry, rescaled step) with install(fuse_projections=True): the discretisation
    kernel, the packed input projection, the scan and the readout against the float64 reference path,
    output, carried state and every parameter gradient."""
    import tsfast_b200
    from tsfast.models import use_backend
    from tsfast.models.architectures.s5 import S5
    from tsfast_b200 import prologue_b200

    torch.manual_seed(1)
    layer32 = S5(24, 16, **kw)
    layer64 = copy.deepcopy(layer32).double().cuda()
    layer32 = layer32.cuda()
    if kw.get("clip_eigs"):  # push some eigenvalues over the clip so that the clamp and its cut gradient are exercised
        with torch.no_grad():
            layer32.Lambda_re[::3] = 0.02
            layer64.Lambda_re[::3] = 0.02
    u = torch.randn(3, 150, 24, device="cuda")
    g = torch.randn(3, 150, 24, device="cuda")
    tsfast_b200.install(fuse_projections=True)
    try:
        before = prologue_b200.calls
        with use_backend("auto"):
            y1, s1 = layer32(u[:, :70], return_state=True)
            y2, s2 = layer32(u[:, 70:], state=s1, return_state=True)
            got = torch.cat((y1, y2), dim=1)
            (got * g).sum().backward()
        assert prologue_b200.calls - before == 4, "two chunks: two discretisations forward, two backward"
        with use_backend("reference"):
            r1, t1 = layer64(u[:, :70].double(), return_state=True)
            r2, t2 = layer64(u[:, 70:].double(), state=t1, return_state=True)
            want = torch.cat((r1, r2), dim=1)
            (want * g.double()).sum().backward()
        assert _rel(got, want) < MODEL_TOL and _rel(torch.view_as_real(s2), torch.view_as_real(t2)) < MODEL_TOL
        for (name, p), q in zip(layer32.named_parameters(), layer64.parameters()):
            assert p.grad is not None, name
            assert _rel(p.grad, q.grad) < MODEL_TOL, (name, kw)
    finally:
        tsfast_b200.uninstall()
        tsfast_b200.install()  # the module fixture keeps the scan backends installed


def test_reference_preference_bypasses_b200(tsfast_installed):
    m = tsfast_installed
    from tsfast.models import use_backend

    model, counter = _build(m, "lru")
    model = model.cuda()
    u = torch.randn(2, 30, 3, device="cuda")
    before = _launches()
    with use_backend("reference"), torch.no_grad():
        model(u)
    assert _launches() == before
    with use_backend("triton"), torch.no_grad():  # the family name install() registers under
        model(u)
    assert _launches()[counter] > before[counter]


@pytest.mark.parametrize("family", ["lru", "mamba"])
def test_compile_fullgraph_through_tsfast_modules(tsfast_installed, family):
    m = tsfast_installed
    model, counter = _build(m, family)
    model = model.cuda()
    model.return_state = False
    u = torch.randn(2, 64, 3, device="cuda")
    eager = model(u)
    before = _launches()[counter]
    out = torch.compile(model, fullgraph=True)(u)
    out.square().mean().backward()
    assert _launches()[counter] > before
    assert _rel(out, eager) < 1e-5
    assert all(p.grad is not None for p in model.parameters())


@pytest.mark.parametrize("family", ["lru", "mamba"])
def test_graphed_stateful_model_of_tsfast(tsfast_installed, family):
    """tsfast's own CUDA-graph wrapper (flat state bridge, make_graphed_callables) around its own
    model, running on these kernels: every replay equals eager, output and parameter gradients.

    Gradients are compared step by step with ``.grad`` reset to None in between, as a training loop
    does: a replayed backward returns its static gradient buffers, so accumulating over replays is
    not something graphed callables support.  The Mamba model hands its (real) state from step to
    step; for the LRU model every step starts from a zero state, because tsfast's flat-state bridge
    stages the state in a float32 buffer and so drops the imaginary part of a complex state whatever
    kernel computes it."""
    m = tsfast_installed
    from tsfast.models._core.cudagraph import GraphedStatefulModel
    from tsfast.models._core.state import detach_state

    model, counter = _build(m, family)
    model = model.cuda()
    eager = copy.deepcopy(model)
    graphed = GraphedStatefulModel(model)
    torch.manual_seed(5)
    before = _launches()[counter]
    state_g = state_e = None
    for step in range(3):
        u = torch.randn(4, 50, 3, device="cuda")
        for mod in (model, eager):
            for p in mod.parameters():
                p.grad = None
        yg, new_g = graphed(u, state_g)
        ye, new_e = eager(u, state=state_e)
        assert _rel(yg, ye) < 1e-5, step
        yg.square().mean().backward()
        ye.square().mean().backward()
        for (name, p), q in zip(model.named_parameters(), eager.parameters()):
            assert _rel(p.grad, q.grad) < 1e-4, (step, name)
        if family == "mamba":
            state_g, state_e = detach_state(new_g), detach_state(new_e)
            for a, b in zip(torch.utils._pytree.tree_leaves(state_g), torch.utils._pytree.tree_leaves(state_e)):
                assert _rel(a, b) < 1e-5, step
    assert not graphed._capture_failed, "tsfast fell back to eager: the capture failed"
    assert graphed._graphed is not None
    assert _launches()[counter] > before


def test_tsfast_own_test_files_pass_with_b200_installed(tmp_path):
    """tsfast's hot-path test files, unmodified, in a child pytest with the backend installed."""
    ref = reference_checkout()
    if ref is None or not (ref / "tests" / "test_scan.py").exists():
        pytest.skip("no reference copy with its tests (python oracle/make_ref.py <checkout>)")
    report = tmp_path / "report.json"
    env = dict(os.environ, B200_DROPIN_REPORT=str(report), CXX="/usr/bin/g++", CC="/usr/bin/gcc", TSFAST_AUTOTUNE_CACHE="1",
               PYTHONPATH=os.pathsep.join([str(ref), str(ROOT), str(ROOT / "tests"), os.environ.get("PYTHONPATH", "")]))
    files = sorted(str(p) for p in (ref / "tests").glob("test_*.py"))
    cmd = [sys.executable, "-m", "pytest", "-q", "--no-header", "-p", "ref_plugin", "-p", "no:cacheprovider",
           "--rootdir", str(ref), "-c", os.devnull, *files]
    r = subprocess.run(cmd, env=env, cwd=str(ref), capture_output=True, text=True, timeout=2400)
    tail = (r.stdout + r.stderr)[-4000:]
    assert report.exists(), tail
    rep = json.loads(report.read_text())
    if os.environ.get("B200_REPORT_DIR") and Path(os.environ["B200_REPORT_DIR"]).is_dir():  # keep the record as files
        out_dir = Path(os.environ["B200_REPORT_DIR"])
        (out_dir / "reference_tests_with_b200.json").write_text(json.dumps(rep, indent=1))
        (out_dir / "reference_tests_with_b200.log").write_text((r.stdout + r.stderr)[-60000:])
    assert rep["failed"] == 0 and r.returncode == 0, (rep, tail)
    assert rep["passed"] > 100
    for slot in ("scan.diagonal", "scan.selective", "mamba.ssm", "mamba.conv", "dynonet.allpole"):
        assert rep["launches"][slot] > 0, f"{slot}: tsfast's tests never reached the B200 module"
