"""Pin the CPU oracle against golden vectors produced by the reference itself (CPU only).

float64 oracle vs the reference's float64 pure-PyTorch paths: agreement to ~1e-9 relative (the
doubling scans and the sequential sweep differ only in summation order).  float32 oracle vs the
same truth: inside the 1e-4 relative bound the reference's own backend tests use
(tests/test_scan_diagonal_backends.py:29-65 of the reference).
"""

import numpy as np
import pytest

from conftest import load_golden, rel_err

TOL64 = 1e-9
TOL32 = 1e-4


def _cast(x, f64):
    if x is None:
        return None
    if np.iscomplexobj(x):
        return x.astype(np.complex128 if f64 else np.complex64)
    return x.astype(np.float64 if f64 else np.float32)


@pytest.mark.parametrize("f64", [True, False])
@pytest.mark.parametrize("kind", ["diag", "sel"])
def test_diagonal_scans(oracle, kind, f64):
    fwd = oracle.diag_fwd if kind == "diag" else oracle.sel_fwd
    bwd = oracle.diag_bwd if kind == "diag" else oracle.sel_bwd
    tol = TOL64 if f64 else TOL32
    for c in load_golden(kind):
        lam, v, x0, g = (_cast(t, f64) for t in (c.lam, c.v, c.x0, c.g))
        M, L, N = v.shape
        lam_lane = np.ascontiguousarray(np.broadcast_to(lam, (M, N))) if kind == "diag" else lam
        out = fwd(lam_lane, v, x0)
        assert rel_err(out, c.ref64_out) < tol, (kind, c.name, "out")
        glam, gv, gx0 = bwd(g, lam_lane, out, x0)
        if kind == "diag" and lam.ndim == 1:
            glam = glam.sum(0)  # autograd folds the lane gradient back onto the broadcast lam
        assert rel_err(gv, c.ref64_gv) < tol, (kind, c.name, "gv")
        assert rel_err(glam, c.ref64_glam) < tol, (kind, c.name, "glam")
        if x0 is not None:
            assert rel_err(gx0, c.ref64_gx0) < tol, (kind, c.name, "gx0")
        if not f64 and c.c32_out is not None:  # the reference's float32 CPU kernel, same arithmetic
            assert rel_err(out, c.c32_out) < 1e-5, (kind, c.name, "c32")


@pytest.mark.parametrize("f64", [True, False])
def test_mamba(oracle, f64):
    tol = TOL64 if f64 else TOL32
    for c in load_golden("mamba"):
        ins = [_cast(getattr(c, k), f64) for k in ("draw", "A", "Bt", "Ct", "u", "z", "Dp", "h0")]
        out, hlast = oracle.mamba_fwd(*ins)
        assert rel_err(out, c.ref64_out) < tol, (c.name, "out")
        assert rel_err(hlast, c.ref64_hlast) < tol, (c.name, "hlast")
        r = oracle.mamba_bwd(*ins, _cast(c.gout, f64), _cast(c.ghlast, f64))
        for k in ("gdraw", "gA", "gBt", "gCt", "gu", "gz", "gDp", "gh0"):
            ref = getattr(c, f"ref64_{k}")
            if ref is None:
                assert k == "gh0" and r[k] is None
                continue
            assert rel_err(r[k], ref) < tol, (c.name, k)
        if not f64:
            assert rel_err(out, c.c32_out) < 1e-5, (c.name, "c32")


@pytest.mark.parametrize("f64", [True, False])
def test_allpole(oracle, f64):
    tol = TOL64 if f64 else TOL32
    for c in load_golden("allpole"):
        a, w, y0, g = (_cast(t, f64) for t in (c.a, c.w, c.y0, c.g))
        y = oracle.allpole_fwd(a, w, y0)
        assert rel_err(y, c.ref64_y) < tol, (c.name, "y")
        ga, gw, gy0 = oracle.allpole_bwd(g, a, y, y0)
        assert rel_err(gw, c.ref64_gw) < tol, (c.name, "gw")
        assert rel_err(ga, c.ref64_ga) < tol, (c.name, "ga")
        if y0 is not None:
            assert rel_err(gy0, c.ref64_gy0) < tol, (c.name, "gy0")


@pytest.mark.parametrize("f64", [True, False])
def test_conv(oracle, f64):
    tol = TOL64 if f64 else TOL32
    for c in load_golden("conv"):
        x, tail, w, bias, gy = (_cast(t, f64) for t in (c.x, c.tail, c.w, c.bias, c.gy))
        out = oracle.conv_fwd(x, tail, w, bias)
        assert rel_err(out, c.ref64_out) < tol, (c.name, "out")
        gx, gtail, gw, gb = oracle.conv_bwd(gy, x, tail, w, bias)
        assert rel_err(gx, c.ref64_gx) < tol, (c.name, "gx")
        assert rel_err(gtail, c.ref64_gtail) < tol, (c.name, "gtail")
        assert rel_err(gw, c.ref64_gw) < tol, (c.name, "gw")
        if bias is not None:
            assert rel_err(gb, c.ref64_gb) < tol, (c.name, "gb")


@pytest.mark.parametrize("f64", [True, False])
def test_gblock(oracle, f64):
    """FIR numerator + all-pole denominator + pair sum against the reference's LinearDynamicalOperator."""
    tol = TOL64 if f64 else TOL32
    for c in load_golden("gblock"):
        u, b, a, tail, x0, g = (_cast(t, f64) for t in (c.u, c.b, c.a, c.tail, c.x0, c.g))
        y, yp, xl, nt = oracle.gblock_fwd(u, b, a, tail, x0)
        assert rel_err(y, c.ref64_y) < tol, (c.name, "y")
        assert rel_err(xl, c.ref64_xlast) < tol, (c.name, "xlast")
        assert rel_err(nt, c.ref64_tail) < tol, (c.name, "tail")
        gu, gb, ga, gt, gx0 = oracle.gblock_bwd(g, u, b, a, yp, tail, x0)
        for k, v in (("gu", gu), ("gb", gb), ("ga", ga)):
            assert rel_err(v, getattr(c, "ref64_" + k)) < tol, (c.name, k)
        if tail is not None:
            assert rel_err(gt, c.ref64_gtail) < tol, (c.name, "gtail")
            assert rel_err(gx0, c.ref64_gx0) < tol, (c.name, "gx0")


def test_allpole_unstable_pole_overflows_without_crash(oracle):
    """An unstable filter must run to non-finite values, not fault (reference tests/test_dynonet.py:165-174)."""
    a = np.array([[-3.0]], dtype=np.float32)
    w = np.ones((1, 400), dtype=np.float32)
    y = oracle.allpole_fwd(a, w, None)
    assert not np.isfinite(y).all()
