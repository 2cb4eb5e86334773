"""Launch path shared by the S1 (constant coefficient) and S2 (per-step coefficient) backends.

Both scans run the same two CUDA kernels; they differ in the coefficient's shape and in the entry
points' names (``b200_diag_*`` / ``b200_sel_*``).  ``Scan`` binds one of the two and offers the
three calls tsfast's backend protocol asks for.
"""

from __future__ import annotations

import torch

from .. import _lib, _spec, status

_DTYPES = (torch.float32, torch.complex64)


class Scan:
    """One of the two diagonal scans on the lane layout ``[rows, L, n]``."""

    def __init__(self, entry: str, per_step: bool):
        self.entry = entry
        coef = ("R", "L", "N") if per_step else ("R", "N")
        self.contract = _spec.Contract(
            op=f"scan_{'selective' if per_step else 'diagonal'}",
            tensors=(_spec.Tensor("v", ("R", "L", "N")), _spec.Tensor("lam", coef),
                     _spec.Tensor("x0", ("R", "N"), optional=True)),
            dtypes=_DTYPES)

    def why_not(self, lam, v, x0) -> str | None:
        return _spec.explain(self.contract, v=v, lam=lam, x0=x0)

    def _call(self, which: str, backward: bool, shape, dtype, device, *pointers):
        L_ = _lib.lib()
        rows, steps, n = shape
        tag = _lib.dtype_tag(dtype)
        ws = _lib.workspace(getattr(L_, f"b200_{self.entry}_workspace_bytes")(tag, int(backward), rows, steps, n), device)
        rc = getattr(L_, f"b200_{self.entry}_{which}")(tag, rows, steps, n, *pointers, _lib.ptr(ws), ws.numel(),
                                                        _lib.stream_ptr(device))
        _lib.check(rc, f"b200_{self.entry}_{which}")
        status.remember(ws)

    def forward(self, lam, v, x0):
        _lib.require_dense_cuda(lam=lam, v=v, x0=x0)
        out = torch.empty_like(v)
        if out.numel():
            self._call("fwd", False, v.shape, v.dtype, v.device, _lib.ptr(lam), _lib.ptr(v), _lib.ptr(x0), _lib.ptr(out))
        return out

    def backward(self, g, lam, out, x0):
        _lib.require_dense_cuda(g=g, lam=lam, out=out, x0=x0)
        glam, gv = torch.empty_like(lam), torch.empty_like(out)
        gx0 = None if x0 is None else torch.empty_like(x0)
        if out.numel():
            self._call("bwd", True, out.shape, out.dtype, out.device, _lib.ptr(g), _lib.ptr(lam), _lib.ptr(out),
                       _lib.ptr(x0), _lib.ptr(glam), _lib.ptr(gv), _lib.ptr(gx0))
        else:  # nothing to scan: the sums over time are empty
            glam.zero_()
            if gx0 is not None:
                gx0.zero_()
        return glam, gv, (lam.new_empty(0) if gx0 is None else gx0)


DIAGONAL = Scan("diag", per_step=False)
SELECTIVE = Scan("sel", per_step=True)
