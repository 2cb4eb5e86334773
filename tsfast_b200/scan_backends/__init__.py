"""Kernel backends for the diagonal scans, one module per op, speaking the reference's
backend-module protocol (``tsfast/models/_core/scan_backends/__init__.py:10-17``):
``supports(lam, v, x0) -> str | None`` plus raw ``forward`` / ``backward`` entry points on the
flattened, contiguous lane layout.
"""
