"""One table-driven checker behind every backend module's ``supports()`` and every op's guard.

A backend states its contract as data: the tensors it takes, their shapes written with named
extents (``"B"``, ``"L"`` ... are bound by the first tensor that mentions them and must agree
afterwards), the dtypes it computes in and the range each extent may take.  ``explain`` walks
that table and returns the first violated rule as a sentence, or ``None``.  The sentence is what
tsfast's dispatcher shows once in its fallback warning and what the ops of this package raise.

``lanes`` is the one place where broadcasting is written: it spreads per-channel coefficients
over the leading dims of a sequence tensor and flattens both onto the kernels' lane layout.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

__all__ = ["Tensor", "Contract", "explain", "demand", "lanes", "dense"]


@dataclass(frozen=True)
class Tensor:
    """One argument of a contract: ``dims`` lists extents as names or fixed integers."""

    name: str
    dims: tuple
    optional: bool = False
    spread: bool = False  # leading dims (all but the last) need only broadcast into those of ``over``
    over: str | None = None


@dataclass(frozen=True)
class Contract:
    op: str
    tensors: tuple
    dtypes: tuple
    ranges: dict = field(default_factory=dict)  # extent name -> (low, high), inclusive
    same_dtype: bool = True


def _fmt(shape) -> str:
    return "[" + ", ".join(str(s) for s in shape) + "]"


def explain(contract: Contract, **given) -> str | None:
    """First rule of ``contract`` that ``given`` breaks, as text; ``None`` when all hold."""
    if not torch.cuda.is_available():
        return "no CUDA device is visible to this process"
    bound: dict[str, int] = {}
    shapes: dict[str, tuple] = {}
    first_dtype = None
    for spec in contract.tensors:
        t = given.get(spec.name)
        if t is None:
            if spec.optional:
                continue
            return f"{spec.name} is required"
        if t.device.type != "cuda":
            return f"{spec.name} lives on {t.device}, the kernels only read CUDA memory"
        if t.dtype not in contract.dtypes:
            want = " or ".join(str(d).replace("torch.", "") for d in contract.dtypes)
            return f"{spec.name} is {str(t.dtype).replace('torch.', '')}, the kernel computes in {want}"
        if contract.same_dtype:
            if first_dtype is None:
                first_dtype = t.dtype
            elif t.dtype != first_dtype:
                return f"{spec.name} is {t.dtype} while the other tensors are {first_dtype}"
        shape = tuple(t.shape)
        shapes[spec.name] = shape
        if spec.spread:
            if len(shape) < 1:
                return f"{spec.name} needs at least one axis"
            last = spec.dims[-1]
            if isinstance(last, str):
                if bound.setdefault(last, shape[-1]) != shape[-1]:
                    return f"{spec.name} has {shape[-1]} entries on its last axis, expected {last}={bound[last]}"
            elif shape[-1] != last:
                return f"{spec.name} has {shape[-1]} entries on its last axis, expected {last}"
            lead = shapes[spec.over][:-1]
            try:
                ok = tuple(torch.broadcast_shapes(shape[:-1], lead)) == tuple(lead)
            except RuntimeError:
                ok = False
            if not ok:
                return f"leading dims {_fmt(shape[:-1])} of {spec.name} cannot be spread over {_fmt(lead)} of {spec.over}"
            continue
        if spec.dims and spec.dims[0] is Ellipsis:
            tail = spec.dims[1:]
            if len(shape) < len(tail):
                return f"{spec.name} has {len(shape)} axes, at least {len(tail)} are needed"
            pairs = zip(tail, shape[len(shape) - len(tail):])
        else:
            if len(shape) != len(spec.dims):
                return f"{spec.name} is {_fmt(shape)}, expected {len(spec.dims)} axes {_fmt(spec.dims)}"
            pairs = zip(spec.dims, shape)
        for want, have in pairs:
            if isinstance(want, str):
                if bound.setdefault(want, have) != have:
                    expected = tuple(bound.get(d, d) if isinstance(d, str) else d for d in spec.dims if d is not Ellipsis)
                    return f"{spec.name} is {_fmt(shape)}, expected {_fmt(expected)}"
            elif want != have:
                return f"{spec.name} is {_fmt(shape)}, expected {_fmt(spec.dims)}"
    for extent, (lo, hi) in contract.ranges.items():
        if extent in bound and not lo <= bound[extent] <= hi:
            return f"{extent}={bound[extent]} is outside what {contract.op} handles ({lo}..{hi})"
    return None


def demand(contract: Contract, **given) -> None:
    """Raise ``RuntimeError`` naming the op when ``explain`` finds a broken rule."""
    why = explain(contract, **given)
    if why is not None:
        raise RuntimeError(f"b200scan::{contract.op}: {why}")


def dense(*tensors):
    """Contiguous versions of the tensors that are present (``None`` stays ``None``)."""
    return tuple(None if t is None else t.contiguous() for t in tensors)


def lanes(seq: torch.Tensor, seq_tail: int, *per_lane):
    """Flatten ``seq [..., tail]`` (``seq_tail`` trailing axes kept) to ``[lanes, tail]`` and spread
    every ``per_lane`` tensor ``[..., k]`` (or ``None``) over the same leading dims as ``[lanes, k]``.

    The expansion happens here, outside the custom ops, so that autograd sums lane gradients back
    onto whatever shape the caller's coefficients had.
    """
    lead = tuple(seq.shape[: seq.dim() - seq_tail])
    flat = seq.reshape((-1,) + tuple(seq.shape[seq.dim() - seq_tail:]))
    out = [flat]
    for t in per_lane:
        out.append(None if t is None else t.expand(lead + (t.shape[-1],)).reshape(-1, t.shape[-1]))
    return out
