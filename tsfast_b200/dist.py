"""Data-parallel plumbing for the scans: one process per GPU, `torch.distributed` underneath.

The scans themselves never communicate: every (batch row x channel) sequence is independent, so
ranks simply take disjoint slices of the batch (`shard_bounds`).  The only collective in a
training step is the gradient all-reduce of the model's parameters, done here on ONE flat bucket
(a DeepLRU has well under a million parameters, so the cost is launch latency, not bandwidth).
tsfast itself has no distributed code; this is new with no counterpart there.  Works with any
backend (`nccl` on GPUs, `gloo` in the CPU tests).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

__all__ = ["shard_bounds", "allreduce_gradients", "reduce_lane_gradient", "dp_train_step", "StepGate"]


def shard_bounds(n: int, rank: int, world: int) -> tuple[int, int]:
    """[lo, hi) of the batch rows rank `rank` owns: contiguous, sizes differing by at most one."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def allreduce_gradients(params, group=None, average: bool = True) -> int:
    """Sum (or average) `.grad` of `params` over the group through one flat buffer.

    Parameters without a gradient contribute zeros so every rank reduces the same layout.
    Returns the number of elements reduced.
    """
    params = [p for p in params if p.requires_grad]
    if not params:
        return 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return sum(p.numel() for p in params)
    # one flat float32 buffer: a single concatenation in, one collective, one multi-tensor copy out (a
    # per-parameter loop of small kernels costs more than the collective itself on a fast link)
    grads = [p.grad if p.grad is not None else torch.zeros_like(p) for p in params]
    flat = torch.cat([g.reshape(-1).to(torch.float32) for g in grads])
    nccl = dist.get_backend(group) == "nccl"
    dist.all_reduce(flat, op=dist.ReduceOp.AVG if (average and nccl) else dist.ReduceOp.SUM, group=group)
    if average and not nccl:
        flat /= world
    pieces = [piece.view_as(p) for piece, p in zip(flat.split([p.numel() for p in params]), params)]
    have = [(p.grad, piece) for p, piece in zip(params, pieces) if p.grad is not None]
    if have:
        torch._foreach_copy_([g for g, _ in have], [piece for _, piece in have])
    for p, piece in zip(params, pieces):
        if p.grad is None:
            p.grad = piece.to(p.dtype).clone()
    return flat.numel()


def reduce_lane_gradient(grad: torch.Tensor, group=None) -> torch.Tensor:
    """Sum over ranks of a gradient whose parameter is shared by all batch rows (lam of S1, a of
    S4, A and Dp of S3): each rank's autograd only folds its own rows, this adds the shards."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=group)
    return grad


def dp_train_step(model, optimizer, loss_fn, xb, yb, group=None):
    """One data-parallel step on this rank's shard: forward, loss, backward, gradient average, update.

    Returns the detached local loss.  Every rank must call it the same number of times.
    """
    optimizer.zero_grad(set_to_none=True)
    out = model(xb)
    if isinstance(out, tuple):
        out = out[0]
    loss = loss_fn(out, yb)
    loss.backward()
    allreduce_gradients(model.parameters(), group=group, average=True)
    optimizer.step()
    return loss.detach()


class StepGate:
    """Host-side failure detection between steps: ranks check in before every step.

    Each rank writes ``step/<k>/<rank>`` into a key-value store (a ``torch.distributed.TCPStore``
    or anything with ``set``/``wait``) before step ``k`` and waits a bounded time for everyone
    else's key.  A rank that died, hung on the host or left shows up as a ``RuntimeError`` naming
    it BEFORE the survivors launch kernels or enter a collective, so no GPU work is ever left
    waiting on a peer that will not come.
    """

    def __init__(self, store, rank: int, world: int, timeout_s: float = 10.0):
        self.store, self.rank, self.world, self.timeout_s = store, rank, world, timeout_s

    def check_in(self, step: int) -> None:
        import datetime

        self.store.set(f"step/{step}/{self.rank}", "1")
        missing = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                self.store.wait([f"step/{step}/{r}"], datetime.timedelta(seconds=self.timeout_s))
            except Exception:  # the store raises on timeout (the exception type varies across builds)
                missing.append(r)
        if missing:
            raise RuntimeError(f"rank(s) {missing} did not check in for step {step} within {self.timeout_s} s")
