"""Host-side logic of the data-parallel path on CPU: two `gloo` ranks.

The scans have no collective, so what is tested is the sharding arithmetic, the flat-bucket
gradient all-reduce (two ranks on half batches reproduce the single-process full-batch gradient
and parameter update), the shared-parameter gradient sum, and that a rank which leaves between steps
is reported to its peer on the host (a store check-in with a short timeout) before the next step."""

import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

from tsfast_b200.dist import StepGate, allreduce_gradients, dp_train_step, reduce_lane_gradient, shard_bounds


def test_shard_bounds_cover_batch_exactly():
    for n in (0, 1, 7, 16, 64, 1024, 1025):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_bounds(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(5, 7), nn.Tanh(), nn.Linear(7, 2))


def _data():
    g = torch.Generator().manual_seed(1)
    return torch.randn(12, 9, 5, generator=g), torch.randn(12, 9, 2, generator=g)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    try:
        x, y = _data()
        lo, hi = shard_bounds(x.shape[0], rank, world)
        model = _model()
        opt = torch.optim.SGD(model.parameters(), lr=0.1)
        loss = dp_train_step(model, opt, nn.functional.mse_loss, x[lo:hi], y[lo:hi])
        lane = reduce_lane_gradient(torch.full((3,), float(rank + 1)))
        n = allreduce_gradients([torch.nn.Parameter(torch.ones(2))])  # a parameter nobody has a grad for
        q.put((rank, [p.detach().numpy().copy() for p in model.parameters()], float(loss), lane.numpy().copy(), n))
    finally:
        dist.destroy_process_group()


def test_two_rank_step_matches_single_process_full_batch():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted((q.get(timeout=120) for _ in range(world)), key=lambda t: t[0])
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    x, y = _data()
    ref = _model()
    opt = torch.optim.SGD(ref.parameters(), lr=0.1)
    dp_train_step(ref, opt, nn.functional.mse_loss, x, y)  # world size 1: plain step on the full batch
    for rank, params, loss, lane, n in results:
        for p, r in zip(params, ref.parameters()):
            torch.testing.assert_close(torch.from_numpy(p), r.detach(), rtol=1e-6, atol=1e-7)
        assert (lane == 3.0).all() and n == 2
    for a, b in zip(results[0][1], results[1][1]):
        assert (a == b).all()  # replicas stay bitwise in sync


def _gate_worker(rank, world, port, q):
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    gate = StepGate(store, rank, world, timeout_s=2.0)
    gate.check_in(0)  # both alive
    if rank == 1:
        q.put((rank, "left after step 0"))
        return  # leaves between steps, nothing in flight
    try:
        gate.check_in(1)
        q.put((rank, "no error"))
    except RuntimeError as e:
        q.put((rank, f"error: {e}"))


def test_peer_that_leaves_is_reported_before_the_next_step():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gate_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(60)
    assert got[1] == "left after step 0"
    assert got[0].startswith("error: rank(s) [1] did not check in for step 1"), got
