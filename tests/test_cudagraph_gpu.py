"""CUDA-graph capture of the scan ops, forward and backward (the constraint tsfast's
GraphedStatefulModel puts on a backend, tsfast/models/_core/cudagraph.py:87-121): no host sync, no
cudaMalloc, all work on the current stream, look-back flags reset by an in-stream memset.  A graph
replayed on new input values must give what eager execution gives."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_graph_capture_of_raw_entry_points_replays_on_new_data():
    from tsfast_b200.scan_backends import diagonal_b200, selective_b200

    torch.manual_seed(0)
    # few chains -> look-back kernel (workspace, flags, memset); many chains -> streaming kernel
    for (M, L, N) in ((2, 700, 64), (64, 300, 256)):
        a = torch.rand(M, L, N, device="cuda") * 0.9
        b = torch.randn(M, L, N, device="cuda")
        g = torch.randn(M, L, N, device="cuda")
        lam = torch.rand(M, N, device="cuda") * 0.9
        for _ in range(2):  # first calls set kernel attributes; keep them out of the capture
            h = selective_b200.forward(a, b, None)
            selective_b200.backward(g, a, h, None)
            diagonal_b200.backward(g, lam, diagonal_b200.forward(lam, b, None), None)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            h = selective_b200.forward(a, b, None)
            ga, gb, _ = selective_b200.backward(g, a, h, None)
            x = diagonal_b200.forward(lam, b, None)
            gl, gv, _ = diagonal_b200.backward(g, lam, x, None)
        for trial in range(2):
            a.copy_(torch.rand_like(a) * 0.9)
            b.normal_()
            g.normal_()
            graph.replay()
            torch.cuda.synchronize()
            he = selective_b200.forward(a, b, None)
            gae, gbe, _ = selective_b200.backward(g, a, he, None)
            xe = diagonal_b200.forward(lam, b, None)
            gle, gve, _ = diagonal_b200.backward(g, lam, xe, None)
            for got, want in ((h, he), (ga, gae), (gb, gbe), (x, xe), (gl, gle), (gv, gve)):
                assert torch.equal(got, want), (M, L, N, trial)


def test_make_graphed_callables_on_the_lru_stack():
    """Forward AND backward of a DeepLRU captured by torch.cuda.make_graphed_callables (what
    GraphedStatefulModel uses) match the eager module."""
    from mirrors import DeepLRU

    torch.manual_seed(1)
    eager = DeepLRU(2, 3, d_model=16, d_state=32, n_layers=2, r_min=0.5, r_max=0.95, max_phase=1.0).cuda()
    graphed_src = DeepLRU(2, 3, d_model=16, d_state=32, n_layers=2).cuda()
    graphed_src.load_state_dict(eager.state_dict())
    sample = torch.randn(4, 257, 2, device="cuda", requires_grad=True)
    graphed = torch.cuda.make_graphed_callables(graphed_src, (sample,))
    for trial in range(2):
        u = torch.randn(4, 257, 2, device="cuda")
        gy = torch.randn(4, 257, 3, device="cuda")
        ue, ug = u.clone().requires_grad_(), u.clone().requires_grad_()
        ye = eager(ue)
        ye.backward(gy)
        yg = graphed(ug)
        yg.backward(gy)
        torch.cuda.synchronize()
        assert torch.allclose(yg, ye, rtol=1e-5, atol=1e-6)
        assert torch.allclose(ug.grad, ue.grad, rtol=1e-4, atol=1e-6)
        for (k, pe), pg in zip(eager.named_parameters(), graphed_src.parameters()):
            assert torch.allclose(pg.grad, pe.grad, rtol=1e-3, atol=1e-5), (k, trial)
        eager.zero_grad(set_to_none=True)
        graphed_src.zero_grad(set_to_none=True)


def test_graph_capture_of_mamba_and_allpole():
    from tsfast_b200 import allpole_b200, mamba_b200

    torch.manual_seed(2)
    B, L, D, N = 2, 70, 40, 16
    r = lambda *s: torch.randn(*s, device="cuda")  # noqa: E731
    ins = [r(B, L, D) * 0.5 - 1, -torch.exp(r(D, N) * 0.3), r(B, L, N), r(B, L, N), r(B, L, D), r(B, L, D), r(D), r(B, D, N)]
    gout = r(B, L, D)
    a, w, y0, g = r(6, 3) * 0.2, r(6, 600), r(6, 3), r(6, 600)

    def run():
        out, hl, chk = mamba_b200._scan_train_op(*ins)
        grads = mamba_b200._scan_bwd_op(gout, None, chk, *ins)
        y = allpole_b200._allpole_op(a, w, y0)
        ag = allpole_b200._allpole_bwd_op(g, a, y, y0)
        return (out, hl, *grads, y, *ag)

    run(), run()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = run()
    ins[4].normal_(), w.normal_(), gout.normal_()
    graph.replay()
    torch.cuda.synchronize()
    for got, want in zip(captured, run()):
        assert torch.equal(got, want)


def test_graph_capture_of_conv_and_dynonet_block():
    from tsfast_b200 import conv_b200, dynonet_b200

    torch.manual_seed(3)
    r = lambda *s: torch.randn(*s, device="cuda")  # noqa: E731
    x, tail, w, bias, gy = r(2, 90, 48), r(2, 48, 3), r(48, 4) * 0.5, r(48), r(2, 90, 48)
    u, b, a = r(2, 1300, 2), r(3, 2, 8) * 0.3, r(3, 2, 2) * 0.2
    st_u, st_x, gyb = r(2, 7, 2), r(2, 6, 2), r(2, 3, 1300)

    def run():
        y = conv_b200._conv_silu_op(x, tail, w, bias)
        cg = conv_b200._conv_silu_bwd_op(gy, x, tail, w, bias)
        yb, yp, xl, ub, taps = dynonet_b200._gblock_op(u, st_u, b, a, st_x, True)
        bg = dynonet_b200._gblock_bwd_op(gyb, ub, taps, a, st_x, yp, u.shape[1], b.shape[-1])
        return (y, *cg, yb, yp, xl, *bg)

    run(), run()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = run()
    x.normal_(), u.normal_(), gyb.normal_()
    graph.replay()
    torch.cuda.synchronize()
    for got, want in zip(captured, run()):
        assert torch.equal(got, want)
