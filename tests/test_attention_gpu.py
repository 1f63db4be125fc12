"""Fused GATv2 and graph-transformer attention on the GPU against the CPU oracle (fp64 ground truth).

Bars: max relative error (relative to the largest reference magnitude of the tensor) <= 1e-5 in
fp32 and <= 2e-2 in bf16/fp16, for outputs and every gradient.
"""

import pytest
import torch

import turbo_gnn_b200 as tg
from helpers import make_graph, random_edges, rel_err
from oracle import scatter_oracle as O
from turbo_gnn_b200 import _C
from turbo_gnn_b200._functions import _FusedGraphAttention, gatv2_function

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-2}
N = 1200


def _graph(idt=torch.int32, q=0.9, seed=1, symmetric=False, n=N):
    ei = random_edges(n, 8 * n, seed, hubs=3, hub_degree=n // 2, self_loops=symmetric, symmetric=symmetric)
    return ei, make_graph(ei, n, idt, quantile=q)


def _rand(shape, seed, dt=torch.float32, std=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * std).to(dt)


def _gatv2_case(ei, g, h, d, dt, n=N, **kw):
    l, r, up = _rand((n, h, d), 10, dt), _rand((n, h, d), 11, dt), _rand((n, h, d), 12, dt)
    a = _rand((h, d), 13, dt, 0.1)
    ref = [t.double().requires_grad_() for t in (l, r, a)]
    want = O.gatv2_aggregate(*ref, ei, n, 0.2)
    want.backward(up.double())
    dev = [t.cuda().requires_grad_() for t in (l, r, a)]
    got = tg.gatv2_aggr(g, *dev, 0.2, **kw)
    got.backward(up.cuda())
    assert got.shape == (n, h, d) and got.dtype == dt
    errs = {"out": rel_err(got.float(), want)}
    for name, dv, rf in zip(("grad_x", "grad_x_neighbors", "grad_attention"), dev, ref):
        assert dv.grad.shape == rf.grad.shape and dv.grad.dtype == dt
        errs[name] = rel_err(dv.grad.float(), rf.grad)
    return errs


def _gt_case(ei, g, h, d, dt, n=N, scale=None, **kw):
    q, k, v, up = (_rand((n, h, d), 20 + i, dt) for i in range(4))
    ref = [t.double().requires_grad_() for t in (q, k, v)]
    want = O.gt_aggregate(*ref, ei, n, scale if scale is not None else d**-0.5)
    want.backward(up.double())
    dev = [t.cuda().requires_grad_() for t in (q, k, v)]
    got = tg.graph_transformer_aggr(g, None, *dev, scale, **kw)
    got.backward(up.cuda())
    assert got.shape == (n, h, d) and got.dtype == dt
    errs = {"out": rel_err(got.float(), want)}
    for name, dv, rf in zip(("dQ", "dK", "dV"), dev, ref):
        errs[name] = rel_err(dv.grad.float(), rf.grad)
    return errs


SHAPES = [(8, 64), (4, 32), (1, 16), (2, 128), (2, 256), (1, 47), (4, 64), (3, 20)]


@pytest.mark.parametrize("idt", [torch.int32, torch.int64])
@pytest.mark.parametrize("h,d", SHAPES)
def test_gatv2_fp32(idt, h, d):
    ei, g = _graph(idt)
    with _C.hub_tier(chunk_edges=128, hub_min_degree=400):
        errs = _gatv2_case(ei, g, h, d, torch.float32)
    assert max(errs.values()) <= TOL[torch.float32], errs


@pytest.mark.parametrize("idt", [torch.int32, torch.int64])
@pytest.mark.parametrize("h,d", SHAPES)
def test_graph_transformer_fp32(idt, h, d):
    ei, g = _graph(idt)
    with _C.hub_tier(chunk_edges=128, hub_min_degree=400):
        errs = _gt_case(ei, g, h, d, torch.float32, scale=0.125)
    assert max(errs.values()) <= TOL[torch.float32], errs


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("h,d", [(4, 64), (8, 32), (1, 256), (2, 40)])
def test_low_precision(dt, h, d):
    ei, g = _graph()
    with _C.hub_tier(chunk_edges=128, hub_min_degree=400):
        e1 = _gatv2_case(ei, g, h, d, dt)
        e2 = _gt_case(ei, g, h, d, dt)
    assert max(e1.values()) <= TOL[dt], e1
    assert max(e2.values()) <= TOL[dt], e2


def test_default_scale_is_inverse_sqrt_head_dim():
    ei, g = _graph()
    errs = _gt_case(ei, g, 2, 64, torch.float32, scale=None)
    assert max(errs.values()) <= TOL[torch.float32], errs


@pytest.mark.parametrize("lw,hw", [(1, 8), (2, 16), (4, 32)])
def test_warp_counts_do_not_change_results(lw, hw):
    ei, g = _graph()
    kw = dict(forward_light_warps=lw, forward_heavy_warps=hw, backward_light_warps=lw, backward_heavy_warps=hw)
    assert max(_gatv2_case(ei, g, 4, 64, torch.float32, **kw).values()) <= TOL[torch.float32]
    assert max(_gt_case(ei, g, 4, 64, torch.float32, **kw).values()) <= TOL[torch.float32]


@pytest.mark.parametrize("q", [-1, 0.5, 0.99])
def test_bucketing_does_not_change_results(q):
    ei, g = _graph()
    gq = g.repartition(forward_huge_degree_threshold_quantile=q, backward_huge_degree_threshold_quantile=q)
    for hub_min in (100, 100000):
        with _C.hub_tier(chunk_edges=64, hub_min_degree=hub_min):
            assert max(_gatv2_case(ei, gq, 2, 64, torch.float32).values()) <= TOL[torch.float32]
            assert max(_gt_case(ei, gq, 2, 64, torch.float32).values()) <= TOL[torch.float32]


def test_undirected_graph_with_aliased_backward_csr():
    ei, g = _graph(symmetric=True)
    assert g.is_directed is False and g.backward_indices is g.forward_indices
    assert max(_gatv2_case(ei, g, 4, 32, torch.float32).values()) <= TOL[torch.float32]
    assert max(_gt_case(ei, g, 4, 32, torch.float32).values()) <= TOL[torch.float32]


def test_empty_rows_give_zero_output_and_minus_inf_lse():
    n = 6
    ei = torch.tensor([[1, 2, 3, 1], [0, 0, 0, 4]])
    g = make_graph(ei, n, torch.int32, quantile=-1)
    l, r = _rand((n, 2, 32), 1).cuda(), _rand((n, 2, 32), 2).cuda()
    a = _rand((2, 32), 3, std=0.1).cuda()
    out, lse = _C.gatv2_forward(l, r, g.forward_indptr, g.forward_indices, a, 0.2, g.light_nodes, g.heavy_nodes, 1, 8)
    empty = torch.tensor([1, 2, 3, 5])
    assert out[empty].eq(0).all() and torch.isinf(lse[empty]).all() and (lse[empty] < 0).all()
    assert torch.isfinite(lse[[0, 4]]).all()
    # a row with one in-edge copies the source row
    assert torch.allclose(out[4], r[1], atol=1e-6)
    out, lse = _C.gt_forward_csr_mh(g.forward_indptr, g.forward_indices, l, r, r, 0.125, g.light_nodes, g.heavy_nodes)
    assert out[empty].eq(0).all() and torch.isinf(lse[empty]).all()
    # gradients of source rows nobody reads are zero, not garbage
    lq = l.clone().requires_grad_()
    tg.graph_transformer_aggr(g, None, lq, r, r, 0.125).sum().backward()
    assert lq.grad[[0, 4, 5]].eq(0).all()


def test_logsumexp_matches_oracle():
    ei, g = _graph()
    h, d = 4, 32
    q, k, v = (_rand((N, h, d), 30 + i) for i in range(3))
    _, lse = _C.gt_forward_csr_mh(g.forward_indptr, g.forward_indices, q.cuda(), k.cuda(), v.cuda(), 0.25,
                                  g.light_nodes, g.heavy_nodes)
    score = (q.double()[ei[0]] * k.double()[ei[1]]).sum(-1) * 0.25
    want = O.attention_lse(score, ei[1], N)
    finite = ~want.isinf()
    assert torch.equal(lse.cpu().isinf(), want.isinf())
    assert (lse.cpu().double()[finite] - want[finite]).abs().max() <= 1e-5


def test_positional_apply_matches_reference_argument_order():
    ei, g = _graph()
    h, d = 2, 64
    q, k, v = (_rand((N, h, d), 40 + i).cuda() for i in range(3))
    a = _rand((h, d), 44, std=0.1).cuda()
    out = gatv2_function.apply(g.forward_indptr, g.forward_indices, g.backward_indptr, g.backward_indices, q, k, a, 0.2,
                               512, g.forward_light_nodes, g.forward_heavy_nodes, g.backward_light_nodes,
                               g.backward_heavy_nodes, 1, 8, 1, 8, g.is_directed)
    assert torch.equal(out, tg.gatv2_aggr(g, q, k, a, 0.2))
    out = _FusedGraphAttention.apply(g.forward_indptr, g.forward_indices, g.backward_indptr, g.backward_indices, q, k,
                                     v, 0.125, g.forward_light_nodes, g.forward_heavy_nodes, g.backward_light_nodes,
                                     g.backward_heavy_nodes, 4, 8, 1, 8, g.is_directed)
    assert torch.equal(out, tg.graph_transformer_aggr(g, None, q, k, v, 0.125))


def test_strided_inputs_from_a_fused_projection():
    # l and r are the two halves of one [N, 2*H*D] projection, as the reference's layer produces them
    ei, g = _graph()
    h, d = 4, 32
    both = _rand((N, 2 * h * d), 50)
    l, r = both[:, : h * d].reshape(N, h, d), both[:, h * d:].reshape(N, h, d)
    a = _rand((h, d), 51, std=0.1)
    dev = both.cuda()
    lv, rv = dev[:, : h * d].view(N, h, d), dev[:, h * d:].view(N, h, d)
    assert not lv.is_contiguous()
    got = tg.gatv2_aggr(g, lv, rv, a.cuda(), 0.2)
    want = O.gatv2_aggregate(l.double(), r.double(), a.double(), ei, N, 0.2)
    assert rel_err(got, want) <= TOL[torch.float32]


def test_invalid_launch_parameters_and_shapes_raise():
    ei, g = _graph(n=300)
    q = _rand((300, 2, 32), 1).cuda()
    a = _rand((2, 32), 2).cuda()
    with pytest.raises(RuntimeError):
        tg.gatv2_aggr(g, q, q, a, 0.2, forward_light_warps=3)
    with pytest.raises(RuntimeError):
        tg.gatv2_aggr(g, q, q, a, 0.2, forward_heavy_warps=4)
    with pytest.raises(RuntimeError):
        tg.graph_transformer_aggr(g, None, q, q, q.half(), 0.1)
    with pytest.raises(RuntimeError):
        tg.gatv2_aggr(g, q, q, a[:, :16], 0.2)
    big = _rand((300, 1, 512), 3).cuda()
    with pytest.raises(RuntimeError):
        tg.graph_transformer_aggr(g, None, big, big, big, 0.1)
    out = tg.gatv2_aggr(g, q.clone().requires_grad_(), q, a, 0.2, grad_A_reduce_row_chunk_size=16)
    with pytest.raises(RuntimeError):
        out.sum().backward()


def test_runs_twice_with_identical_forward_results():
    ei, g = _graph()
    q, k, v = (_rand((N, 4, 64), 60 + i).cuda() for i in range(3))
    a = tg.graph_transformer_aggr(g, None, q, k, v, 0.125)
    b = tg.graph_transformer_aggr(g, None, q, k, v, 0.125)
    assert torch.equal(a, b)  # no atomics in the forward path: bitwise repeatable
