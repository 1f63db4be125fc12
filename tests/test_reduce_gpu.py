"""Segment reductions on the GPU (through the public API -> C ABI) against the CPU oracle.

Bars: min/max values and winners bit-exact; sum/mean max relative error <= 1e-5 in fp32 and
<= 2e-2 in 16-bit types (fp32 accumulation), relative to the largest reference magnitude.
"""

import pytest
import torch

import turbo_gnn_b200 as tg
from helpers import make_graph, random_edges, rel_err
from oracle import scatter_oracle as O
from turbo_gnn_b200 import _C

pytestmark = pytest.mark.gpu

FP32_TOL, LOWP_TOL = 1e-5, 2e-2


def _graph(n=1500, e=15000, seed=1, idt=torch.int32, q=0.9, hubs=3, hub_degree=1200):
    ei = random_edges(n, e, seed, hubs=hubs, hub_degree=hub_degree)
    return ei, make_graph(ei, n, idt, quantile=q)


@pytest.mark.parametrize("idt", [torch.int32, torch.int64])
@pytest.mark.parametrize("dt,feat", [(torch.float32, 128), (torch.float32, 16), (torch.float32, 100),
                                     (torch.float32, 1300), (torch.bfloat16, 256), (torch.float16, 40)])
def test_all_tiers_match_oracle(idt, dt, feat):
    n = 1500
    ei, g = _graph(idt=idt)
    x = torch.randn(n, feat, generator=torch.Generator().manual_seed(2)).to(dt)
    with _C.hub_tier(chunk_edges=256, hub_min_degree=800):  # forces light + heavy + hub rows
        for red in ("min", "max", "sum", "mean"):
            got = tg.reduction_aggr(g, x.cuda(), warps_per_block=4, reduce=red).cpu()
            want = O.segment_reduce(x.float(), ei, n, red)
            if red in ("min", "max"):
                assert torch.equal(got.float(), want), red
            else:
                assert rel_err(got.float(), want) <= (FP32_TOL if dt == torch.float32 else LOWP_TOL), red


@pytest.mark.parametrize("red", ["min", "max"])
@pytest.mark.parametrize("idt", [torch.int32, torch.int64])
def test_winner_indices_and_backward(red, idt):
    n = 600
    ei, g = _graph(n=n, e=5000, idt=idt, hub_degree=500)
    # few distinct values -> many ties: the winner must be the lowest source id
    x = torch.randint(0, 4, (n, 32), generator=torch.Generator().manual_seed(3)).float()
    with _C.hub_tier(chunk_edges=64, hub_min_degree=300):
        out, arg = _C.reduction_aggr_forward_partitioned(
            g.forward_indptr, g.forward_indices, x.cuda(), g.light_nodes, g.heavy_nodes, g.max_degree, 4, 128,
            False, 32, 8, red)
    assert arg.dtype == idt
    assert torch.equal(arg.cpu().long(), O.segment_argreduce(x, ei, n, red))
    assert torch.equal(out.cpu(), O.segment_reduce(x, ei, n, red))
    # backward: all of grad_out[v, f] goes to the winner row
    xg = torch.randn(n, 32, generator=torch.Generator().manual_seed(4))
    xc = xg.cuda().requires_grad_()
    up = torch.randn(n, 32, generator=torch.Generator().manual_seed(5))
    tg.reduction_aggr(g, xc, warps_per_block=1, reduce=red).backward(up.cuda())
    xr = xg.clone().requires_grad_()
    O.segment_reduce(xr, ei, n, red).backward(up)  # no ties for N(0,1) data: autograd agrees
    assert rel_err(xc.grad, xr.grad) <= FP32_TOL


def test_sum_and_mean_backward():
    n = 800
    ei, g = _graph(n=n, e=6000, hub_degree=600)
    x = torch.randn(n, 64, generator=torch.Generator().manual_seed(6))
    up = torch.randn(n, 64, generator=torch.Generator().manual_seed(7))
    for red in ("sum", "mean"):
        xc, xr = x.cuda().requires_grad_(), x.double().requires_grad_()
        tg.reduction_aggr(g, xc, warps_per_block=2, reduce=red).backward(up.cuda())
        O.segment_reduce(xr, ei, n, red).backward(up.double())
        assert rel_err(xc.grad, xr.grad) <= FP32_TOL, red


def test_empty_rows_isolated_nodes_and_tiny_graphs():
    # star: only node 0 has in-edges
    n = 10
    ei = torch.stack([torch.arange(1, n), torch.zeros(n - 1, dtype=torch.long)])
    g = make_graph(ei, n, torch.int32, quantile=0.99)
    x = torch.arange(n, dtype=torch.float32).unsqueeze(1).repeat(1, 16)
    out, arg = _C.reduction_aggr_forward_partitioned(g.forward_indptr, g.forward_indices, x.cuda(), g.light_nodes,
                                                     g.heavy_nodes, g.max_degree, 1, 128, False, 32, 8, "min")
    assert out[0].eq(1).all() and out[1:].eq(0).all()
    assert arg[0].eq(1).all() and arg[1:].eq(-1).all()
    assert tg.reduction_aggr(g, x.cuda(), warps_per_block=1, reduce="max")[0].eq(n - 1).all()
    # all nodes in the light bucket (quantile -1) and an empty heavy bucket
    g2 = g.repartition(forward_huge_degree_threshold_quantile=-1)
    assert g2.heavy_nodes.numel() == 0
    assert torch.equal(tg.reduction_aggr(g2, x.cuda(), warps_per_block=1, reduce="min"), out)
    # a graph without any edge
    g3 = tg.AdjacencyForwardBackwardWithNodeBuckets.from_edge_list(torch.zeros(2, 0, dtype=torch.long), 5,
                                                                   index_dtype=torch.int32).to("cuda")
    assert tg.reduction_aggr(g3, torch.randn(5, 8).cuda(), warps_per_block=1, reduce="sum").eq(0).all()


def test_special_values():
    # +-inf never win, NaN never wins, -0.0 / +0.0 tie goes to the lowest source id
    ei = torch.tensor([[1, 2, 3, 4, 5], [0, 0, 0, 6, 6]])
    x = torch.zeros(7, 4)
    x[1], x[2], x[3] = float("inf"), float("nan"), 2.0
    x[4], x[5] = 0.0, -0.0
    g = make_graph(ei, 7, torch.int32, quantile=-1)
    out, arg = _C.reduction_aggr_forward_partitioned(g.forward_indptr, g.forward_indices, x.cuda(), g.light_nodes,
                                                     g.heavy_nodes, g.max_degree, 1, 128, False, 32, 8, "min")
    assert out[0].eq(2).all() and arg[0].eq(3).all()
    assert arg[6].eq(4).all() and not torch.signbit(out[6]).any()


def test_invariance_to_bucketing_and_launch_parameters():
    n = 1200
    ei, g = _graph(n=n, e=9000, hub_degree=900)
    x = torch.randn(n, 128, generator=torch.Generator().manual_seed(8)).cuda()
    base = tg.reduction_aggr(g, x, warps_per_block=4, reduce="max")
    for q in (-1, 0.5, 0.999):
        gq = g.repartition(forward_huge_degree_threshold_quantile=q)
        for kw in (dict(warps_per_block=1), dict(warps_per_block=4, edges_per_block_heavy_nodes=32),
                   dict(warps_per_block=2, use_2d_kernel=True, tiles_y=16)):
            assert torch.equal(tg.reduction_aggr(gq, x, reduce="max", **kw), base), (q, kw)


def test_noncontiguous_and_unaligned_inputs():
    n = 500
    ei, g = _graph(n=n, e=4000, hub_degree=300)
    wide = torch.randn(n, 96, generator=torch.Generator().manual_seed(9))
    view = wide.cuda()[:, 16:80]  # row stride 96, 64 columns
    want = O.segment_reduce(wide[:, 16:80].contiguous(), ei, n, "min")
    assert torch.equal(tg.reduction_aggr(g, view, warps_per_block=2, reduce="min").cpu(), want)
    odd = wide.cuda()[:, 1:66]  # misaligned base and odd width: copied and padded by the host
    want = O.segment_reduce(wide[:, 1:66].contiguous(), ei, n, "sum")
    assert rel_err(tg.reduction_aggr(g, odd, warps_per_block=2, reduce="sum"), want) <= FP32_TOL


def test_invalid_parameters_raise_runtime_error():
    ei, g = _graph(n=200, e=1000, hubs=0, hub_degree=0)
    x = torch.randn(200, 128).cuda()  # wide enough that the requested block width is not clamped first
    with pytest.raises(RuntimeError):
        tg.reduction_aggr(g, x, warps_per_block=3, reduce="min")
    with pytest.raises(RuntimeError):
        tg.reduction_aggr(g, x, warps_per_block=1, edges_per_block_heavy_nodes=100, reduce="min")
    with pytest.raises(RuntimeError):
        tg.reduction_aggr(g, x, warps_per_block=1, reduce="median")
    with pytest.raises(RuntimeError):
        tg.reduction_aggr(g, x.double(), warps_per_block=1, reduce="min")
    with pytest.raises(RuntimeError):
        tg.reduction_aggr(g, x.cpu(), warps_per_block=1, reduce="min")
