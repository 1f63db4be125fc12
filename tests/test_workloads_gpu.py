"""The five benchmark workloads: shrunken copies against the oracle, full sizes through properties
that do not need a CPU result (constant-value rows, linearity, gradient identities)."""

import pytest
import torch

import turbo_gnn_b200 as tg
from helpers import rel_err
from oracle import scatter_oracle as O
from turbo_gnn_b200 import synthetic

pytestmark = pytest.mark.gpu


def _cpu_edges(wl):
    g = wl.graph
    ptr = g.forward_indptr.long().cpu()
    dst = torch.repeat_interleave(torch.arange(wl.num_nodes), ptr[1:] - ptr[:-1])
    return torch.stack([g.forward_indices.long().cpu(), dst])


def test_cfg0_shrunk_all_reductions_int64():
    wl = synthetic.make_workload(0, "cuda", shrink=0.25)
    assert wl.graph.index_dtype == torch.int64
    ei, x = _cpu_edges(wl), wl.tensors["x"]
    for red in ("min", "max", "sum", "mean"):
        got = tg.reduction_aggr(wl.graph, x, warps_per_block=4, reduce=red)
        want = O.segment_reduce(x.cpu(), ei, wl.num_nodes, red)
        if red in ("min", "max"):
            assert torch.equal(got.cpu(), want)
        else:
            assert rel_err(got, want) <= 1e-5


def test_cfg1_shrunk_gatv2_forward_backward():
    wl = synthetic.make_workload(1, "cuda", shrink=0.02)
    assert wl.graph.is_directed is False  # symmetrised + self loops
    ei, t, n = _cpu_edges(wl), wl.tensors, wl.num_nodes
    dev = [t[k].clone().requires_grad_() for k in ("x", "x_neighbors", "attention_weights")]
    tg.gatv2_aggr(wl.graph, *dev, 0.2).backward(t["grad"])
    ref = [t[k].cpu().double().requires_grad_() for k in ("x", "x_neighbors", "attention_weights")]
    O.gatv2_aggregate(*ref, ei, n, 0.2).backward(t["grad"].cpu().double())
    for a, b in zip(dev, ref):
        assert rel_err(a.grad, b.grad) <= 1e-5


def test_cfg2_shrunk_graph_transformer_forward_backward():
    wl = synthetic.make_workload(2, "cuda", shrink=0.01)
    ei, t, n = _cpu_edges(wl), wl.tensors, wl.num_nodes
    dev = [t[k].clone().requires_grad_() for k in ("Q", "K", "V")]
    out = tg.graph_transformer_aggr(wl.graph, None, *dev, 0.125)
    out.backward(t["grad"])
    ref = [t[k].cpu().double().requires_grad_() for k in ("Q", "K", "V")]
    want = O.gt_aggregate(*ref, ei, n, 0.125)
    want.backward(t["grad"].cpu().double())
    assert rel_err(out, want.detach()) <= 1e-5
    for a, b in zip(dev, ref):
        assert rel_err(a.grad, b.grad) <= 1e-5


def test_cfg3_shrunk_spmm_bf16():
    wl = synthetic.make_workload(3, "cuda", shrink=2**-8)
    ei, t, n = _cpu_edges(wl), wl.tensors, wl.num_nodes
    g = wl.graph
    for norm in ("none", "right"):
        x = t["x"].clone().requires_grad_()
        out = tg.spmm_aggr(x, g.forward_indptr, g.forward_indices, norm, -1, 256)
        out.backward(t["grad"])
        xr = t["x"].cpu().double().requires_grad_()
        want = O.spmm(xr, ei, n, norm)
        want.backward(t["grad"].cpu().double())
        assert rel_err(out.float(), want.detach()) <= 2e-2
        assert rel_err(x.grad.float(), xr.grad) <= 2e-2


def test_cfg2_full_size_properties():
    wl = synthetic.make_workload(2, "cuda")
    g, t, n = wl.graph, wl.tensors, wl.num_nodes
    assert 100_000_000 < wl.num_edges < 130_000_000
    deg = (g.forward_indptr[1:] - g.forward_indptr[:-1]).long()
    has_edges = deg > 0
    # (1) V == const => every non-empty row returns that constant, whatever the scores are
    ones = torch.ones_like(t["V"])
    out = tg.graph_transformer_aggr(g, None, t["Q"], t["K"], ones, 0.125)
    assert (out[has_edges] - 1).abs().max() <= 1e-5 and out[~has_edges].eq(0).all()
    # (2) Q == 0 => uniform attention => the fused op equals the mean aggregation of V
    zero_q = torch.zeros_like(t["Q"])
    out = tg.graph_transformer_aggr(g, None, zero_q, t["K"], t["V"], 0.125)
    mean = tg.reduction_aggr(g, t["V"].reshape(n, -1), warps_per_block=2, reduce="mean").view_as(out)
    assert rel_err(out, mean.cpu()) <= 1e-5
    # (3) softmax gradient identity: sum over sources of dV equals sum over destinations of dO,
    #     because every destination's weights sum to one
    q, k, v = (t[name].clone().requires_grad_() for name in ("Q", "K", "V"))
    tg.graph_transformer_aggr(g, None, q, k, v, 0.125).backward(t["grad"])
    lhs = v.grad.double().sum(0)
    rhs = t["grad"][has_edges].double().sum(0)
    assert (lhs - rhs).abs().max() / rhs.abs().max() <= 1e-4
    # (4) shifting K of a destination along Q-independent directions leaves dQ finite and dK rows of
    #     empty destinations zero
    assert torch.isfinite(q.grad).all() and torch.isfinite(k.grad).all()
    assert k.grad[~has_edges].eq(0).all()


def test_cfg3_full_size_properties():
    wl = synthetic.make_workload(3, "cuda")
    g, t, n = wl.graph, wl.tensors, wl.num_nodes
    assert n == 1 << 22 and g.index_dtype == torch.int32
    deg = (g.forward_indptr[1:] - g.forward_indptr[:-1]).float()
    ones = torch.ones(n, 256, dtype=torch.bfloat16, device="cuda")
    # A @ 1 = in-degree (exact in fp32 accumulation; bf16 rounding of the stored result only)
    out = tg.spmm_aggr(ones, g.forward_indptr, g.forward_indices, "none", -1, 256)
    assert torch.equal(out[:, 0].float(), deg.bfloat16().float()) and torch.equal(out[:, 0], out[:, 255])
    # mean of ones is one on every non-empty row
    out = tg.spmm_aggr(ones, g.forward_indptr, g.forward_indices, "right", -1, 256)
    assert torch.equal(out[:, 3].float(), (deg > 0).float())
    # transpose: 1^T A = out-degree
    x = ones.clone().requires_grad_()
    tg.spmm_aggr(x, g.forward_indptr, g.forward_indices, "none", -1, 256).backward(ones)
    out_deg = torch.bincount(g.forward_indices.long(), minlength=n).float()
    assert torch.equal(x.grad[:, 7].float(), out_deg.bfloat16().float())
    # linearity in fp32: A(2x) == 2 A(x) bit for bit (scaling by two is exact)
    xf = t["x"][:, :64].float().contiguous()
    a = tg.spmm_aggr(xf, g.forward_indptr, g.forward_indices, "none", -1, 256)
    b = tg.spmm_aggr(2 * xf, g.forward_indptr, g.forward_indices, "none", -1, 256)
    assert torch.equal(2 * a, b)


def test_cfg1_full_size_min_max_sanity():
    wl = synthetic.make_workload(1, "cuda")
    g, n = wl.graph, wl.num_nodes
    x = wl.tensors["x"].reshape(n, -1)
    mn = tg.reduction_aggr(g, x, reduce="min")
    mx = tg.reduction_aggr(g, x, reduce="max")
    mean = tg.reduction_aggr(g, x, reduce="mean")
    assert (mn <= mean + 1e-5).all() and (mean <= mx + 1e-5).all()
    # self loops: every node sees itself
    assert (mn <= x).all() and (mx >= x).all()
    # idempotence: min over the same neighbourhood of a constant field is that constant
    c = torch.full_like(x, 3.25)
    assert tg.reduction_aggr(g, c, reduce="min").eq(3.25).all()
