"""Drop-in behaviour on the GPU: autotune=True, AMP, the raw C ABI, and the sharded ops at world size 1."""

import ctypes

import pytest
import torch

import turbo_gnn_b200 as tg
from helpers import make_graph, random_edges, rel_err
from oracle import scatter_oracle as O
from turbo_gnn_b200 import _abi, _C, _schedule
from turbo_gnn_b200 import dist as tdist
from turbo_gnn_b200._autotune import AutotuneConfig, TunableKernel

pytestmark = pytest.mark.gpu

FAST = AutotuneConfig(warmup=1, iters=1)


@pytest.fixture(autouse=True)
def _fresh_singletons():
    TunableKernel._shared_instances.clear()
    yield
    TunableKernel._shared_instances.clear()


def _graph(n=800, seed=1, idt=torch.int32):
    ei = random_edges(n, 8 * n, seed, hubs=2, hub_degree=n // 2)
    return ei, make_graph(ei, n, idt, quantile=0.95)


def test_reduction_autotune_matches_default_and_caches():
    ei, g = _graph()
    x = torch.randn(800, 64).cuda()
    base = tg.reduction_aggr(g, x, warps_per_block=2, reduce="max")
    tuned = tg.reduction_aggr(g, x, reduce="max", autotune=True, autotune_config=FAST)
    assert torch.equal(tuned, base)
    kernel = tg.ReductionAggrKernel._get_or_create(reduce="max")
    assert kernel._inline_cache.lookup(g, 64) is not None
    assert kernel._inline_cache.lookup(g, 32) is None
    assert torch.equal(tg.reduction_aggr(g, x, reduce="max", autotune=True), base)  # cache hit
    assert tg.ReductionAggrKernel._get_or_create(reduce="min") is not kernel
    xg = x.clone().requires_grad_()
    tg.reduction_aggr(g, xg, reduce="max", autotune=True).sum().backward()
    assert xg.grad is not None and torch.isfinite(xg.grad).all()


def test_attention_autotune_and_direct_kernel_call():
    ei, g = _graph()
    n, h, d = 800, 2, 32
    q, k, v = (torch.randn(n, h, d, generator=torch.Generator().manual_seed(i)).cuda() for i in range(3))
    a = (torch.randn(h, d, generator=torch.Generator().manual_seed(9)) * 0.1).cuda()
    base = tg.gatv2_aggr(g, q, k, a, 0.2)
    tuned = tg.gatv2_aggr(g, q, k, a, 0.2, autotune=True, autotune_config=FAST)
    assert rel_err(tuned, base.cpu()) <= 1e-6
    base = tg.graph_transformer_aggr(g, q, q, k, v, 0.25)
    tuned = tg.graph_transformer_aggr(g, q, q, k, v, 0.25, autotune=True, autotune_config=FAST)
    assert rel_err(tuned, base.cpu()) <= 1e-6
    kern = tg.GraphTransformerAggrKernel()
    out = kern(g, q, autotune=True, autotune_config=FAST, Q=q, K=k, V=v, scale=0.25)
    assert out.shape == (n, h, d) and rel_err(out, base.cpu()) <= 1e-6
    qg = q.clone().requires_grad_()
    tg.graph_transformer_aggr(g, q, qg, k, v, 0.25, autotune=True).sum().backward()
    assert torch.isfinite(qg.grad).all()


def test_autocast_casts_like_the_reference():
    ei, g = _graph()
    x = torch.randn(800, 64).cuda()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = tg.reduction_aggr(g, x, warps_per_block=1, reduce="min")
    assert out.dtype == torch.bfloat16
    assert torch.equal(out.cpu().float(), O.segment_reduce(x.cpu().bfloat16().float(), ei, 800, "min"))


def test_raw_c_abi_call_with_plain_pointers():
    """The library is usable without any of the Python host: raw pointers in, status out."""
    ei, g = _graph(n=500, seed=3)
    n, f = 500, 64
    x = torch.randn(n, f, generator=torch.Generator().manual_seed(4))
    xd = x.cuda()
    out = torch.empty(n, f, device="cuda")
    sched = _schedule.split_tiers(g.forward_indptr, g.forward_light_nodes, g.forward_heavy_nodes, 64, 100)
    need = _abi.workspace_bytes(_abi.OP_WEIGHTED_SUM, torch.float32, torch.int32, sched.num_chunks, f)
    assert sched.num_chunks > 0 and need > 0
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    args = _abi.SegmentReduceArgs()
    args.exec.device, args.exec.stream = 0, torch.cuda.current_stream().cuda_stream
    args.csr.indptr, args.csr.indices = g.forward_indptr.data_ptr(), g.forward_indices.data_ptr()
    args.csr.num_rows, args.csr.num_cols, args.csr.num_edges, args.csr.itype = n, n, g.forward_indices.numel(), 0
    args.sched = sched.to_struct(4, 8)
    for m, t in ((args.x, xd), (args.out, out)):
        m.data, m.rows, m.cols, m.row_stride, m.dtype = t.data_ptr(), n, f, f, 0
    args.reduce, args.workspace, args.workspace_bytes = 2, ws.data_ptr(), need
    lib = _abi.load_library()
    assert lib.tgnn_segment_reduce_forward(ctypes.byref(args)) == 0
    assert rel_err(out, O.segment_reduce(x, ei, n, "sum")) <= 1e-5
    # too little scratch is reported, not overrun
    args.workspace_bytes = 16
    assert lib.tgnn_segment_reduce_forward(ctypes.byref(args)) == -4
    assert "scratch" in _abi.last_error()
    # wrong launch parameter
    args.workspace_bytes = need
    args.sched.light_warps = 3
    assert lib.tgnn_segment_reduce_forward(ctypes.byref(args)) == -3


def test_runs_on_a_side_stream():
    ei, g = _graph()
    x = torch.randn(800, 128).cuda()
    want = tg.reduction_aggr(g, x, warps_per_block=4, reduce="sum")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        got = tg.reduction_aggr(g, x, warps_per_block=4, reduce="sum")
    side.synchronize()
    assert torch.equal(got, want)


def test_sharded_ops_at_world_size_one_equal_the_plain_ops():
    ei, g = _graph(n=700, seed=5)
    n, h, d = 700, 4, 32
    shard = tdist.shard_graph(g, 0, 1, quantile=0.95)
    assert shard.num_local == n and shard.max_rows >= n
    q, k, v, up = (torch.randn(n, h, d, generator=torch.Generator().manual_seed(20 + i)).cuda() for i in range(4))
    ref = [t.clone().requires_grad_() for t in (q, k, v)]
    tg.graph_transformer_aggr(g, None, *ref, 0.25).backward(up)
    got = [t.clone().requires_grad_() for t in (q, k, v)]
    out = tdist.sharded_graph_transformer_aggr(shard, *got, 0.25)
    out.backward(up)
    for a, b in zip(got, ref):
        assert rel_err(a.grad, b.grad.cpu()) <= 1e-6
    a = (torch.randn(h, d, generator=torch.Generator().manual_seed(30)) * 0.1).cuda()
    ref = [t.clone().requires_grad_() for t in (q, k, a)]
    tg.gatv2_aggr(g, *ref, 0.2).backward(up)
    got = [t.clone().requires_grad_() for t in (q, k, a)]
    tdist.sharded_gatv2_aggr(shard, *got, 0.2).backward(up)
    for x1, x2 in zip(got, ref):
        assert rel_err(x1.grad, x2.grad.cpu()) <= 1e-5
    x = torch.randn(n, 64, generator=torch.Generator().manual_seed(31)).cuda()
    for norm in ("none", "right", "both"):
        xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
        ya = tdist.sharded_spmm_aggr(shard, xa, norm)
        yb = tg.spmm_aggr(xb, g.forward_indptr, g.forward_indices, norm, -1, 256)
        ya.sum().backward()
        yb.sum().backward()
        assert rel_err(ya, yb.detach().cpu()) <= 1e-6 and rel_err(xa.grad, xb.grad.cpu()) <= 1e-6


def test_calls_can_be_captured_in_a_cuda_graph_and_replayed():
    """Light + heavy + hub tiers of two ops inside one captured graph (the fork to the library's
    side stream and the join back are part of the capture); replays follow the inputs."""
    from helpers import make_graph, random_edges
    from oracle import scatter_oracle as O

    n = 3000
    ei = random_edges(n, 20 * n, 77, hubs=3, hub_degree=2500)
    g = make_graph(ei, n, torch.int32, quantile=0.9)
    x = torch.randn(n, 64, device="cuda")
    q, k, v = (torch.randn(n, 2, 32, device="cuda") for _ in range(3))
    with _C.hub_tier(cta_min_degree=64, hub_min_degree=1024, chunk_edges=256):
        for _ in range(2):  # warm-up outside the capture: schedules, side stream, caches
            tg.reduction_aggr(g, x, reduce="sum")
            tg.graph_transformer_aggr(g, None, q, k, v, 0.2)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            s_out = tg.reduction_aggr(g, x, reduce="sum")
            a_out = tg.graph_transformer_aggr(g, None, q, k, v, 0.2)
    for seed in (1, 2):
        gen = torch.Generator(device="cuda").manual_seed(seed)
        x.copy_(torch.randn(n, 64, device="cuda", generator=gen))
        q.copy_(torch.randn(n, 2, 32, device="cuda", generator=gen))
        graph.replay()
        torch.cuda.synchronize()
        assert rel_err(s_out, O.segment_reduce(x.cpu(), ei, n, "sum")) <= 1e-5
        assert rel_err(a_out, O.gt_aggregate(q.cpu(), k.cpu(), v.cpu(), ei, n, 0.2)) <= 1e-5


def test_event_between_the_graph_transformer_backward_halves():
    """dQ and dV are final when the event fires, before the dK pass has run."""
    n = 2000
    ei = random_edges(n, 30 * n, 78)
    g = make_graph(ei, n, torch.int32)
    q, k, v = (torch.randn(n, 4, 32, device="cuda", requires_grad=True) for _ in range(3))
    out = tg.graph_transformer_aggr(g, None, q, k, v, 0.2)
    up = torch.randn_like(out)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), up)
    ev = tg.gt_source_grads_ready()
    assert ev is not None
    side = torch.cuda.Stream()
    side.wait_event(ev)
    with torch.cuda.stream(side):
        dq_host = dq.to("cpu", non_blocking=False)
    ref = [t.detach().double().cpu().requires_grad_() for t in (q, k, v)]
    want = O.gt_aggregate(*ref, ei, n, 0.2)
    want.backward(up.double().cpu())
    assert rel_err(dq_host, ref[0].grad) <= 1e-5 and rel_err(dk, ref[1].grad) <= 1e-5
