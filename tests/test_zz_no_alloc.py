"""tgnn_spmm_static_scratch: the SpMM entry point for hosts that cannot supply scratch memory.

Some hosts of this library only pass on device pointers they were given (a cgo / JNI / ctypes
binding with no device allocator) or run with all device memory reserved at start-up, so they can
provide inputs and the output but not the hub-tier scratch.  For them the library keeps a fixed
scratch array of its own.  This test drives that entry point through the raw C ABI exactly as such
a host would -- every buffer exists before the first call, nothing is allocated in between -- and
compares it with tgnn_spmm (caller scratch) on two calls in a row, the second one with other
inputs so that stale partial results from the first call would show.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""

import ctypes

import pytest
import torch

from helpers import make_graph, random_edges
from turbo_gnn_b200 import _abi, _schedule

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 8 << 20  # TGNN_STATIC_SCRATCH_BYTES in include/tgnn_abi.h


def _args(graph, sched, x, out, row_scale=None, workspace=None):
    n_rows = graph.forward_indptr.numel() - 1
    a = _abi.SpmmArgs()
    a.exec.device = x.device.index
    a.exec.stream = torch.cuda.current_stream().cuda_stream
    a.csr = _abi.csr_of(graph.forward_indptr, graph.forward_indices, x.shape[0])
    a.sched = sched.to_struct(4, 8)
    a.x, a.out = _abi.mat_of(x), _abi.mat_of(out)
    a.row_scale = _abi.ptr(row_scale)
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    assert a.out.rows == n_rows
    return a


@pytest.mark.parametrize("dt,feat", [(torch.float32, 128), (torch.bfloat16, 256)])
def test_static_scratch_matches_caller_scratch_twice_in_a_row(dt, feat):
    lib = _abi.load_library()
    n = 3000
    ei = random_edges(n, 20000, 41, hubs=4, hub_degree=2500)
    graph = make_graph(ei, n, torch.int32, quantile=0.9)
    sched = _schedule.split_tiers(graph.forward_indptr, graph.forward_light_nodes, graph.forward_heavy_nodes,
                                  chunk_edges=128, hub_min_degree=1000)
    assert sched.num_chunks > 20  # the hub tier, i.e. the scratch, is really in use
    need = _abi.workspace_bytes(_abi.OP_WEIGHTED_SUM, dt, torch.int32, sched.num_chunks, feat)
    assert 0 < need <= STATIC_SCRATCH_BYTES

    gen = torch.Generator().manual_seed(42)
    inputs = [torch.randn(n, feat, generator=gen).to(dt).cuda() for _ in range(2)]
    scale = (torch.rand(n, generator=gen) + 0.5).cuda()
    caller_ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    want = [torch.empty(n, feat, dtype=dt, device="cuda") for _ in range(2)]
    got = [torch.full((n, feat), float("nan"), dtype=dt, device="cuda") for _ in range(2)]
    torch.cuda.synchronize()

    for x, w in zip(inputs, want):
        assert lib.tgnn_spmm(ctypes.byref(_args(graph, sched, x, w, scale, caller_ws))) == 0, _abi.last_error()
    before = torch.cuda.memory_allocated()
    for x, g in zip(inputs, got):  # two calls back to back, no scratch passed, nothing allocated
        assert lib.tgnn_spmm_static_scratch(ctypes.byref(_args(graph, sched, x, g, scale))) == 0, _abi.last_error()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    for g, w in zip(got, want):
        # same kernels, same order of operations: the results agree bit for bit, which is well
        # inside the 1e-5 (fp32) / 2e-2 (bf16) bars of the other tests
        assert torch.equal(g, w)
    assert not torch.equal(got[0], got[1])


def test_static_scratch_refuses_oversized_schedules():
    lib = _abi.load_library()
    n = 3000
    ei = random_edges(n, 20000, 43, hubs=40, hub_degree=2500)
    graph = make_graph(ei, n, torch.int32, quantile=0.9)
    sched = _schedule.split_tiers(graph.forward_indptr, graph.forward_light_nodes, graph.forward_heavy_nodes,
                                  chunk_edges=32, hub_min_degree=32)
    feat = 2048
    need = _abi.workspace_bytes(_abi.OP_WEIGHTED_SUM, torch.float32, torch.int32, sched.num_chunks, feat)
    assert need > STATIC_SCRATCH_BYTES
    x = torch.randn(n, feat, device="cuda")
    out = torch.empty(n, feat, device="cuda")
    status = lib.tgnn_spmm_static_scratch(ctypes.byref(_args(graph, sched, x, out)))
    assert status == -4
    msg = _abi.last_error()
    assert str(need) in msg and str(STATIC_SCRATCH_BYTES) in msg
