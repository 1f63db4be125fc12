"""Graph construction kernels (radix sort based COO -> CSR, degree order statistics, row partition)
against the torch ops the reference builds its graph object with (turbo_gnn/graph.py:11-67).
Everything here is integer work: the comparison is bit-exact."""

import pytest
import torch

from turbo_gnn_b200 import graph as tgraph
from turbo_gnn_b200 import graph_build
from turbo_gnn_b200.graph import AdjacencyForwardBackwardWithNodeBuckets as Graph

pytestmark = pytest.mark.gpu


def _edges(n, e, seed, dtype=torch.int64, skew=False):
    g = torch.Generator().manual_seed(seed)
    if skew:  # a few very popular endpoints and many untouched ones
        src = (torch.rand(e, generator=g) ** 4 * n).long().clamp_(max=n - 1)
        dst = (torch.rand(e, generator=g) ** 6 * n).long().clamp_(max=n - 1)
    else:
        src = torch.randint(0, n, (e,), generator=g)
        dst = torch.randint(0, n, (e,), generator=g)
    return torch.stack([src, dst]).to(dtype).cuda()


def _torch_csr(ei, n, transpose):
    ptr, cols, _, counts = tgraph.build_csr_as_is(ei.long(), None, n, do_transpose=transpose)
    return ptr, cols, counts


@pytest.mark.parametrize("n,e,seed,skew", [(1, 5, 0, False), (7, 0, 1, False), (50, 400, 2, False), (1000, 30_000, 3, True),
                                           (20_000, 700_000, 4, True), (300_000, 5_000_000, 5, False)])
@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.int64, torch.int64), (torch.int32, torch.int32),
                                                (torch.int64, torch.int32)])
def test_coo_to_csr_matches_torch(n, e, seed, skew, in_dtype, out_dtype):
    ei = _edges(n, e, seed, in_dtype, skew)
    for transpose in (True, False):
        rows, cols = (ei[1], ei[0]) if transpose else (ei[0], ei[1])
        ptr, idx, order = graph_build.coo_to_csr(rows, cols, n, out_dtype, want_order=True)
        want_ptr, want_idx, _ = _torch_csr(ei, n, transpose)
        assert ptr.dtype == out_dtype and idx.dtype == out_dtype
        assert torch.equal(ptr.long(), want_ptr)
        assert torch.equal(idx.long(), want_idx)
        # the permutation reproduces the sorted edge list, equal pairs in input order
        o = order.long()
        assert torch.equal(cols.long()[o], want_idx)
        key = rows.long()[o] * n + cols.long()[o]
        assert bool((key[1:] >= key[:-1]).all())
        same = key[1:] == key[:-1]
        assert bool((o[1:][same] > o[:-1][same]).all())


def test_coo_to_csr_rejects_ids_out_of_range():
    ei = _edges(100, 1000, 6)
    ei[0, 17] = 100
    with pytest.raises(RuntimeError, match="outside"):
        graph_build.coo_to_csr(ei[1], ei[0], 100)
    ei[0, 17] = -1
    with pytest.raises(RuntimeError, match="outside"):
        graph_build.coo_to_csr(ei[1], ei[0], 100)


@pytest.mark.parametrize("quantile", [0.99, 0.5, 0.0, 1.0, 0.731, -1])
@pytest.mark.parametrize("n,e,seed", [(1, 3, 0), (2, 9, 1), (1000, 20_000, 2), (200_000, 3_000_000, 3)])
@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_bucketing_matches_torch_quantile(quantile, n, e, seed, dtype):
    ei = _edges(n, e, seed, skew=True)
    ptr, _, counts = _torch_csr(ei, n, True)
    want_light, want_heavy = tgraph._bucket_nodes_by_degree(counts, quantile, index_dtype=dtype)
    light, heavy, top = graph_build.bucket_rows(ptr.to(dtype), quantile, index_dtype=dtype)
    assert top == int(counts.max())
    assert light.dtype == dtype and heavy.dtype == dtype
    assert torch.equal(light, want_light)
    assert torch.equal(heavy, want_heavy)


@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64, torch.uint32, None])
@pytest.mark.parametrize("is_directed", [None, True, False])
def test_graph_object_equals_host_build(index_dtype, is_directed):
    n = 5000
    ei = _edges(n, 60_000, 11, skew=True)
    if is_directed is False:
        ei = torch.cat([ei, ei.flip(0)], 1)
    on_gpu = Graph.from_edge_list(ei, n, quantile=0.97, index_dtype=index_dtype, is_directed=is_directed)
    on_host = Graph.from_edge_list(ei.cpu(), n, quantile=0.97, index_dtype=index_dtype, is_directed=is_directed)
    assert on_gpu.is_directed == on_host.is_directed and on_gpu.max_degree == on_host.max_degree
    for name in Graph._INDEX_FIELDS:
        a, b = getattr(on_gpu, name), getattr(on_host, name)
        assert a.dtype == b.dtype, name
        assert torch.equal(tgraph._signed(a).cpu(), tgraph._signed(b)), name
