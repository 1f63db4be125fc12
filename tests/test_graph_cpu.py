"""graph.py against fixtures produced by the reference's own turbo_gnn/graph.py (bit-exact)."""

import os

import pytest
import torch

from turbo_gnn_b200.graph import (
    AdjacencyForwardBackwardWithNodeBuckets as Graph,
    _bucket_nodes_by_degree,
    build_csr_as_is,
)

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "graph_cases.pt")
FIELDS = ("forward_indptr", "forward_indices", "backward_indptr", "backward_indices", "forward_light_nodes",
          "forward_heavy_nodes", "backward_light_nodes", "backward_heavy_nodes")
DTYPES = {None: None, "None": None, "torch.int32": torch.int32, "torch.int64": torch.int64}


def _cases():
    return torch.load(GOLDEN, weights_only=False)


@pytest.mark.parametrize("idx", range(6))
def test_from_edge_list_is_bit_exact(idx):
    rec = _cases()[idx]
    c = rec["case"]
    g = Graph.from_edge_list(rec["edge_index"], c["n"], quantile=c["quantile"], index_dtype=DTYPES[c["index_dtype"]],
                             is_directed=c["is_directed"])
    for f in FIELDS:
        got, want = getattr(g, f), rec[f]
        assert got.dtype == want.dtype and torch.equal(got, want), f
    assert g.max_degree == rec["max_degree"]
    assert g.is_directed == rec["is_directed"]
    assert (g.backward_indptr.data_ptr() == g.forward_indptr.data_ptr()) == rec["aliased"]
    r = g.repartition(forward_huge_degree_threshold_quantile=0.5)
    assert torch.equal(r.forward_light_nodes, rec["repart_fwd_light"])
    assert torch.equal(r.forward_heavy_nodes, rec["repart_fwd_heavy"])
    assert torch.equal(r.backward_light_nodes, rec["repart_bwd_light"])
    assert r.forward_indptr.data_ptr() == g.forward_indptr.data_ptr()  # CSR shared, not copied
    g2 = Graph.from_csr(g.forward_indptr, g.forward_indices, g.backward_indptr, g.backward_indices, quantile=0.75,
                        index_dtype=DTYPES[c["index_dtype"]], is_directed=c["is_directed"])
    assert torch.equal(g2.forward_heavy_nodes, rec["from_csr_fwd_heavy"])
    assert torch.equal(g2.backward_heavy_nodes, rec["from_csr_bwd_heavy"])


def test_csr_layout_and_direction():
    ei = torch.tensor([[0, 2, 2, 1], [1, 1, 0, 2]])  # src -> dst
    g = Graph.from_edge_list(ei, 3, quantile=-1)
    # forward rows are destinations listing sources in ascending order
    assert g.forward_indptr.tolist() == [0, 1, 3, 4]
    assert g.forward_indices.tolist() == [2, 0, 2, 1]
    assert g.backward_indptr.tolist() == [0, 1, 2, 4]
    assert g.backward_indices.tolist() == [1, 2, 0, 1]
    assert g.forward_heavy_nodes.numel() == 0 and g.light_nodes.tolist() == [0, 1, 2]
    assert g.max_degree == 2 and g.is_directed is True


def test_bucket_threshold_uses_fp32_quantile():
    deg = torch.tensor([1, 1, 2, 3, 10, 50])
    light, heavy = _bucket_nodes_by_degree(deg, 0.5)
    cut = torch.quantile(deg.float(), 0.5).item()
    assert light.tolist() == [i for i, d in enumerate(deg.tolist()) if d < cut]
    assert heavy.tolist() == [i for i, d in enumerate(deg.tolist()) if d >= cut]
    light, heavy = _bucket_nodes_by_degree(deg, -1, index_dtype=torch.int32)
    assert heavy.numel() == 0 and light.dtype == torch.int32 and light.numel() == 6


def test_build_csr_keeps_duplicates_and_weights():
    ei = torch.tensor([[1, 0, 1, 1], [0, 1, 0, 2]])
    w = torch.tensor([0.5, 1.5, 2.5, 3.5])
    ptr, cols, ww, counts = build_csr_as_is(ei, w, 3, do_transpose=False)
    assert ptr.tolist() == [0, 1, 4, 4] and cols.tolist() == [1, 0, 0, 2] and counts.tolist() == [1, 3, 0]
    assert sorted(ww[1:3].tolist()) == [0.5, 2.5] and ww[0].item() == 1.5 and ww[3].item() == 3.5


def test_undirected_detection_aliasing_and_to():
    ei = torch.tensor([[0, 1, 1, 2], [1, 0, 2, 1]])
    g = Graph.from_edge_list(ei, 3, quantile=-1, index_dtype=torch.int32)
    assert g.is_directed is False
    assert g.backward_indptr is g.forward_indptr and g.backward_indices is g.forward_indices
    assert g.to("cpu") is g and g.backward_indices is g.forward_indices
    r = g.repartition(backward_huge_degree_threshold_quantile=0.5)
    assert r.is_directed is False and r.backward_indptr is r.forward_indptr
    assert r.index_dtype == torch.int32 and g.device.type == "cpu"


def test_unsigned_index_dtype_round_trip():
    ei = torch.tensor([[0, 1, 2, 2], [1, 2, 0, 1]])
    g = Graph.from_edge_list(ei, 3, quantile=0.5, index_dtype=torch.uint32)
    assert g.forward_indptr.dtype == torch.uint32 and g.forward_light_nodes.dtype == torch.uint32
    assert g.max_degree == 2
    assert Graph._to_signed_view(g.forward_indptr).dtype == torch.int32


def test_mixed_dtypes_rejected():
    ei = torch.tensor([[0, 1], [1, 0]])
    g = Graph.from_edge_list(ei, 2)
    with pytest.raises(AssertionError):
        Graph(g.forward_indptr, g.forward_indices.int(), g.backward_indptr, g.backward_indices, g.forward_light_nodes,
              g.forward_heavy_nodes, g.backward_light_nodes, g.backward_heavy_nodes)
