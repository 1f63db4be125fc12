"""Sweep harness: argument handling, table layout and the torch scatter comparator (host only)."""

import torch

from helpers import random_edges
from oracle import scatter_oracle as O
from turbo_gnn_b200 import sweep


def test_arguments_and_defaults():
    a = sweep.parse_args(["--conv_type", "gt", "--workloads", "cfg1", "cfg2", "--precisions", "none", "bf16",
                          "--graph_modes", "directed", "undirected", "--hidden", "32", "64", "--heads", "4"])
    assert a.conv_type == "gt" and a.workloads == ["cfg1", "cfg2"] and a.hidden == [32, 64] and a.heads == [4]
    assert a.precisions == ["none", "bf16"] and a.graph_modes == ["directed", "undirected"] and not a.no_reference


def test_table_has_one_line_per_row_and_handles_missing_comparator():
    rows = [sweep.SweepRow("gt", "cfg1", "none", "directed", 64, 4, 10, 20, 1.0, 2.0, 30.0, 60.0, 1e-6),
            sweep.SweepRow("sum", "cfg3", "bf16", "undirected", 256, 1, 10, 20, 1.0, None, None, None, None)]
    text = sweep.format_table(rows).splitlines()
    assert len(text) == 4 and text[0].count("|") == text[2].count("|") == text[3].count("|")
    assert "30.0" in text[2] and rows[0].speedup == 30.0 and rows[1].speedup is None


def test_comparator_agrees_with_the_oracle():
    n = 300
    ei = random_edges(n, 3000, 5, hubs=2, hub_degree=100, self_loops=True)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(n, 24, generator=g)
    for conv in ("min", "max", "sum", "mean"):
        got = sweep.scatter_reference(conv, ei, n, {"x": x}, {})
        assert torch.allclose(got, O.segment_reduce(x, ei, n, conv), atol=1e-5), conv
    l, r, a = torch.randn(n, 2, 8, generator=g), torch.randn(n, 2, 8, generator=g), torch.randn(2, 8, generator=g)
    got = sweep.scatter_reference("gatv2", ei, n, {"x": l, "x_neighbors": r, "attention_weights": a}, {})
    assert torch.allclose(got, O.gatv2_aggregate(l, r, a, ei, n, 0.2), atol=1e-5)
    q, k, v = (torch.randn(n, 2, 8, generator=g) for _ in range(3))
    got = sweep.scatter_reference("gt", ei, n, {"Q": q, "K": k, "V": v}, {"scale": 0.3})
    assert torch.allclose(got, O.gt_aggregate(q, k, v, ei, n, 0.3), atol=1e-5)
