"""Seeded synthetic graphs and feature tensors with the shapes of the five benchmark workloads.

No public dataset is read anywhere: Chung-Lu and R-MAT generators stand in for
the graphs whose node / edge / feature counts the workloads quote.  Everything
is a pure function of (workload, seed, device type, shrink factor); all ranks
of a multi-GPU run call it with the same arguments and obtain the same graph.
Generation runs with torch ops on the requested device, so the 10^8-edge
graphs are built on the GPU in well under a second.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .graph import AdjacencyForwardBackwardWithNodeBuckets


def _gen(device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def power_law_weights(n: int, exponent: float, lo: float, hi: float, mean: float, gen: torch.Generator) -> torch.Tensor:
    """n expected degrees: truncated Pareto(exponent) on [lo, hi], rescaled to the requested mean."""
    u = torch.rand(n, generator=gen, device=gen.device, dtype=torch.float64)
    a = 1.0 - exponent
    x = (lo**a + u * (hi**a - lo**a)) ** (1.0 / a)
    return x * (mean / x.mean())


def chung_lu_edges(n: int, num_edges: int, w_out: torch.Tensor, w_in: torch.Tensor, gen: torch.Generator) -> torch.Tensor:
    """[2, num_edges] int64: endpoints drawn independently with probability proportional to the weights."""

    def draw(w):
        cdf = torch.cumsum(w / w.sum(), 0)
        cdf[-1] = 1.0
        r = torch.rand(num_edges, generator=gen, device=gen.device, dtype=torch.float64)
        return torch.searchsorted(cdf, r).clamp_(max=n - 1)

    return torch.stack([draw(w_out), draw(w_in)], 0)


def rmat_edges(scale: int, num_edges: int, a: float, b: float, c: float, gen: torch.Generator) -> torch.Tensor:
    """[2, num_edges] int64 R-MAT edges over 2**scale nodes (quadrant probabilities a, b, c, 1-a-b-c)."""
    src = torch.zeros(num_edges, dtype=torch.int64, device=gen.device)
    dst = torch.zeros(num_edges, dtype=torch.int64, device=gen.device)
    for _ in range(scale):
        r = torch.rand(num_edges, generator=gen, device=gen.device)
        right = ((r >= a) & (r < a + b)) | (r >= a + b + c)  # quadrants b and d set the column bit
        down = r >= a + b  # quadrants c and d set the row bit
        src = (src << 1) | down.long()
        dst = (dst << 1) | right.long()
    return torch.stack([src, dst], 0)


def dedup_edges(edge_index: torch.Tensor, n: int) -> torch.Tensor:
    key = torch.unique(edge_index[0] * n + edge_index[1])
    return torch.stack([key // n, key % n], 0)


def add_self_loops(edge_index: torch.Tensor, n: int) -> torch.Tensor:
    loops = torch.arange(n, device=edge_index.device, dtype=edge_index.dtype)
    return torch.cat([edge_index, torch.stack([loops, loops], 0)], 1)


def symmetrise(edge_index: torch.Tensor) -> torch.Tensor:
    return torch.cat([edge_index, edge_index.flip(0)], 1)


def graph_from_edges(edge_index: torch.Tensor, n: int, index_dtype=torch.int32, quantile: float = 0.99,
                     is_directed: bool | None = None) -> AdjacencyForwardBackwardWithNodeBuckets:
    return AdjacencyForwardBackwardWithNodeBuckets.from_edge_list(
        edge_index, n, quantile=quantile, index_dtype=index_dtype, is_directed=is_directed
    )


@dataclass
class Workload:
    """One benchmark case: the graph, its COO edges and the named input tensors."""

    name: str
    op: str  # "reduce" | "gatv2" | "gt" | "spmm" | "gatv2_model"
    num_nodes: int
    edge_index: torch.Tensor
    graph: AdjacencyForwardBackwardWithNodeBuckets
    tensors: dict = field(default_factory=dict)
    params: dict = field(default_factory=dict)

    @property
    def num_edges(self) -> int:
        return self.graph.forward_indices.numel()


def _shrunk(v: int, shrink: float, floor: int = 64) -> int:
    return max(floor, int(round(v * shrink)))


def make_workload(cfg: int, device="cuda", shrink: float = 1.0, index_dtype=None, quantile: float = 0.99) -> Workload:
    """Build workload 0..4; ``shrink`` < 1 scales node and edge counts for tests and profiler captures."""
    device = torch.device(device)
    gen = _gen(device, cfg)
    fgen = _gen(device, 1000 + cfg)

    def randn(*shape, dtype=torch.float32, std=1.0):
        return (torch.randn(*shape, generator=fgen, device=device, dtype=torch.float32) * std).to(dtype)

    if cfg == 0:
        n = _shrunk(20_000, shrink)
        w = power_law_weights(n, 2.1, 1.0, 2000.0, 10.0, gen)
        e = chung_lu_edges(n, int(n * 10), w, w, gen)
        e = dedup_edges(add_self_loops(e, n), n)
        g = graph_from_edges(e, n, index_dtype or torch.int64, quantile)
        return Workload("cfg0_segment_reduce", "reduce", n, e, g, {"x": randn(n, 128)},
                        {"reduce": ["min", "max", "sum", "mean"]})
    if cfg == 1:
        n = _shrunk(169_343, shrink)
        w = power_law_weights(n, 2.0, 1.0, float(max(n // 170, 8)), 6.887, gen)
        e = chung_lu_edges(n, _shrunk(1_166_243, shrink), w, w, gen)
        e = dedup_edges(add_self_loops(symmetrise(e), n), n)
        g = graph_from_edges(e, n, index_dtype or torch.int32, quantile)
        t = {"x": randn(n, 8, 64), "x_neighbors": randn(n, 8, 64), "attention_weights": randn(8, 64, std=0.1),
             "grad": randn(n, 8, 64)}
        return Workload("cfg1_gatv2", "gatv2", n, e, g, t, {"negative_slope": 0.2})
    if cfg == 2:
        n = _shrunk(232_965, shrink)
        mean_deg = min(492.0, n / 8)
        hi = min(19_000.0, n / 2)
        w = power_law_weights(n, 2.2, min(95.0, hi / 8), hi, mean_deg, gen)
        e = chung_lu_edges(n, int(n * mean_deg * 1.04), w, w, gen)
        e = dedup_edges(e, n)
        g = graph_from_edges(e, n, index_dtype or torch.int32, quantile)
        t = {"Q": randn(n, 4, 64), "K": randn(n, 4, 64), "V": randn(n, 4, 64), "grad": randn(n, 4, 64)}
        return Workload("cfg2_graph_transformer", "gt", n, e, g, t, {"scale": 0.125})
    if cfg == 3:
        scale = 22 if shrink >= 1.0 else max(10, 22 + int(round(torch.log2(torch.tensor(shrink)).item())))
        n = 1 << scale
        e = rmat_edges(scale, n * 16, 0.57, 0.19, 0.19, gen)
        e = dedup_edges(e, n)
        g = graph_from_edges(e, n, index_dtype or torch.int32, quantile)
        t = {"x": randn(n, 256, dtype=torch.bfloat16), "grad": randn(n, 256, dtype=torch.bfloat16)}
        return Workload("cfg3_spmm_rmat", "spmm", n, e, g, t, {"norm": ["none", "right"]})
    if cfg == 4:
        n = _shrunk(2_449_029, shrink)
        w = power_law_weights(n, 2.2, 4.0, float(max(n // 100, 16)), 25.5, gen)
        e = chung_lu_edges(n, _shrunk(62_400_000, shrink), w, w, gen)
        e = dedup_edges(symmetrise(e), n)
        g = graph_from_edges(e, n, index_dtype or torch.int32, quantile)
        t = {"features": randn(n, 100)}
        return Workload("cfg4_gatv2_two_layer", "gatv2_model", n, e, g, t,
                        {"layers": [(4, 64), (1, 47)], "negative_slope": 0.2})
    raise ValueError(f"unknown workload {cfg}")
