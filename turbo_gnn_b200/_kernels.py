"""Tunable-kernel declarations: which launch parameters each op exposes to the autotuner.

Mirror of the reference's ``turbo_gnn/_kernels.py`` (``ReductionAggrKernel`` 11-70,
``GATv2AggrKernel`` 73-157, ``GraphTransformerAggrKernel`` 160-238): same class names,
constructor keywords and attribute names.  The grids are re-targeted at the three-tier
schedule of this library:

* ``*_light_warps`` / ``forward_warps_per_block``  warps per CTA in the warp-per-row tier
* ``*_heavy_warps`` / ``forward_tiles_y``          warps per CTA in the CTA-per-row and hub tiers
* ``forward_edges_per_block_heavy_nodes`` / ``hub_chunk_edges``  edges per hub chunk
* ``hub_min_degree``                                degree from which a heavy row is edge-split
* ``*_huge_degree_threshold_quantile``              light/heavy cut of the graph (graph axis)
"""

from __future__ import annotations

from turbo_gnn_b200 import _C
from turbo_gnn_b200._autotune import TunableKernel, TunableParam
from turbo_gnn_b200._functions import ReductionAggrFunction, _FusedGraphAttention, gatv2_function

_QUANTILES = [-1, 0.9, 0.99, 0.999]


def _quantile_axis(side: str) -> list[TunableParam]:
    return [TunableParam(f"{side}_huge_degree_threshold_quantile", list(_QUANTILES), default=-1)]


class _HubTunables:
    """Hub-tier attributes shared by the attention kernels; applied around each execution."""

    hub_chunk_edges = None  # None: derived from the graph
    hub_min_degree = None
    column_tiles = None

    def _hub(self):
        return _C.hub_tier(chunk_edges=self.hub_chunk_edges, hub_min_degree=self.hub_min_degree,
                           column_tiles=self.column_tiles)

    @staticmethod
    def _hub_axes() -> list[TunableParam]:
        return [
            TunableParam("hub_chunk_edges", [None, 2048], default=None),
            TunableParam("hub_min_degree", [None, 4096], default=None),
            TunableParam("column_tiles", [None, 1], default=None),
        ]


class ReductionAggrKernel(TunableKernel):
    """Segment min / max / sum / mean; one shared instance per ``reduce`` mode."""

    def __init__(self, reduce: str = "min", **kwargs):
        super().__init__()
        self.reduce = reduce
        self.forward_warps_per_block = kwargs.get("warps_per_block", 8)
        self.forward_edges_per_block_heavy_nodes = kwargs.get("edges_per_block_heavy_nodes", 128)
        self.forward_use_2d_kernel = kwargs.get("use_2d_kernel", False)
        self.forward_features_per_block = kwargs.get("features_per_block", 32)
        self.forward_tiles_y = kwargs.get("tiles_y", 8)

    def _execute(self, graph, x, **kwargs):
        return ReductionAggrFunction.apply(
            graph.forward_indptr, graph.forward_indices, x, graph.light_nodes, graph.heavy_nodes, graph.max_degree,
            self.forward_warps_per_block, self.forward_edges_per_block_heavy_nodes, self.forward_use_2d_kernel,
            self.forward_features_per_block, self.forward_tiles_y, self.reduce,
        )

    def get_tunable_forward_kernel_params(self) -> list[TunableParam]:
        return [
            TunableParam("forward_warps_per_block", [2, 4, 8], default=8),
            TunableParam("forward_edges_per_block_heavy_nodes", [64, 128, 512], default=128),
            TunableParam("forward_use_2d_kernel", [False, True], default=False),
            TunableParam("forward_tiles_y", [4, 16], default=8),
        ]

    def get_tunable_forward_graph_params(self) -> list[TunableParam]:
        return _quantile_axis("forward")


class GATv2AggrKernel(_HubTunables, TunableKernel):
    """Fused GATv2 aggregation."""

    def __init__(self, **kwargs):
        super().__init__()
        self.backward_grad_A_reduce_row_chunk_size = kwargs.get("grad_A_reduce_row_chunk_size", 512)
        self.forward_light_warps = kwargs.get("forward_light_warps", 1)
        self.forward_heavy_warps = kwargs.get("forward_heavy_warps", 8)
        self.backward_light_warps = kwargs.get("backward_light_warps", 1)
        self.backward_heavy_warps = kwargs.get("backward_heavy_warps", 8)

    def _execute(self, graph, x, *, x_neighbors=None, attention_weights=None, negative_slope=None, **kwargs):
        with self._hub():
            return gatv2_function.apply(
                graph.forward_indptr, graph.forward_indices, graph.backward_indptr, graph.backward_indices, x,
                x_neighbors, attention_weights, negative_slope, self.backward_grad_A_reduce_row_chunk_size,
                graph.forward_light_nodes, graph.forward_heavy_nodes, graph.backward_light_nodes,
                graph.backward_heavy_nodes, self.forward_light_warps, self.forward_heavy_warps,
                self.backward_light_warps, self.backward_heavy_warps, graph.is_directed,
            )

    def get_tunable_forward_kernel_params(self) -> list[TunableParam]:
        return [
            TunableParam("forward_light_warps", [1, 2, 4], default=1),
            TunableParam("forward_heavy_warps", [8, 16], default=8),
            *self._hub_axes(),
        ]

    def get_tunable_forward_graph_params(self) -> list[TunableParam]:
        return _quantile_axis("forward")

    def get_tunable_backward_kernel_params(self) -> list[TunableParam]:
        return [
            TunableParam("backward_grad_A_reduce_row_chunk_size", [32, 64, 128, 256, 512, 1024, 2048], default=512),
            TunableParam("backward_light_warps", [1, 2, 4], default=1),
            TunableParam("backward_heavy_warps", [8, 16], default=8),
        ]

    def get_tunable_backward_graph_params(self) -> list[TunableParam]:
        return _quantile_axis("backward")

    def make_forward_bench_fn(self, x, graph_repr, **kwargs):
        fixed = {k: kwargs[k] for k in ("x_neighbors", "attention_weights", "negative_slope")}
        return lambda: self._execute(graph_repr, x, **fixed)


class GraphTransformerAggrKernel(_HubTunables, TunableKernel):
    """Fused multi-head graph-transformer attention."""

    def __init__(self, **kwargs):
        super().__init__()
        self.forward_light_warps = kwargs.get("forward_light_warps", 4)
        self.forward_heavy_warps = kwargs.get("forward_heavy_warps", 8)
        self.backward_light_warps = kwargs.get("backward_light_warps", 1)
        self.backward_heavy_warps = kwargs.get("backward_heavy_warps", 8)

    def _execute(self, graph, x, *, Q=None, K=None, V=None, scale=None, **kwargs):
        with self._hub():
            return _FusedGraphAttention.apply(
                graph.forward_indptr, graph.forward_indices, graph.backward_indptr, graph.backward_indices, Q, K, V,
                scale, graph.forward_light_nodes, graph.forward_heavy_nodes, graph.backward_light_nodes,
                graph.backward_heavy_nodes, self.forward_light_warps, self.forward_heavy_warps,
                self.backward_light_warps, self.backward_heavy_warps, graph.is_directed,
            )

    def get_tunable_forward_kernel_params(self) -> list[TunableParam]:
        return [
            TunableParam("forward_light_warps", [1, 2, 4], default=4),
            TunableParam("forward_heavy_warps", [8, 16], default=8),
            *self._hub_axes(),
        ]

    def get_tunable_forward_graph_params(self) -> list[TunableParam]:
        return _quantile_axis("forward")

    def get_tunable_backward_kernel_params(self) -> list[TunableParam]:
        return [
            TunableParam("backward_light_warps", [1, 2, 4], default=1),
            TunableParam("backward_heavy_warps", [8, 16], default=8),
        ]

    def get_tunable_backward_graph_params(self) -> list[TunableParam]:
        return _quantile_axis("backward")

    def make_forward_bench_fn(self, x, graph_repr, **kwargs):
        fixed = {k: kwargs[k] for k in ("Q", "K", "V", "scale")}
        return lambda: self._execute(graph_repr, x, **fixed)
