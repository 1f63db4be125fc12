"""turbo_gnn_b200 -- GNN aggregation kernels for NVIDIA B200 behind the ``turbo_gnn`` API.

Public surface (identical names to the reference package ``turbo_gnn``):

- :class:`AdjacencyForwardBackwardWithNodeBuckets` -- dual-CSR graph with degree buckets
- :func:`reduction_aggr`  -- segment min / max (also sum / mean) over incoming neighbours
- :func:`gatv2_aggr`      -- fused GATv2 attention aggregation
- :func:`graph_transformer_aggr` -- fused multi-head dot-product graph attention
- :func:`spmm_aggr`, :func:`csr_SPMM_normalized` -- normalised sparse x dense product
- autotuning: ``autotune=True`` on the three tunable ops, :class:`AutotuneConfig`,
  :class:`TunableKernel`, :class:`TunableParam`, :func:`with_autotune`

All compute runs in ``libturbo_gnn_b200.so`` (hand-written CUDA for sm_100a, C ABI in
``include/tgnn_abi.h``); build it with ``python -m turbo_gnn_b200.build``.
"""

from turbo_gnn_b200._autotune import AutotuneConfig, TunableKernel, TunableParam, with_autotune
from turbo_gnn_b200._kernels import GATv2AggrKernel, GraphTransformerAggrKernel, ReductionAggrKernel
from turbo_gnn_b200._C import gt_source_grads_ready, source_rows_arriving
from turbo_gnn_b200.graph import AdjacencyForwardBackwardWithNodeBuckets
from turbo_gnn_b200.ops import (
    csr_SPMM_normalized,
    gatv2_aggr,
    graph_transformer_aggr,
    reduction_aggr,
    spmm_aggr,
)

__all__ = [
    "AdjacencyForwardBackwardWithNodeBuckets",
    "TunableParam",
    "AutotuneConfig",
    "TunableKernel",
    "with_autotune",
    "ReductionAggrKernel",
    "GATv2AggrKernel",
    "GraphTransformerAggrKernel",
    "reduction_aggr",
    "gatv2_aggr",
    "graph_transformer_aggr",
    "spmm_aggr",
    "csr_SPMM_normalized",
    "gt_source_grads_ready",
    "source_rows_arriving",
]
