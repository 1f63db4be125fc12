"""Dual-CSR graph container with degree buckets.

Host-side mirror of the reference's ``turbo_gnn/graph.py`` (container
``graph.py:70-330``, COO->CSR ``graph.py:39-67``, quantile bucketing
``graph.py:11-36``): same class name, fields, constructors and results, so a
graph built here is element-for-element what the reference builds.  The
forward CSR has one row per DESTINATION node listing its sources; the backward
CSR is its transpose.  ``light``/``heavy`` row lists per direction drive the
first two tiers of the kernel schedule; the hub tier is carved out of the
heavy list later, by :mod:`turbo_gnn_b200._schedule`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

_UNSIGNED_TO_SIGNED = {torch.uint32: torch.int32, torch.uint64: torch.int64}


def _signed(t: torch.Tensor) -> torch.Tensor:
    """Reinterpret an unsigned index tensor as signed (no copy) so torch can do arithmetic on it."""
    target = _UNSIGNED_TO_SIGNED.get(t.dtype)
    return t if target is None else t.view(target)


def _row_degrees(indptr: torch.Tensor) -> torch.Tensor:
    p = _signed(indptr)
    return p[1:] - p[:-1]


def _bucket_nodes_by_degree(
    degree_counts: torch.Tensor,
    quantile: float,
    index_dtype: torch.dtype | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Split node ids into (light, heavy) at a degree quantile.

    The cut is ``torch.quantile`` of the fp32 degrees (linear interpolation);
    a node is heavy when its degree is >= the cut.  ``quantile == -1`` puts the
    cut above the maximum degree, i.e. every node is light.
    """
    if quantile == -1:
        cut = degree_counts.max().item() + 1
    else:
        cut = torch.quantile(degree_counts.float(), quantile).item()
    is_heavy = degree_counts >= cut
    heavy = is_heavy.nonzero(as_tuple=False).view(-1)
    light = (~is_heavy).nonzero(as_tuple=False).view(-1)
    if index_dtype is not None:
        light, heavy = light.to(index_dtype), heavy.to(index_dtype)
    return light, heavy


def build_csr_as_is(
    edge_index: torch.Tensor,
    edge_weight: Optional[torch.Tensor],
    num_nodes: int,
    do_transpose: bool = False,
):
    """COO -> CSR without deduplication.

    ``do_transpose=False`` keys rows on ``edge_index[0]``; ``True`` keys them on
    ``edge_index[1]`` (the forward CSR of the kernels).  Entries are ordered by
    (row, column).  Returns ``(row_ptr int64 [N+1], cols, weights or None, counts)``.
    """
    r, c = (1, 0) if do_transpose else (0, 1)
    row_of_edge, col_of_edge = edge_index[r], edge_index[c]
    order = torch.argsort(row_of_edge * num_nodes + col_of_edge)
    row_sorted = row_of_edge[order]
    cols = col_of_edge[order]
    weights = None if edge_weight is None else edge_weight[order]
    counts = torch.bincount(row_sorted, minlength=num_nodes)
    row_ptr = torch.zeros(num_nodes + 1, dtype=torch.long, device=row_sorted.device)
    torch.cumsum(counts, 0, out=row_ptr[1:])
    return row_ptr, cols, weights, counts


@dataclass
class AdjacencyForwardBackwardWithNodeBuckets:
    """Forward + backward CSR of one graph with light/heavy row lists per direction.

    All eight index tensors share one dtype (int32, int64, uint32 or uint64).
    When the two CSRs are element-wise equal (an undirected graph) the backward
    fields alias the forward tensors.
    """

    forward_indptr: torch.Tensor
    forward_indices: torch.Tensor
    backward_indptr: torch.Tensor
    backward_indices: torch.Tensor
    forward_light_nodes: torch.Tensor
    forward_heavy_nodes: torch.Tensor
    backward_light_nodes: torch.Tensor
    backward_heavy_nodes: torch.Tensor

    max_degree: int = -1
    _device: torch.device = torch.device("cpu")
    is_directed: bool | None = None  # None: decide by comparing the two CSRs

    _INDEX_FIELDS = (
        "forward_indptr",
        "forward_indices",
        "backward_indptr",
        "backward_indices",
        "forward_light_nodes",
        "forward_heavy_nodes",
        "backward_light_nodes",
        "backward_heavy_nodes",
    )

    def __post_init__(self):
        self._device = self.forward_indptr.device
        self.index_dtype = self.forward_indptr.dtype
        for name in self._INDEX_FIELDS[1:]:
            got = getattr(self, name).dtype
            assert got == self.index_dtype, f"{name} dtype {got} doesn't match forward_indptr dtype {self.index_dtype}"

        self.max_degree = _row_degrees(self.forward_indptr).max().item()
        assert self.max_degree != -1

        if self.is_directed is None:
            same = torch.equal(self.forward_indptr, self.backward_indptr) and torch.equal(
                self.forward_indices, self.backward_indices
            )
            self.is_directed = not same
        if not self.is_directed:
            self._alias_backward()

    def _alias_backward(self) -> None:
        self.backward_indptr = self.forward_indptr
        self.backward_indices = self.forward_indices

    @staticmethod
    def _to_signed_view(t: torch.Tensor) -> torch.Tensor:
        return _signed(t)

    @property
    def light_nodes(self) -> torch.Tensor:
        return self.forward_light_nodes

    @property
    def heavy_nodes(self) -> torch.Tensor:
        return self.forward_heavy_nodes

    @property
    def device(self) -> torch.device:
        return self._device

    @property
    def num_nodes(self) -> int:
        return self.forward_indptr.numel() - 1

    @property
    def num_edges(self) -> int:
        return self.forward_indices.numel()

    def repartition(self, **kwargs) -> "AdjacencyForwardBackwardWithNodeBuckets":
        """Same CSR tensors (shared, not copied), new light/heavy split.

        Keyword ``forward_huge_degree_threshold_quantile`` and/or
        ``backward_huge_degree_threshold_quantile`` re-bucket that direction;
        a direction whose keyword is absent keeps its lists.
        """
        lists = {
            "forward": (self.forward_light_nodes, self.forward_heavy_nodes),
            "backward": (self.backward_light_nodes, self.backward_heavy_nodes),
        }
        for side in ("forward", "backward"):
            q = kwargs.get(f"{side}_huge_degree_threshold_quantile")
            if q is not None:
                deg = _row_degrees(getattr(self, f"{side}_indptr"))
                lists[side] = _bucket_nodes_by_degree(deg, q, index_dtype=self.index_dtype)
        return AdjacencyForwardBackwardWithNodeBuckets(
            forward_indptr=self.forward_indptr,
            forward_indices=self.forward_indices,
            backward_indptr=self.backward_indptr,
            backward_indices=self.backward_indices,
            forward_light_nodes=lists["forward"][0],
            forward_heavy_nodes=lists["forward"][1],
            backward_light_nodes=lists["backward"][0],
            backward_heavy_nodes=lists["backward"][1],
            is_directed=self.is_directed,
        )

    def to(self, device) -> "AdjacencyForwardBackwardWithNodeBuckets":
        """Move every tensor in place (aliasing preserved) and return ``self``."""
        self.forward_indptr = self.forward_indptr.to(device)
        self.forward_indices = self.forward_indices.to(device)
        if self.is_directed:
            self.backward_indptr = self.backward_indptr.to(device)
            self.backward_indices = self.backward_indices.to(device)
        else:
            self._alias_backward()
        for name in self._INDEX_FIELDS[4:]:
            setattr(self, name, getattr(self, name).to(device))
        self._device = self.forward_indptr.device
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
        return self

    @classmethod
    def _assemble(cls, fwd, bwd, fwd_counts, bwd_counts, quantile, index_dtype, is_directed):
        """Shared tail of the constructors: dtype cast, aliasing, bucketing."""
        fwd_indptr, fwd_indices = fwd
        if index_dtype is not None:
            fwd_indptr, fwd_indices = fwd_indptr.to(index_dtype), fwd_indices.to(index_dtype)
        if is_directed is False:
            bwd_indptr, bwd_indices = fwd_indptr, fwd_indices
        else:
            bwd_indptr, bwd_indices = bwd
            if index_dtype is not None:
                bwd_indptr, bwd_indices = bwd_indptr.to(index_dtype), bwd_indices.to(index_dtype)
        idx_dt = index_dtype or fwd_indptr.dtype

        def bucket(indptr, counts):
            if indptr.is_cuda and indptr.numel() > 1:  # the library's own selection + partition kernels
                from . import graph_build

                light, heavy, _ = graph_build.bucket_rows(indptr, quantile, index_dtype=idx_dt)
                return light, heavy
            if counts is None:
                counts = _row_degrees(indptr)
            return _bucket_nodes_by_degree(counts, quantile, index_dtype=idx_dt)

        fwd_light, fwd_heavy = bucket(fwd_indptr, fwd_counts)
        if is_directed is False:
            bwd_light, bwd_heavy = fwd_light, fwd_heavy
        else:
            bwd_light, bwd_heavy = bucket(bwd_indptr, bwd_counts)
        return cls(
            forward_indptr=fwd_indptr,
            forward_indices=fwd_indices,
            backward_indptr=bwd_indptr,
            backward_indices=bwd_indices,
            forward_light_nodes=fwd_light,
            forward_heavy_nodes=fwd_heavy,
            backward_light_nodes=bwd_light,
            backward_heavy_nodes=bwd_heavy,
            is_directed=is_directed,
        )

    @classmethod
    def from_edge_list(
        cls,
        edge_index: torch.Tensor,
        num_nodes: int,
        quantile: float = 0.99,
        index_dtype: torch.dtype | None = None,
        is_directed: bool | None = None,
    ) -> "AdjacencyForwardBackwardWithNodeBuckets":
        """Build both CSRs from a COO ``edge_index`` of shape [2, E] (row 0 = source, row 1 = destination).

        ``is_directed=False`` skips the backward CSR and aliases it to the forward one.  An edge
        list on a CUDA device is sorted and bucketed by the library's own kernels
        (:mod:`turbo_gnn_b200.graph_build`), a host edge list by the torch ops below; the arrays
        are the same either way.
        """
        if edge_index.is_cuda:
            from . import graph_build

            out_dt = index_dtype or torch.int64
            src, dst = edge_index[0], edge_index[1]

            def csr(rows, cols):
                ptr, idx, _ = graph_build.coo_to_csr(rows, cols, num_nodes, out_dt)
                if index_dtype is None and idx.dtype != edge_index.dtype:
                    idx = idx.to(edge_index.dtype)  # the torch path keeps the edge list's dtype here
                return ptr, idx

            fwd = csr(dst, src)
            bwd = csr(src, dst) if is_directed is not False else None
            return cls._assemble(fwd, bwd, None, None, quantile, index_dtype, is_directed)
        f_ptr, f_idx, _, f_counts = build_csr_as_is(edge_index, None, num_nodes, do_transpose=True)
        bwd, b_counts = None, None
        if is_directed is not False:
            b_ptr, b_idx, _, b_counts = build_csr_as_is(edge_index, None, num_nodes, do_transpose=False)
            bwd = (b_ptr, b_idx)
        return cls._assemble((f_ptr, f_idx), bwd, f_counts, b_counts, quantile, index_dtype, is_directed)

    @classmethod
    def from_csr(
        cls,
        fwd_indptr: torch.Tensor,
        fwd_indices: torch.Tensor,
        bwd_indptr: torch.Tensor,
        bwd_indices: torch.Tensor,
        quantile: float = 0.99,
        index_dtype: torch.dtype | None = None,
        is_directed: bool | None = None,
    ) -> "AdjacencyForwardBackwardWithNodeBuckets":
        """Wrap caller-built forward and backward CSR arrays (no transposition is done here)."""
        return cls._assemble(
            (fwd_indptr, fwd_indices), (bwd_indptr, bwd_indices), None, None, quantile, index_dtype, is_directed
        )

    @classmethod
    def from_dgl(
        cls,
        dgl_graph,
        quantile: float = 0.99,
        index_dtype: torch.dtype | None = None,
        is_directed: bool | None = None,
    ) -> "AdjacencyForwardBackwardWithNodeBuckets":
        """Build from a DGL graph object (DGL itself is not required by this package)."""
        src, dst = dgl_graph.edges()
        return cls.from_edge_list(
            torch.stack([src, dst], dim=0),
            dgl_graph.num_nodes(),
            quantile=quantile,
            index_dtype=index_dtype,
            is_directed=is_directed,
        )
