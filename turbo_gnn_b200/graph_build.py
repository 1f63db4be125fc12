"""Graph construction on the GPU: COO -> CSR, transposed CSR and light / heavy bucketing.

The reference builds its graph object with torch ops (``turbo_gnn/graph.py:39-67``: argsort of
``row * N + col``, ``bincount``, ``cumsum``; ``graph.py:11-36``: ``torch.quantile`` of the degrees
and two ``nonzero`` calls).  The functions here return the same arrays, bit for bit, from the
library's own radix sort (``csrc/graph_build.cuh``); ``AdjacencyForwardBackwardWithNodeBuckets``
uses them whenever the edge list lives on a CUDA device.  There is no CPU path in this module.
"""

from __future__ import annotations

import torch

from . import _abi

_MAX_ITEMS = (1 << 31) - 1


def _scratch(num_items: int, device: torch.device) -> tuple[torch.Tensor, int]:
    need = _abi.graph_workspace_bytes(num_items)
    return torch.empty(need, dtype=torch.uint8, device=device), need


def _signed(t: torch.Tensor) -> torch.Tensor:
    if t.dtype == torch.uint32:
        return t.view(torch.int32)
    if t.dtype == torch.uint64:
        return t.view(torch.int64)
    return t


def coo_to_csr(row_ids: torch.Tensor, col_ids: torch.Tensor, num_nodes: int,
               index_dtype: torch.dtype = torch.int64, want_order: bool = False):
    """``(indptr [N+1], indices [E], order or None)``: CSR keyed on ``row_ids``, entries ordered by
    (row, column).  ``order[k]`` is the position in the input of CSR entry ``k`` (int32).

    Raises ``RuntimeError`` when an id lies outside ``[0, num_nodes)``.
    """
    if not row_ids.is_cuda or not col_ids.is_cuda:
        raise RuntimeError("coo_to_csr needs CUDA tensors; the torch path of graph.py covers the host")
    if row_ids.dtype != col_ids.dtype or row_ids.shape != col_ids.shape or row_ids.dim() != 1:
        raise RuntimeError("row_ids and col_ids must be 1-D tensors of one dtype and length")
    num_edges = row_ids.numel()
    if num_edges > _MAX_ITEMS or num_nodes > _MAX_ITEMS:
        raise RuntimeError("the GPU graph builder takes fewer than 2^31 edges and nodes")
    rows, cols = _signed(row_ids).contiguous(), _signed(col_ids).contiguous()
    out_dt = _signed(torch.empty(0, dtype=index_dtype)).dtype
    dev = rows.device
    indptr = torch.empty(num_nodes + 1, dtype=out_dt, device=dev)
    indices = torch.empty(num_edges, dtype=out_dt, device=dev)
    order = torch.empty(num_edges, dtype=torch.int32, device=dev) if want_order else None
    bad = torch.zeros(1, dtype=torch.int32, device=dev)
    ws, ws_bytes = _scratch(num_edges, dev)
    args = _abi.CooToCsrArgs(
        exec=_abi.exec_of(rows),
        row_ids=_abi.ptr(rows),
        col_ids=_abi.ptr(cols),
        itype_in=_abi.itype_code(rows.dtype),
        itype_out=_abi.itype_code(out_dt),
        num_edges=num_edges,
        num_nodes=num_nodes,
        indptr=indptr.data_ptr(),
        indices=_abi.ptr(indices),
        edge_order=_abi.ptr(order),
        bad_ids=bad.data_ptr(),
        workspace=ws.data_ptr(),
        workspace_bytes=ws_bytes,
    )
    _abi.call("tgnn_coo_to_csr", args)
    if int(bad.item()) != 0:
        raise RuntimeError(f"edge list holds node ids outside [0, {num_nodes})")
    if index_dtype != out_dt:  # unsigned index types share the bits of their signed twin
        indptr, indices = indptr.view(index_dtype), indices.view(index_dtype)
    return indptr, indices, order


def quantile_cut(indptr: torch.Tensor, quantile: float) -> tuple[float, int]:
    """``(cut, max_degree)``: the value ``torch.quantile(degrees.float(), quantile)`` returns
    (linear interpolation between the two neighbouring order statistics, computed with the same
    float32 operations), or ``max_degree + 1`` for ``quantile == -1``.
    """
    ptr = _signed(indptr)
    n = ptr.numel() - 1
    if n <= 0:
        raise RuntimeError("quantile of an empty graph")
    dev = ptr.device
    if quantile == -1:
        k_lo = k_hi = n - 1
        weight = None
    else:
        if not 0.0 <= quantile <= 1.0:
            raise RuntimeError("quantile() q values must be in the range [0, 1]")
        rank = torch.tensor(quantile, dtype=torch.float32) * (n - 1)
        k_lo = int(rank.floor().item())
        k_hi = int(rank.ceil().item())
        weight = rank - rank.floor()
    out = torch.empty(3, dtype=torch.int64, device=dev)
    ws, ws_bytes = _scratch(n, dev)
    args = _abi.DegreeOrderStatsArgs(exec=_abi.exec_of(ptr), indptr=ptr.data_ptr(), itype=_abi.itype_code(ptr.dtype),
                                     num_rows=n, k_lo=k_lo, k_hi=k_hi, out=out.data_ptr(), workspace=ws.data_ptr(),
                                     workspace_bytes=ws_bytes)
    _abi.call("tgnn_degree_order_stats", args)
    lo, hi, top = (int(v) for v in out.tolist())
    if weight is None:
        return float(top + 1), top
    below = torch.tensor(float(lo), dtype=torch.float32, device=dev)
    above = torch.tensor(float(hi), dtype=torch.float32, device=dev)
    cut = torch.lerp(below, above, weight.to(dev)).item()
    return cut, top


def partition_rows(indptr: torch.Tensor, cut: float, index_dtype: torch.dtype | None = None):
    """``(light, heavy)``: ascending ids of the rows with ``float(degree) < cut`` / ``>= cut``."""
    ptr = _signed(indptr)
    n = ptr.numel() - 1
    dev = ptr.device
    rows = torch.empty(n, dtype=ptr.dtype, device=dev)
    num_light = torch.empty(1, dtype=torch.int64, device=dev)
    ws, ws_bytes = _scratch(n, dev)
    args = _abi.PartitionRowsArgs(exec=_abi.exec_of(ptr), indptr=ptr.data_ptr(), itype=_abi.itype_code(ptr.dtype),
                                  cut=float(cut), num_rows=n, rows_out=rows.data_ptr(),
                                  num_light=num_light.data_ptr(), workspace=ws.data_ptr(), workspace_bytes=ws_bytes)
    _abi.call("tgnn_partition_rows", args)
    k = int(num_light.item())
    light, heavy = rows[:k], rows[k:]
    if index_dtype is not None and index_dtype != rows.dtype:
        if _signed(torch.empty(0, dtype=index_dtype)).dtype == rows.dtype:
            light, heavy = light.view(index_dtype), heavy.view(index_dtype)
        else:
            light, heavy = light.to(index_dtype), heavy.to(index_dtype)
    return light, heavy


def bucket_rows(indptr: torch.Tensor, quantile: float, index_dtype: torch.dtype | None = None):
    """``(light, heavy, max_degree)`` of one CSR direction at a degree quantile."""
    cut, top = quantile_cut(indptr, quantile)
    light, heavy = partition_rows(indptr, cut, index_dtype)
    return light, heavy, top
