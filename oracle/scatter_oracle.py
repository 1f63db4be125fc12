"""CPU oracle: a restatement of the reference's pure-PyTorch scatter aggregations.

TEST INFRASTRUCTURE ONLY.  Nothing under ``turbo_gnn_b200/`` imports this file;
it is used by ``tests/``, by ``__graft_entry__.smoke()`` as the checker and by
``bench.py``'s CPU-baseline leg as the thing timed on the host.

What it follows (paths inside the reference project):
  * ``src/backends/torch_native_backend/conv.py:24-29``   scatter-add helper
  * ``src/backends/torch_native_backend/conv.py:32-68``   edge softmax
  * ``src/backends/torch_native_backend/conv.py:472-503`` min / max / sum / mean aggregation
  * ``src/backends/torch_native_backend/conv.py:506-529`` GATv2 aggregation
  * ``src/backends/torch_native_backend/conv.py:532-552`` graph-transformer aggregation
  * ``csrc/spmm/edge_norm_kernels.cu:26-60``              SpMM edge normalisation (none/right/left/both)
Gradients come from torch autograd through these functions, which is how the
reference's own tests obtain them (``tests/correctness/test_gatv2_correctness.py:189-190``).

Pinned by ``tests/golden/*.pt``: outputs of the reference's own classes, generated
in a container that has the reference tree by ``tests/golden/make_golden.py``, and by
the closed-form cases of the reference's tests restated in ``tests/test_oracle_cpu.py``.

Graph convention: ``edge_index[0]`` = source, ``edge_index[1]`` = destination;
results are indexed by destination.  All functions work in the dtype of their
inputs (pass float64 tensors for a ground-truth run).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def scatter_add_rows(values: torch.Tensor, index: torch.Tensor, num_rows: int) -> torch.Tensor:
    """out[index[e]] += values[e] for values of shape [E, ...]."""
    out = torch.zeros((num_rows,) + tuple(values.shape[1:]), dtype=values.dtype, device=values.device)
    shape = (-1,) + (1,) * (values.dim() - 1)
    out.scatter_add_(0, index.view(shape).expand_as(values), values)
    return out


def edge_softmax(scores: torch.Tensor, dst: torch.Tensor, num_nodes: int) -> torch.Tensor:
    """Softmax of edge scores ([E] or [E, H]) over the edges that share a destination."""
    squeeze = scores.dim() == 1
    s = scores.unsqueeze(1) if squeeze else scores
    idx = dst.unsqueeze(1).expand_as(s)
    top = torch.full((num_nodes, s.shape[1]), float("-inf"), dtype=s.dtype, device=s.device)
    top.scatter_reduce_(0, idx, s, reduce="amax", include_self=True)
    e = torch.exp(s - top[dst])
    denom = torch.zeros((num_nodes, s.shape[1]), dtype=s.dtype, device=s.device)
    denom.scatter_add_(0, idx, e)
    alpha = e / denom[dst].clamp(min=1e-16)
    return alpha.squeeze(1) if squeeze else alpha


def segment_reduce(x: torch.Tensor, edge_index: torch.Tensor, num_nodes: int, reduce: str) -> torch.Tensor:
    """min / max / sum / mean of source rows per destination; a node without in-edges gets zeros."""
    src, dst = edge_index[0], edge_index[1]
    msg = x[src]
    if reduce in ("min", "max"):
        fill = float("inf") if reduce == "min" else float("-inf")
        out = torch.full((num_nodes, x.shape[1]), fill, dtype=x.dtype, device=x.device)
        idx = dst.unsqueeze(1).expand(-1, x.shape[1])
        out.scatter_reduce_(0, idx, msg, reduce="amin" if reduce == "min" else "amax", include_self=False)
        return torch.where(out.isinf(), torch.zeros_like(out), out)
    if reduce == "sum":
        return scatter_add_rows(msg, dst, num_nodes)
    if reduce == "mean":
        total = scatter_add_rows(msg, dst, num_nodes)
        count = torch.zeros(num_nodes, 1, dtype=x.dtype, device=x.device)
        count.scatter_add_(0, dst.unsqueeze(1), torch.ones(dst.numel(), 1, dtype=x.dtype, device=x.device))
        return total / count.clamp(min=1)
    raise ValueError(f"Unknown reduce: {reduce}")


def segment_argreduce(x: torch.Tensor, edge_index: torch.Tensor, num_nodes: int, reduce: str) -> torch.Tensor:
    """Winner source id per (destination, feature) with ties to the LOWEST source id, -1 for no in-edge.

    The reference's kernel keeps the first strictly better value while walking a row in
    ascending column order (``csrc/reduction/reduction_aggr.cu:48-59``), which is this rule.
    Dense O(N * max_degree) loops: small graphs only.
    """
    src, dst = edge_index[0], edge_index[1]
    arg = torch.full((num_nodes, x.shape[1]), -1, dtype=torch.long)
    best = torch.full((num_nodes, x.shape[1]), float("inf") if reduce == "min" else float("-inf"), dtype=x.dtype)
    order = torch.argsort(src, stable=True)
    for e in order.tolist():
        u, v = int(src[e]), int(dst[e])
        better = x[u] < best[v] if reduce == "min" else x[u] > best[v]
        best[v] = torch.where(better, x[u], best[v])
        arg[v] = torch.where(better, torch.full_like(arg[v], u), arg[v])
    return arg


def spmm_edge_weights(edge_index: torch.Tensor, num_nodes: int, norm: str, dtype=torch.float32) -> torch.Tensor:
    """Per-edge weight of the normalised SpMM; degrees are clamped to >= 1."""
    src, dst = edge_index[0], edge_index[1]
    ones = torch.ones(src.numel(), dtype=dtype)
    in_deg = torch.zeros(num_nodes, dtype=dtype).scatter_add_(0, dst, ones).clamp(min=1)
    out_deg = torch.zeros(num_nodes, dtype=dtype).scatter_add_(0, src, ones).clamp(min=1)
    if norm == "none":
        return ones
    if norm == "right":
        return 1.0 / in_deg[dst]
    if norm == "left":
        return 1.0 / out_deg[src]
    if norm == "both":
        return 1.0 / torch.sqrt(out_deg[src] * in_deg[dst])
    raise ValueError(f"unknown norm '{norm}'")


def spmm(x: torch.Tensor, edge_index: torch.Tensor, num_nodes: int, norm: str = "none",
         edge_weight: torch.Tensor | None = None) -> torch.Tensor:
    """out[v] = sum over edges (u -> v) of weight * x[u]."""
    w = spmm_edge_weights(edge_index, num_nodes, norm, dtype=x.dtype)
    if edge_weight is not None:
        w = w * edge_weight.to(x.dtype)
    return scatter_add_rows(x[edge_index[0]] * w.unsqueeze(1), edge_index[1], num_nodes)


def gatv2_aggregate(x_left: torch.Tensor, x_right: torch.Tensor, attn: torch.Tensor, edge_index: torch.Tensor,
                    num_nodes: int, negative_slope: float = 0.2) -> torch.Tensor:
    """GATv2 aggregation of pre-projected features; x_left/x_right [N, H, D], attn [H, D]; returns [N, H, D]."""
    src, dst = edge_index[0], edge_index[1]
    z = F.leaky_relu(x_left[dst] + x_right[src], negative_slope=negative_slope)
    score = (z * attn.unsqueeze(0)).sum(-1)
    alpha = edge_softmax(score, dst, num_nodes)
    return scatter_add_rows(x_right[src] * alpha.unsqueeze(-1), dst, num_nodes)


def gt_aggregate(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, edge_index: torch.Tensor, num_nodes: int,
                 scale: float) -> torch.Tensor:
    """Graph-transformer aggregation: score = <Q[src], K[dst]> * scale; returns [N, H, D]."""
    src, dst = edge_index[0], edge_index[1]
    score = (q[src] * k[dst]).sum(-1) * scale
    alpha = edge_softmax(score, dst, num_nodes)
    return scatter_add_rows(v[src] * alpha.unsqueeze(-1), dst, num_nodes)


def attention_lse(score: torch.Tensor, dst: torch.Tensor, num_nodes: int) -> torch.Tensor:
    """log-sum-exp of edge scores per destination ([N, H]); -inf for a node without in-edges."""
    idx = dst.unsqueeze(1).expand_as(score)
    top = torch.full((num_nodes, score.shape[1]), float("-inf"), dtype=score.dtype)
    top.scatter_reduce_(0, idx, score, reduce="amax", include_self=True)
    safe_top = torch.where(top.isinf(), torch.zeros_like(top), top)
    denom = torch.zeros_like(top).scatter_add_(0, idx, torch.exp(score - safe_top[dst]))
    return torch.where(denom > 0, safe_top + torch.log(denom), torch.full_like(top, float("-inf")))


def two_layer_gatv2(x: torch.Tensor, w1: torch.Tensor, a1: torch.Tensor, w2: torch.Tensor, a2: torch.Tensor,
                    edge_index: torch.Tensor, num_nodes: int, negative_slope: float = 0.2) -> torch.Tensor:
    """Two GATv2 layers with an ELU between them.

    Each layer is the data flow of the reference's GATv2 layer without its output projection
    (``src/backends/torch_native_backend/conv.py``: one bias-free Linear whose output splits into
    the destination-side and source-side halves, then the edge-softmax aggregation).  ``w`` is the
    ``[2 * H * D, in]`` Linear weight and ``a`` the ``[H, D]`` attention vector of a layer.
    """
    h = x
    for layer, (w, a) in enumerate(((w1, a1), (w2, a2))):
        heads, d = a.shape
        left, right = (h @ w.t()).split(heads * d, -1)
        h = gatv2_aggregate(left.view(-1, heads, d), right.view(-1, heads, d), a, edge_index, num_nodes,
                            negative_slope).reshape(num_nodes, heads * d)
        if layer == 0:
            h = F.elu(h)
    return h
