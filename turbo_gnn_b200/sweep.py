"""Sweep harness: forward / backward timings of the aggregation ops over workloads, precisions and
graph modes, beside a plain-torch scatter comparator on the same GPU.

    python -m turbo_gnn_b200.sweep --conv_type gatv2 --workloads cfg1 --precisions none bf16 \\
        --graph_modes directed undirected --hidden 64 --heads 8 --out sweep.jsonl

The reference drives the same kind of table from ``scripts/kernel_launch_comparison.py`` (aggr-mode
forward/backward timings ``:191-244``, precision and graph-mode sweeps ``:95-118``) across its
backend registry; here the target backend is this library and the comparator is the scatter
formulation in torch (``index_add_`` / ``scatter_reduce_`` / edge softmax), which runs on any GPU
and needs no extra package.  Each row also records the largest deviation between the two.  The
module is a regression tracker, not part of the timed benchmark.
"""

from __future__ import annotations

import argparse
import json
import sys
from dataclasses import asdict, dataclass

import torch

CONV_TYPES = ("min", "max", "sum", "mean", "spmm", "gatv2", "gt")
PRECISIONS = {"none": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}
GRAPH_MODES = ("directed", "undirected_directed_kernel", "undirected")


@dataclass
class SweepRow:
    conv_type: str
    workload: str
    precision: str
    graph_mode: str
    hidden: int
    heads: int
    nodes: int
    edges: int
    fwd_ms: float
    bwd_ms: float | None
    ref_fwd_ms: float | None
    ref_bwd_ms: float | None
    max_abs_diff: float | None

    @property
    def speedup(self) -> float | None:
        if self.ref_fwd_ms is None:
            return None
        ours = self.fwd_ms + (self.bwd_ms or 0.0)
        return (self.ref_fwd_ms + (self.ref_bwd_ms or 0.0)) / ours


# ---- comparator: scatter formulation in plain torch ---------------------------------------------


def _edge_softmax(score, dst, n):
    top = torch.full((n,) + score.shape[1:], float("-inf"), dtype=score.dtype, device=score.device)
    idx = dst.view(-1, *([1] * (score.dim() - 1))).expand_as(score)
    top.scatter_reduce_(0, idx, score, reduce="amax", include_self=True)
    e = torch.exp(score - top[dst])
    return e / torch.zeros_like(top).scatter_add_(0, idx, e)[dst]


def scatter_reference(conv_type: str, ei: torch.Tensor, n: int, tensors: dict, params: dict):
    src, dst = ei[0], ei[1]
    if conv_type in ("sum", "mean", "spmm", "min", "max"):
        x = tensors["x"]
        msg = x[src]
        idx = dst.unsqueeze(1).expand_as(msg)
        if conv_type in ("sum", "spmm"):
            return torch.zeros_like(x).index_add_(0, dst, msg)
        if conv_type == "mean":
            deg = torch.bincount(dst, minlength=n).clamp_(min=1).to(x.dtype).unsqueeze(1)
            return torch.zeros_like(x).index_add_(0, dst, msg) / deg
        out = torch.zeros_like(x).scatter_reduce_(0, idx, msg, reduce="amin" if conv_type == "min" else "amax",
                                                  include_self=False)
        return out
    if conv_type == "gatv2":
        l, r, a = tensors["x"], tensors["x_neighbors"], tensors["attention_weights"]
        z = torch.nn.functional.leaky_relu(l[dst] + r[src], params.get("negative_slope", 0.2))
        alpha = _edge_softmax((z * a.unsqueeze(0)).sum(-1), dst, n)
        return torch.zeros_like(l).index_add_(0, dst, r[src] * alpha.unsqueeze(-1))
    q, k, v = tensors["Q"], tensors["K"], tensors["V"]
    alpha = _edge_softmax((q[src] * k[dst]).sum(-1) * params["scale"], dst, n)
    return torch.zeros_like(v).index_add_(0, dst, v[src] * alpha.unsqueeze(-1))


# ---- target: this library -----------------------------------------------------------------------------


def library_call(conv_type: str, graph, tensors: dict, params: dict):
    import turbo_gnn_b200 as tg

    if conv_type in ("min", "max", "sum", "mean"):
        return tg.reduction_aggr(graph, tensors["x"], warps_per_block=4, reduce=conv_type)
    if conv_type == "spmm":
        return tg.spmm_aggr(tensors["x"], graph.forward_indptr, graph.forward_indices, "none", -1, tensors["x"].shape[1])
    if conv_type == "gatv2":
        return tg.gatv2_aggr(graph, tensors["x"], tensors["x_neighbors"], tensors["attention_weights"],
                             params.get("negative_slope", 0.2))
    return tg.graph_transformer_aggr(graph, None, tensors["Q"], tensors["K"], tensors["V"], params["scale"],
                                     forward_light_warps=1)


# ---- one cell of the table --------------------------------------------------------------------------------


def _time(fn, warmup: int, iters: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def make_inputs(conv_type: str, n: int, hidden: int, heads: int, dtype: torch.dtype, device, seed: int = 0):
    g = torch.Generator(device=device).manual_seed(seed)

    def randn(*shape, std=1.0):
        return (torch.randn(*shape, generator=g, device=device) * std).to(dtype)

    if conv_type == "gatv2":
        return {"x": randn(n, heads, hidden), "x_neighbors": randn(n, heads, hidden),
                "attention_weights": randn(heads, hidden, std=0.1)}, {"negative_slope": 0.2}
    if conv_type == "gt":
        return {k: randn(n, heads, hidden) for k in ("Q", "K", "V")}, {"scale": hidden ** -0.5}
    return {"x": randn(n, hidden * heads)}, {}


def measure(conv_type: str, workload: str, precision: str, graph_mode: str, hidden: int, heads: int,
            shrink: float = 1.0, warmup: int = 3, iters: int = 10, with_reference: bool = True,
            reference_edge_limit: int = 8_000_000, device="cuda") -> SweepRow:
    from . import synthetic
    from .graph import AdjacencyForwardBackwardWithNodeBuckets as Graph

    wl = synthetic.make_workload(int(workload.replace("cfg", "")), device=device, shrink=shrink)
    ei, n = wl.edge_index, wl.num_nodes
    if graph_mode != "directed":
        ei = synthetic.dedup_edges(synthetic.symmetrise(ei), n)
    directed = graph_mode != "undirected"  # "undirected": one CSR serves both directions
    graph = Graph.from_edge_list(ei, n, quantile=0.99, index_dtype=torch.int32, is_directed=directed)
    dtype = PRECISIONS[precision]
    tensors, params = make_inputs(conv_type, n, hidden, heads, dtype, device)
    leaves = list(tensors.values())
    for t in leaves:
        t.requires_grad_(True)
    out = library_call(conv_type, graph, tensors, params)
    upstream = torch.randn_like(out)

    fwd = _time(lambda: library_call(conv_type, graph, tensors, params), warmup, iters)

    def fwd_bwd():
        o = library_call(conv_type, graph, tensors, params)
        torch.autograd.grad(o, leaves, upstream)

    bwd = max(_time(fwd_bwd, warmup, iters) - fwd, 0.0)

    ref_fwd = ref_bwd = diff = None
    if with_reference and ei.shape[1] <= reference_edge_limit:  # the scatter form materialises [E, F] messages
        long_ei = ei.long()
        with torch.no_grad():  # deviation against the comparator evaluated in fp32
            ref_out = scatter_reference(conv_type, long_ei, n, {k: v.float() for k, v in tensors.items()}, params)
            diff = float((ref_out - out.float()).abs().max())
            del ref_out
        ref_fwd = _time(lambda: scatter_reference(conv_type, long_ei, n, tensors, params), 1, max(iters // 3, 1))

        def ref_fwd_bwd():
            o = scatter_reference(conv_type, long_ei, n, tensors, params)
            torch.autograd.grad(o, leaves, upstream)

        ref_bwd = max(_time(ref_fwd_bwd, 1, max(iters // 3, 1)) - ref_fwd, 0.0)
    return SweepRow(conv_type, workload, precision, graph_mode, hidden, heads, n, int(ei.shape[1]), fwd, bwd, ref_fwd,
                    ref_bwd, diff)


# ---- table ------------------------------------------------------------------------------------------------------


def format_table(rows: list[SweepRow]) -> str:
    head = ("| conv | workload | precision | graph mode | heads x hidden | nodes | edges | fwd ms | bwd ms | "
            "torch fwd ms | torch bwd ms | speed-up | max abs diff |")
    lines = [head, "|" + "---|" * 13]

    def f(v, spec=".3f"):
        return "-" if v is None else format(v, spec)

    for r in rows:
        lines.append(f"| {r.conv_type} | {r.workload} | {r.precision} | {r.graph_mode} | {r.heads} x {r.hidden} | "
                     f"{r.nodes} | {r.edges} | {f(r.fwd_ms)} | {f(r.bwd_ms)} | {f(r.ref_fwd_ms)} | {f(r.ref_bwd_ms)} | "
                     f"{f(r.speedup, '.1f')} | {f(r.max_abs_diff, '.2e')} |")
    return "\n".join(lines)


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Aggregation-op sweep: this library beside a torch scatter comparator")
    p.add_argument("--conv_type", required=True, choices=CONV_TYPES)
    p.add_argument("--workloads", nargs="+", default=["cfg1"], help="graphs of the benchmark generator (cfg0..cfg4)")
    p.add_argument("--precisions", nargs="+", default=["none"], choices=sorted(PRECISIONS))
    p.add_argument("--graph_modes", nargs="+", default=["directed"], choices=GRAPH_MODES)
    p.add_argument("--hidden", nargs="+", type=int, default=[64])
    p.add_argument("--heads", nargs="+", type=int, default=[1])
    p.add_argument("--shrink", type=float, default=1.0)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--no-reference", action="store_true", help="skip the torch scatter comparator")
    p.add_argument("--device", type=int, default=0)
    p.add_argument("--out", default=None, help="append one JSON line per row to this file")
    return p.parse_args(argv)


def main(argv=None) -> int:
    args = parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("the sweep needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(args.device)
    rows = []
    for wl in args.workloads:
        for prec in args.precisions:
            for mode in args.graph_modes:
                for hidden in args.hidden:
                    for heads in args.heads:
                        row = measure(args.conv_type, wl, prec, mode, hidden, heads, args.shrink, args.warmup, args.iters,
                                      not args.no_reference, device=f"cuda:{args.device}")
                        rows.append(row)
                        if args.out:
                            with open(args.out, "a") as fh:
                                fh.write(json.dumps({**asdict(row), "speedup": row.speedup}) + "\n")
    print(format_table(rows))
    return 0


if __name__ == "__main__":
    sys.exit(main())
