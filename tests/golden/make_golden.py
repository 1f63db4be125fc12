"""Regenerates tests/golden/*.pt from the reference project itself.

Run where a checkout of the reference project is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's OWN code -- ``turbo_gnn/graph.py`` (CSR construction, quantile
bucketing, repartition) and the pure-PyTorch scatter classes of
``src/backends/torch_native_backend/conv.py`` that the reference's tests use as their oracle --
runs them on small seeded inputs and stores inputs and outputs.  Third-party packages the
reference imports at module level but that these classes never call (torch_geometric, dgl, the
compiled ``turbo_gnn._C``) are replaced by empty stand-ins so that the import succeeds.  The
fixtures pin ``oracle/scatter_oracle.py`` and ``turbo_gnn_b200/graph.py``; the tests only read the
``.pt`` files, never the reference tree.
"""

from __future__ import annotations

import importlib.abc
import importlib.machinery
import os
import sys
from unittest.mock import MagicMock

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


class _StandIn(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    roots = ("torch_geometric", "dgl", "ogb", "torch_scatter", "torch_sparse", "cugraph", "pylibcugraphops",
             "comet_ml")

    def find_spec(self, name, path, target=None):
        if name.split(".")[0] in self.roots:
            return importlib.machinery.ModuleSpec(name, self, is_package=True)
        return None

    def create_module(self, spec):
        m = MagicMock()
        m.__name__, m.__path__, m.__spec__ = spec.name, [], spec
        return m

    def exec_module(self, module):
        pass


def _edges(n, e, seed, self_loops=False, symmetric=False):
    g = torch.Generator().manual_seed(seed)
    ei = torch.stack([torch.randint(0, n, (e,), generator=g), torch.randint(0, n, (e,), generator=g)])
    if symmetric:
        ei = torch.cat([ei, ei.flip(0)], 1)
    if self_loops:
        ei = torch.cat([ei, torch.arange(n).repeat(2, 1)], 1)
    key = torch.unique(ei[0] * n + ei[1])
    return torch.stack([key // n, key % n])


def main(ref_root: str) -> None:
    sys.meta_path.insert(0, _StandIn())
    sys.modules["turbo_gnn._C"] = MagicMock()
    sys.path.insert(0, ref_root)
    import src.backends.torch_native_backend.conv as conv  # noqa: E402  (the reference's oracle)
    from turbo_gnn.graph import AdjacencyForwardBackwardWithNodeBuckets as RefGraph  # noqa: E402

    torch.manual_seed(0)

    # ---- graph construction -------------------------------------------------------------
    graphs = []
    cases = [
        dict(n=50, e=400, seed=1, quantile=0.9, index_dtype=None, is_directed=None),
        dict(n=200, e=3000, seed=2, quantile=0.99, index_dtype=torch.int32, is_directed=None),
        dict(n=64, e=500, seed=3, quantile=-1, index_dtype=torch.int32, is_directed=None),
        dict(n=120, e=900, seed=4, quantile=0.95, index_dtype=torch.int64, is_directed=True),
        dict(n=80, e=600, seed=5, quantile=0.9, index_dtype=torch.int32, is_directed=None, symmetric=True),
        dict(n=80, e=600, seed=6, quantile=0.9, index_dtype=torch.int32, is_directed=False, symmetric=True),
    ]
    fields = ("forward_indptr", "forward_indices", "backward_indptr", "backward_indices", "forward_light_nodes",
              "forward_heavy_nodes", "backward_light_nodes", "backward_heavy_nodes")
    for c in cases:
        ei = _edges(c["n"], c["e"], c["seed"], self_loops=True, symmetric=c.get("symmetric", False))
        g = RefGraph.from_edge_list(ei, c["n"], quantile=c["quantile"], index_dtype=c["index_dtype"],
                                    is_directed=c["is_directed"])
        rec = {"case": {k: (str(v) if isinstance(v, torch.dtype) else v) for k, v in c.items()}, "edge_index": ei,
               "max_degree": g.max_degree, "is_directed": g.is_directed,
               "aliased": g.backward_indptr.data_ptr() == g.forward_indptr.data_ptr()}
        rec.update({f: getattr(g, f).clone() for f in fields})
        r = g.repartition(forward_huge_degree_threshold_quantile=0.5)
        rec["repart_fwd_light"] = r.forward_light_nodes.clone()
        rec["repart_fwd_heavy"] = r.forward_heavy_nodes.clone()
        rec["repart_bwd_light"] = r.backward_light_nodes.clone()
        g2 = RefGraph.from_csr(g.forward_indptr, g.forward_indices, g.backward_indptr, g.backward_indices,
                               quantile=0.75, index_dtype=c["index_dtype"], is_directed=c["is_directed"])
        rec["from_csr_fwd_heavy"] = g2.forward_heavy_nodes.clone()
        rec["from_csr_bwd_heavy"] = g2.backward_heavy_nodes.clone()
        graphs.append(rec)
    torch.save(graphs, os.path.join(HERE, "graph_cases.pt"))

    # ---- aggregation math -------------------------------------------------------------------
    agg = []
    for n, e, seed, f in ((40, 300, 11, 8), (100, 1200, 12, 32)):
        ei = _edges(n, e, seed)
        x = torch.randn(n, f)
        rec = {"n": n, "edge_index": ei, "x": x}
        for red in ("min", "max", "sum", "mean"):
            rec[red] = conv._ScatterSimpleAggOnly(red)(x, (ei, None, n)).clone()
        agg.append(rec)
    torch.save(agg, os.path.join(HERE, "reduce_cases.pt"))

    attn = []
    for n, e, seed, h, d in ((30, 200, 21, 2, 4), (90, 1000, 22, 4, 16)):
        ei = _edges(n, e, seed, self_loops=(seed == 22))
        left, right, val, up = (torch.randn(n, h, d) for _ in range(4))
        gat = conv._ScatterGATv2AggOnly(h, d, negative_slope=0.2)
        a = gat.attn.detach().clone().view(h, d)
        li, ri = left.clone().requires_grad_(), right.clone().requires_grad_()
        out = gat(li, ri, (ei, None, n))
        out.backward(up.reshape(n, -1))
        gt = conv._ScatterGTAggOnly(h, d)
        q, k, v = left.clone().requires_grad_(), right.clone().requires_grad_(), val.clone().requires_grad_()
        out2 = gt(q, k, v, (ei, None, n))
        out2.backward(up.reshape(n, -1))
        attn.append({
            "n": n, "h": h, "d": d, "edge_index": ei, "left": left, "right": right, "value": val, "upstream": up,
            "attn": a, "gat_out": out.detach().clone(), "gat_grad_left": li.grad.clone(),
            "gat_grad_right": ri.grad.clone(), "gat_grad_attn": gat.attn.grad.detach().clone().view(h, d),
            "gt_scale": gt.scale, "gt_out": out2.detach().clone(), "gt_dq": q.grad.clone(), "gt_dk": k.grad.clone(),
            "gt_dv": v.grad.clone(),
        })
    torch.save(attn, os.path.join(HERE, "attention_cases.pt"))

    sm = []
    for n, e, seed in ((25, 150, 31),):
        ei = _edges(n, e, seed)
        s1, s2 = torch.randn(ei.shape[1]), torch.randn(ei.shape[1], 3)
        sm.append({"n": n, "edge_index": ei, "s1": s1, "s2": s2,
                   "a1": conv._edge_softmax(s1, ei[1], n).clone(), "a2": conv._edge_softmax(s2, ei[1], n).clone()})
    torch.save(sm, os.path.join(HERE, "softmax_cases.pt"))
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".pt")))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py /path/to/reference")
    main(sys.argv[1])
