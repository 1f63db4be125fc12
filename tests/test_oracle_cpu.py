"""Pins the CPU oracle: against outputs of the reference's own classes (tests/golden/*.pt) and
against the closed-form cases the reference's tests use (star graph, K3, isolated vertex,
3-node GATv2, 6-node graph transformer)."""

import ctypes
import os

import pytest
import torch

from oracle import scatter_oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _load(name):
    return torch.load(os.path.join(GOLDEN, name), weights_only=False)


def test_reduce_matches_reference_outputs():
    for rec in _load("reduce_cases.pt"):
        for red in ("min", "max", "sum", "mean"):
            got = O.segment_reduce(rec["x"], rec["edge_index"], rec["n"], red)
            assert torch.equal(got, rec[red]), red


def test_edge_softmax_matches_reference_outputs():
    for rec in _load("softmax_cases.pt"):
        assert torch.equal(O.edge_softmax(rec["s1"], rec["edge_index"][1], rec["n"]), rec["a1"])
        assert torch.equal(O.edge_softmax(rec["s2"], rec["edge_index"][1], rec["n"]), rec["a2"])


def test_attention_matches_reference_outputs_and_gradients():
    for rec in _load("attention_cases.pt"):
        n, ei, up = rec["n"], rec["edge_index"], rec["upstream"]
        left, right, a = (rec[k].clone().requires_grad_() for k in ("left", "right", "attn"))
        out = O.gatv2_aggregate(left, right, a, ei, n, 0.2)
        out.backward(up)
        assert torch.allclose(out.reshape(n, -1), rec["gat_out"], atol=1e-6, rtol=1e-6)
        assert torch.allclose(left.grad, rec["gat_grad_left"], atol=1e-6, rtol=1e-5)
        assert torch.allclose(right.grad, rec["gat_grad_right"], atol=1e-6, rtol=1e-5)
        assert torch.allclose(a.grad, rec["gat_grad_attn"], atol=1e-5, rtol=1e-5)
        q, k, v = (rec[name].clone().requires_grad_() for name in ("left", "right", "value"))
        out = O.gt_aggregate(q, k, v, ei, n, rec["gt_scale"])
        out.backward(up)
        assert torch.allclose(out.reshape(n, -1), rec["gt_out"], atol=1e-6, rtol=1e-6)
        for t, name in ((q, "gt_dq"), (k, "gt_dk"), (v, "gt_dv")):
            assert torch.allclose(t.grad, rec[name], atol=1e-6, rtol=1e-5), name


# ---- closed-form cases --------------------------------------------------------------------------


def test_star_graph_min_max_mean():
    # nodes 1..9 -> node 0, node i carries the value i in every feature
    n, f = 10, 16
    ei = torch.stack([torch.arange(1, n), torch.zeros(n - 1, dtype=torch.long)])
    x = torch.arange(n, dtype=torch.float32).unsqueeze(1).repeat(1, f)
    mn, mx = O.segment_reduce(x, ei, n, "min"), O.segment_reduce(x, ei, n, "max")
    want_min, want_max = torch.zeros(n, f), torch.zeros(n, f)
    want_min[0], want_max[0] = 1.0, n - 1.0
    assert torch.equal(mn, want_min) and torch.equal(mx, want_max)
    assert torch.allclose(O.segment_reduce(x, ei, n, "mean")[0], torch.full((f,), 5.0))
    assert torch.equal(O.segment_reduce(x, ei, n, "mean")[1:], torch.zeros(n - 1, f))


def test_complete_graph_on_three_nodes():
    n, f = 3, 16
    rows, cols = torch.meshgrid(torch.arange(n), torch.arange(n), indexing="ij")
    keep = rows != cols
    ei = torch.stack([rows[keep], cols[keep]])
    x = torch.arange(n, dtype=torch.float32).unsqueeze(1).repeat(1, f)
    want_min = torch.tensor([1.0, 0.0, 0.0]).unsqueeze(1).repeat(1, f)
    want_max = torch.tensor([2.0, 2.0, 1.0]).unsqueeze(1).repeat(1, f)
    assert torch.equal(O.segment_reduce(x, ei, n, "min"), want_min)
    assert torch.equal(O.segment_reduce(x, ei, n, "max"), want_max)


def test_isolated_vertex_gets_zero():
    ei = torch.tensor([[0, 1], [1, 0]])
    x = torch.arange(1, 4, dtype=torch.float32).unsqueeze(1).repeat(1, 16)
    want = torch.tensor([2.0, 1.0, 0.0]).unsqueeze(1).repeat(1, 16)
    for red in ("min", "max", "sum", "mean"):
        assert torch.equal(O.segment_reduce(x, ei, 3, red), want), red


def test_self_loop_only_graph_is_identity_for_mean():
    n = 7
    ei = torch.arange(n).repeat(2, 1)
    x = torch.randn(n, 5)
    assert torch.equal(O.segment_reduce(x, ei, n, "mean"), x)


def test_gatv2_three_node_closed_form():
    # edges 0->1 and 2->1, one head, attention vector of ones, identity projections
    x = torch.tensor([[1.0, 3.0], [-1.0, 0.0], [2.0, 1.0]])
    ei = torch.tensor([[0, 2], [1, 1]])
    feats = x.view(3, 1, 2)
    out = O.gatv2_aggregate(feats, feats, torch.ones(1, 2), ei, 3, 0.2).view(3, 2)
    e01 = torch.nn.functional.leaky_relu(x[0] + x[1], 0.2).sum()
    e21 = torch.nn.functional.leaky_relu(x[2] + x[1], 0.2).sum()
    z = torch.exp(e01) + torch.exp(e21)
    want = torch.zeros(3, 2)
    want[1] = torch.exp(e01) / z * x[0] + torch.exp(e21) / z * x[2]
    assert torch.allclose(out, want, atol=1e-6, rtol=1e-6)


def test_graph_transformer_six_node_closed_form():
    torch.manual_seed(3)
    n, h, d = 6, 4, 4
    edges = torch.tensor([(1, 0), (2, 0), (3, 0), (1, 4), (2, 5), (1, 5)])
    ei = edges.T.contiguous()
    q, k, v = (torch.randn(n, h, d, requires_grad=True) for _ in range(3))
    scale = d**-0.5
    out = O.gt_aggregate(q, k, v, ei, n, scale)
    want = torch.zeros(n, h, d)
    for i in range(n):
        inc = (ei[1] == i).nonzero().view(-1)
        if inc.numel() == 0:
            continue
        s = torch.stack([(q[ei[0, e]] * k[i]).sum(-1) * scale for e in inc])  # [deg, h]
        p = torch.exp(s) / torch.exp(s).sum(0)
        want[i] = torch.einsum("ehd,eh->hd", v[ei[0, inc]], p)
    assert torch.allclose(out, want, atol=1e-6)
    g1 = torch.autograd.grad((out**2).sum(), (q, k, v), retain_graph=True)
    g2 = torch.autograd.grad((want**2).sum(), (q, k, v))
    for a, b in zip(g1, g2):
        assert torch.allclose(a, b, atol=1e-5)


def test_spmm_norms_against_dense():
    torch.manual_seed(0)
    n = 12
    ei = torch.unique(torch.randint(0, n, (2, 60)), dim=1)
    x = torch.randn(n, 5, dtype=torch.float64)
    A = torch.zeros(n, n, dtype=torch.float64)
    A[ei[1], ei[0]] = 1.0  # row = destination
    din = A.sum(1).clamp(min=1)
    dout = A.sum(0).clamp(min=1)
    dense = {
        "none": A @ x,
        "right": (A / din[:, None]) @ x,
        "left": (A / dout[None, :]) @ x,
        "both": (A / din[:, None].sqrt() / dout[None, :].sqrt()) @ x,
    }
    for norm, want in dense.items():
        assert torch.allclose(O.spmm(x, ei, n, norm), want, atol=1e-12), norm


def test_argreduce_prefers_lowest_source_on_ties():
    ei = torch.tensor([[3, 1, 2], [0, 0, 0]])
    x = torch.tensor([[9.0], [5.0], [5.0], [5.0]])
    assert O.segment_argreduce(x, ei, 4, "min")[0, 0].item() == 1
    assert O.segment_argreduce(x, ei, 4, "max")[0, 0].item() == 1
    assert O.segment_argreduce(x, ei, 4, "min")[1, 0].item() == -1


# ---- the C restatement agrees with the torch restatement -----------------------------------------


def _c_lib():
    import __graft_entry__ as entry

    path = entry.build_oracle()
    if path is None:
        pytest.skip("gcc not available")
    return ctypes.CDLL(path)


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def test_c_oracle_matches_torch_oracle():
    lib = _c_lib()
    torch.manual_seed(5)
    n, h, d = 60, 2, 8
    ei = torch.unique(torch.randint(0, n, (2, 700)), dim=1)
    order = torch.argsort(ei[1] * n + ei[0])
    src, dst = ei[0][order].contiguous(), ei[1][order]
    indptr = torch.zeros(n + 1, dtype=torch.long)
    indptr[1:] = torch.cumsum(torch.bincount(dst, minlength=n), 0)
    x = torch.randn(n, h * d)
    for code, red in enumerate(("min", "max", "sum", "mean")):
        out = torch.empty(n, h * d)
        arg = torch.empty(n, h * d, dtype=torch.long)
        lib.ref_segment_reduce(_p(indptr), _p(src), ctypes.c_int64(n), _p(x), ctypes.c_int64(h * d),
                               ctypes.c_int(code), _p(out), _p(arg))
        want = O.segment_reduce(x, ei, n, red)
        if code < 2:
            assert torch.equal(out, want)
            assert torch.equal(arg, O.segment_argreduce(x, ei, n, red))
        else:
            assert torch.allclose(out, want, atol=1e-5, rtol=1e-5)
    l, r, v = torch.randn(n, h, d), torch.randn(n, h, d), torch.randn(n, h, d)
    a = torch.randn(h, d) * 0.3
    out, lse = torch.empty(n, h, d), torch.empty(n, h)
    lib.ref_gatv2_forward(_p(indptr), _p(src), ctypes.c_int64(n), _p(l), _p(r), _p(a), ctypes.c_int64(h),
                          ctypes.c_int64(d), ctypes.c_float(0.2), _p(out), _p(lse))
    assert torch.allclose(out, O.gatv2_aggregate(l, r, a, ei, n, 0.2), atol=1e-5, rtol=1e-5)
    lib.ref_gt_forward(_p(indptr), _p(src), ctypes.c_int64(n), _p(l), _p(r), _p(v), ctypes.c_int64(h),
                       ctypes.c_int64(d), ctypes.c_float(0.25), _p(out), _p(lse))
    assert torch.allclose(out, O.gt_aggregate(l, r, v, ei, n, 0.25), atol=1e-5, rtol=1e-5)
    score = (l[ei[0]] * r[ei[1]]).sum(-1) * 0.25
    want_lse = O.attention_lse(score, ei[1], n)
    finite = ~want_lse.isinf()
    assert torch.allclose(lse[finite], want_lse[finite], atol=1e-5, rtol=1e-5)
    assert torch.equal(lse.isinf(), want_lse.isinf())
