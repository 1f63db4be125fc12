"""Sweep harness on the GPU: one small cell per op family, the library against the torch comparator."""

import pytest
import torch

from turbo_gnn_b200 import sweep

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("conv,workload,shrink,hidden,heads,mode,precision,tol", [
    ("gatv2", "cfg1", 0.02, 32, 2, "directed", "none", 1e-4),
    ("gt", "cfg1", 0.02, 64, 4, "undirected", "none", 1e-4),
    ("sum", "cfg0", 0.2, 64, 1, "undirected_directed_kernel", "none", 1e-3),
    ("max", "cfg0", 0.2, 64, 1, "directed", "none", 0.0),
    ("spmm", "cfg3", 2 ** -10, 128, 1, "directed", "bf16", 0.5),
])
def test_one_cell(conv, workload, shrink, hidden, heads, mode, precision, tol):
    row = sweep.measure(conv, workload, precision, mode, hidden, heads, shrink=shrink, warmup=1, iters=2)
    assert row.fwd_ms > 0 and row.bwd_ms is not None and row.ref_fwd_ms > 0
    assert row.max_abs_diff <= tol, row
    assert row.speedup > 0
    assert sweep.format_table([row]).count("\n") == 2
