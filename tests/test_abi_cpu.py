"""The C-ABI library: loads without a GPU, exports every declared symbol, and the ctypes mirror
of each struct has the size and field offsets the C compiler gives it."""

import ctypes
import os
import re
import shutil
import subprocess

import pytest

from turbo_gnn_b200 import _abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "tgnn_abi.h")

STRUCTS = {
    "tgnn_exec": _abi.Exec,
    "tgnn_csr": _abi.Csr,
    "tgnn_schedule": _abi.Schedule,
    "tgnn_mat": _abi.Mat,
    "tgnn_segment_reduce_args": _abi.SegmentReduceArgs,
    "tgnn_segment_reduce_bwd_args": _abi.SegmentReduceBwdArgs,
    "tgnn_degree_norm_args": _abi.DegreeNormArgs,
    "tgnn_spmm_args": _abi.SpmmArgs,
    "tgnn_head_dot_args": _abi.HeadDotArgs,
    "tgnn_gatv2_fwd_args": _abi.Gatv2FwdArgs,
    "tgnn_gatv2_bwd_dst_args": _abi.Gatv2BwdDstArgs,
    "tgnn_gatv2_bwd_src_args": _abi.Gatv2BwdSrcArgs,
    "tgnn_gt_fwd_args": _abi.GtFwdArgs,
    "tgnn_gt_bwd_dst_args": _abi.GtBwdDstArgs,
    "tgnn_gt_bwd_src_args": _abi.GtBwdSrcArgs,
    "tgnn_gt_bwd_dk_args": _abi.GtBwdDkArgs,
    "tgnn_coo_to_csr_args": _abi.CooToCsrArgs,
    "tgnn_degree_order_stats_args": _abi.DegreeOrderStatsArgs,
    "tgnn_partition_rows_args": _abi.PartitionRowsArgs,
}


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tgnn_[a-z0-9_]+)\s*\(", text)))


def test_library_loads_and_reports_version():
    lib = _abi.load_library()
    assert lib.tgnn_abi_version() == _abi.ABI_VERSION


def test_every_declared_symbol_is_exported_and_bound():
    lib = _abi.load_library()
    declared = _declared_functions()
    assert len(declared) >= 14
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but missing from the library"
        assert name in _abi.ENTRY_POINTS, f"{name} has no ctypes binding"
    assert sorted(_abi.ENTRY_POINTS) == declared


def test_workspace_query_without_gpu():
    assert _abi.workspace_bytes(_abi.OP_GT_FWD, __import__("torch").float32, __import__("torch").int32, 0, 256) == 0
    import torch

    one = _abi.workspace_bytes(_abi.OP_GT_FWD, torch.float32, torch.int32, 1, 256)
    ten = _abi.workspace_bytes(_abi.OP_GT_FWD, torch.float32, torch.int32, 10, 256)
    assert one > 0 and ten == 10 * one
    # min/max keeps a value and an index per feature: int64 indices need more than int32
    a = _abi.workspace_bytes(_abi.OP_REDUCE_MINMAX, torch.float32, torch.int32, 4, 128)
    b = _abi.workspace_bytes(_abi.OP_REDUCE_MINMAX, torch.float32, torch.int64, 4, 128)
    assert b > a > 0


def test_graph_workspace_query_without_gpu():
    small, large = _abi.graph_workspace_bytes(1000), _abi.graph_workspace_bytes(1_000_000)
    assert small > 0 and large - small >= 24 * (1_000_000 - 1000) - 4096  # two key and two payload buffers


def test_invalid_call_returns_status_and_message_not_a_crash():
    args = _abi.SegmentReduceArgs()  # all zero: null pointers, but reduce=0 and device 0
    args.reduce = 99
    with pytest.raises(RuntimeError, match="reduce must be"):
        _abi.call("tgnn_segment_reduce_forward", args)
    assert "reduce must be" in _abi.last_error()


@pytest.mark.skipif(shutil.which("gcc") is None, reason="gcc not available")
def test_struct_layout_matches_the_c_compiler(tmp_path):
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void) {"]
    for cname, cls in STRUCTS.items():
        lines.append(f'printf("{cname} size %zu\\n", sizeof({cname}));')
        for field, _ in cls._fields_:
            lines.append(f'printf("{cname} {field} %zu\\n", offsetof({cname}, {field}));')
    lines += ["return 0; }"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    seen = 0
    for line in out.splitlines():
        cname, field, value = line.split()
        cls = STRUCTS[cname]
        if field == "size":
            assert ctypes.sizeof(cls) == int(value), cname
        else:
            assert getattr(cls, field).offset == int(value), f"{cname}.{field}"
        seen += 1
    assert seen > 100
