"""CPU checks of the boundary: the C ABI library loads and exports every symbol the header declares, the torch
extension exposes the reference's binding names, and the host-side argument logic raises what the reference raises.
No kernel runs here."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "opsgnn_b200.h")


def _declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"OPSGNN_API\s+[\w\s\*]+?\b(opsgnn_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from ops_gnn import _cabi

    library = _cabi.load()
    declared = _declared_symbols()
    assert len(declared) >= 19
    missing = [name for name in declared if not hasattr(library, name)]
    assert not missing, f"declared in the header but not exported: {missing}"
    assert sorted(_cabi.EXPORTS) == declared, "ops_gnn/_cabi.py must list exactly the header's entry points"


def test_status_strings_and_argument_rejection_need_no_gpu():
    from ops_gnn import _cabi

    library = _cabi.load()
    assert library.opsgnn_status_string(0) == b"ok"
    assert b"workspace" in library.opsgnn_status_string(-3)
    size = ctypes.c_int64()
    assert library.opsgnn_csr_plan_bytes(1000, 5000, ctypes.byref(size)) == 0
    assert size.value == ((1000 + 5000 + 1023) // 1024 + 1) * 8  # one int64 per block of 1024 items, plus one
    assert library.opsgnn_csr_plan_bytes(-1, 0, ctypes.byref(size)) == -1
    desc = _cabi.CsrReduceDesc(10, 10, 7, 20, 1, 3, 20, 0, 0, _cabi.I64, _cabi.I64, _cabi.F32, _cabi.F32)
    assert library.opsgnn_csr_reduce_workspace_bytes(ctypes.byref(desc), ctypes.byref(size)) == -1  # 7 % 3 != 0
    desc.value_width = 7
    assert library.opsgnn_csr_reduce_workspace_bytes(ctypes.byref(desc), ctypes.byref(size)) == 0 and size.value > 0


def test_pybind_surface_matches_the_reference_binding():
    import ops_gnn

    names = ("segment_csr segment_csr_value segment_coo_forward segment_coo_value sddmm_csr spmm_sum_csr spmm_max_csr "
             "spmm_min_csr unified_spmm_csr scatter_forward scatter_softmax_forward scatter_softmax_backward "
             "scatter_log_softmax_forward scatter_log_softmax_backward scatter_logsumexp_forward "
             "scatter_logsumexp_backward segment_logsumexp_forward ind2ptr ptr2ind has_private_use1_kernel").split()
    for name in names:
        assert hasattr(ops_gnn._pybind, name), name
    sub = ops_gnn._pybind.torch_sparse_spmm
    for name in ("forward", "validate", "value_backward", "convert", "permute_values", "tensor_version"):
        assert hasattr(sub, name), name
    assert (ops_gnn._pybind.SEGMENT_COO_SUM, ops_gnn._pybind.SEGMENT_COO_MEAN, ops_gnn._pybind.SEGMENT_COO_MIN,
            ops_gnn._pybind.SEGMENT_COO_MAX) == (0, 1, 2, 3)
    assert sub.tensor_version(torch.zeros(1)) == 0
    assert isinstance(ops_gnn._pybind.has_private_use1_kernel("aten::add"), bool)


def test_no_cpu_path():
    import ops_gnn
    from ops_gnn.torch_sparse_spmm import csr_spmm

    ptr, col, x = torch.tensor([0, 1]), torch.tensor([0]), torch.ones(1, 4)
    with pytest.raises(ValueError, match="CUDA"):
        csr_spmm(ptr, col, None, x)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops_gnn.spmm(ptr, col, x)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops_gnn.segment_csr(x, ptr)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops_gnn.sddmm_csr(ptr, col, x, x)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops_gnn.scatter_softmax(x, torch.tensor([0]))
    with pytest.raises(RuntimeError, match="CUDA"):
        ops_gnn.segment_logsumexp(x, ptr)


def test_spmm_option_parsing_and_errors():
    from ops_gnn.spmm import _NativeScaledGather, _parse_call_options, spmm

    assert _parse_call_options("spmm", ("mul", "max"), {"rhs": 3}) == ("mul", "max", None, 3)
    with pytest.raises(TypeError, match="multiple values"):
        _parse_call_options("spmm", ("mul",), {"op": "add"})
    with pytest.raises(TypeError, match="unexpected keyword"):
        _parse_call_options("spmm", (), {"bogus": 1})
    with pytest.raises(TypeError, match="at most seven"):
        _parse_call_options("spmm", (1, 2, 3, 4, 5), {})
    ptr, col, x = torch.tensor([0, 1]), torch.tensor([0]), torch.ones(1, 4)
    with pytest.raises(RuntimeError, match="op must be"):
        spmm(ptr, col, x, "pow")
    with pytest.raises(RuntimeError, match="reduce must be"):
        spmm(ptr, col, x, "copy_lhs", "prod")
    with pytest.raises(ValueError, match="copy_lhs requires x"):
        spmm(ptr, col, None)
    with pytest.raises(ValueError, match="requires both"):
        spmm(ptr, col, x, "mul")
    with pytest.raises(TypeError, match="must be a Tensor"):
        spmm(ptr, [0], x)
    groups = _NativeScaledGather.weights_per_edge
    node = torch.zeros(5, 8, 64)
    assert groups(node, torch.zeros(9, 8, 1)) == 8
    assert groups(node, torch.zeros(9, 1, 1)) == 1
    assert groups(node, torch.zeros(9)) == 1
    assert groups(node, torch.zeros(9, 8, 64)) == 512
    assert groups(node, torch.zeros(9, 1, 64)) is None
    assert groups(node, torch.zeros(9, 4, 1)) is None


def test_sddmm_and_grouped_argument_errors():
    import ops_gnn

    ptr, col, x = torch.tensor([0, 1]), torch.tensor([0]), torch.ones(1, 4)
    with pytest.raises(ValueError, match="op must be"):
        ops_gnn.sddmm_csr(ptr, col, x, x, "pow")
    with pytest.raises(ValueError, match="lhs_target must be"):
        ops_gnn.sddmm_csr(ptr, col, x, x, "dot", "w")
    with pytest.raises(ValueError, match="rhs is not used"):
        ops_gnn.sddmm_csr(ptr, col, x, x, "copy_lhs")
    with pytest.raises(ValueError, match="same feature dim"):
        ops_gnn.sddmm_csr(ptr, col, x, torch.ones(1, 3))
    with pytest.raises(TypeError, match="indptr must be a Tensor"):
        ops_gnn.sddmm_csr([0, 1], col, x, x)
    with pytest.raises(IndexError, match="Dimension out of range"):
        ops_gnn.scatter_softmax(x, torch.tensor([0]), dim=5)
    with pytest.raises(TypeError, match="index dtype"):
        ops_gnn.scatter_log_softmax(x, torch.tensor([0.0]))
    with pytest.raises(ValueError, match="index must be 1-D"):
        ops_gnn.scatter_logsumexp(x, torch.tensor([[0]]))
    with pytest.raises(ValueError, match="reduce value"):
        ops_gnn.segment_csr(x, ptr, None, "prod")
    with pytest.raises(ValueError, match="segment_coo supports"):
        ops_gnn.segment_coo(x, torch.tensor([0]), None, None, "prod")
    with pytest.raises(IndexError, match="Dimension out of range"):
        ops_gnn.scatter(x, torch.tensor([0]), dim=7)
    with pytest.raises(TypeError, match="torch.int64"):
        ops_gnn.scatter(x, torch.tensor([0], dtype=torch.int32), dim=0)


def test_device_selection(monkeypatch):
    from ops_gnn import _device

    monkeypatch.setenv("OPS_GNN_TARGET", "sm100")
    assert _device.select_target() == "sm100"
    monkeypatch.setenv("OPS_GNN_TARGET", "sm90")
    with pytest.raises(ValueError, match="OPS_GNN_TARGET"):
        _device.select_target()
    monkeypatch.delenv("OPS_GNN_TARGET")
    if not torch.cuda.is_available():
        assert _device.select_target() == "sm100"


def test_static_scratch_covers_its_stated_maximum():
    """The built-in array of `opsgnn_sddmm_csr_static` must hold the plan of the largest call it accepts: the workspace
    query for 2^24 edges gives the array's size (256 KiB + one entry), one edge more asks for more."""
    import ctypes

    from ops_gnn import _cabi

    lib = _cabi.load()
    size = ctypes.c_int64()
    at_limit = _cabi.SddmmDesc(10, 1 << 24, 64, 10, 10, 0, 0, 2, _cabi.I64, _cabi.F32)
    assert lib.opsgnn_sddmm_workspace_bytes(ctypes.byref(at_limit), ctypes.byref(size)) == 0
    assert size.value == ((1 << 24) // 512 + 1) * 8
    beyond = _cabi.SddmmDesc(10, (1 << 24) + 512, 64, 10, 10, 0, 0, 2, _cabi.I64, _cabi.F32)
    assert lib.opsgnn_sddmm_workspace_bytes(ctypes.byref(beyond), ctypes.byref(size)) == 0
    assert size.value > ((1 << 24) // 512 + 1) * 8
