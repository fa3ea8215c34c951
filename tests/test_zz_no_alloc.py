"""The scratch-free SDDMM entry point (`opsgnn_sddmm_csr_static`) against the regular one, through the C ABI.

Some callers cannot hand the library device scratch: a plug-in inside a host application that has committed the whole
GPU to its own pool, or a loop in which allocator calls are forbidden.  For them the library keeps the row plan of
SDDMM in a fixed internal array.  This test drives both entry points with raw device pointers on the same inputs,
twice in a row (the second call reuses the array the first one filled, on a different graph size), and expects
bit-identical results: both run the same kernels and differ only in where the plan lives.  It also checks that a
request beyond the array's capacity is refused.  The file sorts last so a `-x` run has already run everything else.
"""
import ctypes

import pytest
import torch

from conftest import requires_gpu

pytestmark = requires_gpu


def _graph(device, rows, seed, index_dtype=torch.int64):
    gen = torch.Generator().manual_seed(seed)
    degree = torch.randint(0, 12, (rows,), generator=gen)
    degree[2] = 3000
    ptr = torch.zeros(rows + 1, dtype=torch.int64)
    ptr[1:] = degree.cumsum(0)
    col = torch.randint(0, rows, (int(ptr[-1]),), generator=gen)
    lhs = torch.randn(rows, 64, generator=gen)
    rhs = torch.randn(rows, 64, generator=gen)
    return [t.to(device) for t in (ptr.to(index_dtype), col.to(index_dtype), lhs, rhs)]


def _run(lib, cabi, static, ptr, col, lhs, rhs, op="dot"):
    nnz = col.numel()
    desc = cabi.SddmmDesc(ptr.numel() - 1, nnz, lhs.size(1), lhs.size(0), rhs.size(0), cabi.SDDMM_OPS[op], 0, 2,
                          cabi.torch_dtype_id(ptr.dtype), cabi.F32)
    out = torch.full((nnz,) if op == "dot" else (nnz, lhs.size(1)), float("nan"), device=ptr.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = [ctypes.byref(desc)] + [ctypes.c_void_p(t.data_ptr()) for t in (ptr, col, lhs, rhs, out)]
    if static:
        status = lib.opsgnn_sddmm_csr_static(*args, stream)
    else:
        size = ctypes.c_int64()
        assert lib.opsgnn_sddmm_workspace_bytes(ctypes.byref(desc), ctypes.byref(size)) == 0
        scratch = torch.empty(max(size.value, 8), dtype=torch.uint8, device=ptr.device)
        status = lib.opsgnn_sddmm_csr(*args, ctypes.c_void_p(scratch.data_ptr()), scratch.numel(), stream)
    assert status == 0, lib.opsgnn_status_string(status)
    torch.cuda.synchronize()
    return out


def test_static_scratch_matches_regular_entry_point(cuda_device):
    from ops_gnn import _cabi

    lib = _cabi.load()
    import oracle

    # calls in a row share the internal array: two graph sizes, both index widths, the dot product and an elementwise op
    for rows, seed, index_dtype, op in ((5000, 1, torch.int64, "dot"), (1200, 2, torch.int64, "dot"),
                                        (3000, 3, torch.int32, "dot"), (2000, 4, torch.int32, "mul")):
        inputs = _graph(cuda_device, rows, seed, index_dtype)
        regular = _run(lib, _cabi, False, *inputs, op=op)
        fixed = _run(lib, _cabi, True, *inputs, op=op)
        assert not torch.isnan(fixed).any()
        assert torch.equal(fixed, regular)
        # third leg: the CPU oracle, so the entry point stands on its own
        ptr, col, lhs, rhs = (t.cpu() for t in inputs)
        want = oracle.sddmm_oracle(ptr, col, lhs.double(), rhs.double(), op, "u", "v")
        scale = oracle.sddmm_oracle(ptr, col, lhs.double().abs(), rhs.double().abs(), op, "u", "v").clamp(min=1.0)
        assert float(((fixed.cpu().double() - want).abs() / scale).max()) <= 1e-5, f"{op} against the oracle"
    too_many = _cabi.SddmmDesc(10, (1 << 24) + 1, 64, 10, 10, 0, 0, 2, _cabi.I64, _cabi.F32)
    status = lib.opsgnn_sddmm_csr_static(ctypes.byref(too_many), None, None, None, None, None, None)
    assert status == -4 and b"maximum" in lib.opsgnn_status_string(status)
