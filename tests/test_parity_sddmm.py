"""GPU parity of sddmm_csr against the reference's golden (fixtures) and the CPU oracle."""
import pytest
import torch

import oracle
from conftest import assert_close, assert_same, load_golden, requires_gpu

pytestmark = requires_gpu


def test_sddmm_fixtures(cuda_device):
    import ops_gnn

    for i, c in enumerate(load_golden("sddmm_csr")):
        what = f"case {i} {c['op']} {c['lhs'].dtype} targets=({c['lhs_target']},{c['rhs_target']}) feat={c['lhs'].shape[1:]}"
        lhs = c["lhs"].to(cuda_device) if c["op"] != "copy_rhs" else None
        rhs = c["rhs"].to(cuda_device) if c["op"] != "copy_lhs" else None
        got = ops_gnn.sddmm_csr(c["indptr"].to(cuda_device), c["indices"].to(cuda_device), lhs, rhs, c["op"],
                                c["lhs_target"], c["rhs_target"])
        if c["op"] in ("copy_lhs", "copy_rhs"):
            assert_same(got, c["out"], what)
        elif c["op"] == "dot":
            assert got.dtype == c["out"].dtype
            assert_close(got, c["out"], what=what)
        else:
            assert_close(got, c["out"], what=what)


def test_rmat_dot(cuda_device):
    """BASELINE config 3 shape at reduced scale: R-MAT graph, int32 indices, F = 64 fp32, out[e] = <A[row], B[col]>."""
    import bench
    import ops_gnn

    rowptr, col = bench.rmat_csr(16, 16 << 16, cuda_device, seed=3, index_dtype=torch.int32)
    nodes = 1 << 16
    gen = torch.Generator(device=cuda_device).manual_seed(5)
    a = torch.randn(nodes, 64, device=cuda_device, generator=gen)
    b = torch.randn(nodes, 64, device=cuda_device, generator=gen)
    got = ops_gnn.sddmm_csr(rowptr, col, a, b, "dot", "u", "v")
    want = oracle.sddmm_oracle(rowptr.cpu(), col.cpu(), a.cpu().double(), b.cpu().double(), "dot", 0, 2)
    bound = 1e-5 * (a.cpu().abs().double()[torch.repeat_interleave(torch.arange(nodes), (rowptr[1:] - rowptr[:-1]).cpu().long())]
                    * b.cpu().abs().double()[col.cpu().long()]).sum(-1).clamp(min=1.0)
    assert bool(((got.cpu().double() - want).abs() <= bound).all())
    out = torch.empty_like(got)
    assert ops_gnn.sddmm_csr(rowptr, col, a, b, "dot", 0, 2, out).data_ptr() == out.data_ptr()
    assert torch.equal(out, got)
    with pytest.raises(RuntimeError, match="sddmm_csr"):
        ops_gnn.sddmm_csr(rowptr, col, a[:10], b, "dot")
    with pytest.raises(ValueError, match="op must be"):
        ops_gnn.sddmm_csr(rowptr, col, a, b, "pow")
