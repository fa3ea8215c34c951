"""GPU parity of gather_csr / gather_coo (the row expansions that invert the segment reductions) against the
reference's golden (fixtures: its own known-answer table in every dtype it lists, plus seeded cases) and the oracle at
BASELINE config 2's shape; `out=` identity, non-contiguous and aliasing `out`, and the argument errors of the
reference's host checks (csrc/npu/gather_csr/op_host/gather_csr.cpp:95-160)."""
import pytest
import torch

import oracle
from conftest import assert_same, load_golden, requires_gpu

pytestmark = requires_gpu


def test_gather_fixtures(cuda_device):
    import ops_gnn

    for i, c in enumerate(load_golden("gather")):
        src, ptr = c["src"].to(cuda_device), c["indptr"].to(cuda_device)
        what = f"case {i} {c['src'].dtype} {tuple(c['src'].shape)} ptr{tuple(c['indptr'].shape)} {c['source']}"
        assert_same(ops_gnn.gather_csr(src, ptr), c["out"], "gather_csr " + what)
        out = torch.full(c["out"].shape, 3, dtype=src.dtype, device=cuda_device)
        assert ops_gnn.gather_csr(src, ptr, out).data_ptr() == out.data_ptr()
        assert_same(out, c["out"], "gather_csr out= " + what)
        if "index" in c:
            index = c["index"].to(cuda_device)
            assert_same(ops_gnn.gather_coo(src, index), c["out"], "gather_coo " + what)
            assert ops_gnn.gather_coo(src, index, out.zero_()).data_ptr() == out.data_ptr()
            assert_same(out, c["out"], "gather_coo out= " + what)


def test_gather_inverts_segment_sum_at_config2(cuda_device):
    """Config 2 shape: 1,048,576 x 128 rows in geometric segments.  gather_csr(segment values) against the oracle, and
    as the gradient of a segment sum: d/dsrc sum(w * segment_sum(src)) = gather_csr(w)."""
    import ops_gnn

    gen = torch.Generator().manual_seed(20261127)
    rows, feat = 1 << 20, 128
    lengths = torch.empty(rows // 4).geometric_(1.0 / 8, generator=gen).long()
    ends = lengths.cumsum(0)
    count = int(torch.searchsorted(ends, torch.tensor(rows))) + 1
    ptr = torch.zeros(count + 1, dtype=torch.int64)
    ptr[1:] = ends[:count].clamp(max=rows)
    index = torch.repeat_interleave(torch.arange(count), ptr[1:] - ptr[:-1])
    weights = torch.randn(count, feat, generator=gen)
    d_w, d_ptr, d_index = weights.to(cuda_device), ptr.to(cuda_device), index.to(cuda_device)
    expanded = ops_gnn.gather_csr(d_w, d_ptr)
    assert_same(expanded, oracle.gather_csr_oracle(weights, ptr), "gather_csr config 2")
    assert_same(ops_gnn.gather_coo(d_w, d_index), oracle.gather_coo_oracle(weights, index), "gather_coo config 2")
    src = torch.randn(rows, feat, generator=gen).to(cuda_device)
    # adjoint identity: <w, segment_sum(src)> = <gather_csr(w), src>
    left = float((d_w.double() * ops_gnn.segment_sum_csr(src, d_ptr).double()).sum())
    right = float((expanded.double() * src.double()).sum())
    assert abs(left - right) <= 1e-6 * float((expanded.double() * src.double()).abs().sum())


def test_gather_out_contract_and_errors(cuda_device):
    import ops_gnn

    src = torch.arange(24, dtype=torch.float32, device=cuda_device).reshape(4, 6)
    ptr = torch.tensor([2, 2, 5, 5, 7], device=cuda_device)          # rows 0..1 uncovered, empty segments
    want = oracle.gather_csr_oracle(src.cpu(), ptr.cpu())
    holder = torch.full((7, 12), -1.0, device=cuda_device)
    strided = holder[:, ::2]                                          # non-contiguous out: computed aside, copied back
    assert ops_gnn.gather_csr(src, ptr, strided) is strided
    assert_same(strided, want, "non-contiguous out")
    assert float(holder[:, 1::2].min()) == -1.0, "bytes between the strided columns are untouched"
    assert_same(ops_gnn.gather_csr(src.t().contiguous().t(), ptr), want, "non-contiguous src")
    big = torch.zeros(11, 6, device=cuda_device)
    big[:4] = src
    aliased = ops_gnn.gather_csr(big[:4], ptr, big[:7])              # out aliases src: src is read from a copy
    assert_same(aliased, want, "out aliasing src")
    with pytest.raises(RuntimeError, match="indptr dtype must be int64"):
        ops_gnn.gather_csr(src, ptr.int())
    with pytest.raises(RuntimeError, match="must equal indptr.size"):
        ops_gnn.gather_csr(src, ptr[:-1])
    with pytest.raises(RuntimeError, match="non-decreasing"):
        ops_gnn.gather_csr(src, torch.tensor([0, 3, 2, 5, 7], device=cuda_device))
    with pytest.raises(RuntimeError, match="out.size"):
        ops_gnn.gather_csr(src, ptr, torch.empty(8, 6, device=cuda_device))
    with pytest.raises(RuntimeError, match="CUDA"):
        ops_gnn.gather_csr(src.cpu(), ptr.cpu())
    with pytest.raises(RuntimeError, match="index values must lie"):
        ops_gnn.gather_coo(src, torch.tensor([0, 1, 4], device=cuda_device))
    with pytest.raises(RuntimeError, match="prefix shapes"):
        ops_gnn.gather_coo(src.reshape(2, 2, 6), torch.zeros(3, 2, dtype=torch.int64, device=cuda_device))
    empty = ops_gnn.gather_csr(torch.empty(0, 6, device=cuda_device), torch.zeros(1, dtype=torch.int64, device=cuda_device))
    assert empty.shape == (0, 6)


def test_copy_rows_async(cuda_device):
    """`copy_rows_async` is one stream-ordered cudaMemcpyAsync: bit-exact, ordered after earlier work on the stream, and
    it refuses mismatched or strided operands."""
    import ops_gnn

    copy = ops_gnn._pybind.copy_rows_async
    src = torch.randn(4097, 96, device=cuda_device)
    dst = torch.zeros(8200, 96, device=cuda_device)
    side = torch.cuda.Stream(cuda_device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        doubled = src * 2                       # produced on the side stream right before the copy reads it
        copy(doubled, dst[100:4197])
        copy(src[:0], dst[:0])                  # empty: nothing to do
    torch.cuda.current_stream().wait_stream(side)
    assert torch.equal(dst[100:4197], src * 2)
    assert not dst[:100].any() and not dst[4197:].any()
    with pytest.raises(RuntimeError):
        copy(src, dst[:4096])                   # sizes differ
    with pytest.raises(RuntimeError):
        copy(src[:, :48], dst[:4097, :48])      # not contiguous
    with pytest.raises(RuntimeError):
        copy(src, torch.zeros(4097, 96, dtype=torch.float64, device=cuda_device))
