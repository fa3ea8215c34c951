"""GPU parity of segment_csr / segment_coo / segment_logsumexp / ind2ptr / ptr2ind against the reference's goldens
(fixtures) and the CPU oracle."""
import pytest
import torch

import oracle
from conftest import assert_close, assert_same, load_golden, requires_gpu

pytestmark = requires_gpu


def _gpu(t, device):
    return None if t is None else t.to(device)


def test_segment_csr_fixtures(cuda_device):
    import ops_gnn

    for i, c in enumerate(load_golden("segment_csr")):
        what = f"case {i} {c['reduce']} {c['src'].dtype} ptr{tuple(c['indptr'].shape)}"
        src, indptr = _gpu(c["src"], cuda_device), _gpu(c["indptr"], cuda_device)
        if c["reduce"] in ("min", "max"):
            fn = ops_gnn.segment_min_csr if c["reduce"] == "min" else ops_gnn.segment_max_csr
            out, arg = fn(src, indptr)
            assert_same(out, c["out"], what)
            assert_same(arg, c["arg"], what + " arg")
        else:
            out = ops_gnn.segment_csr(src, indptr, None, c["reduce"])
            if c["src"].dtype.is_floating_point:
                # the golden accumulates in the value dtype: its bf16 sums are themselves a few bf16 roundings off
                assert_close(out, c["out"], what=what,
                             magnitude=oracle.segment_csr_oracle(c["src"].double().abs(), c["indptr"], c["reduce"]))
            else:
                assert_same(out, c["out"], what)


def test_segment_coo_fixtures(cuda_device):
    import ops_gnn

    for i, c in enumerate(load_golden("segment_coo")):
        what = f"case {i} {c['reduce']} {c['src'].dtype} out={c['out_in'] is not None}"
        src, index = _gpu(c["src"], cuda_device), _gpu(c["index"], cuda_device)
        seed = None if c["out_in"] is None else c["out_in"].clone().to(cuda_device)
        if c["reduce"] in ("min", "max"):
            fn = ops_gnn.segment_min_coo if c["reduce"] == "min" else ops_gnn.segment_max_coo
            out, arg = fn(src, index, seed, c["dim_size"])
            assert_same(out, c["out"], what)
            assert_same(arg, c["arg"], what + " arg")
            if seed is not None:
                assert out.data_ptr() == seed.data_ptr()
        else:
            out = ops_gnn.segment_coo(src, index, seed, c["dim_size"], c["reduce"])
            if c["src"].dtype.is_floating_point:
                assert_close(out, c["out"], what=what)
            else:
                assert_same(out, c["out"], what)


def test_segment_logsumexp_fixtures(cuda_device):
    import ops_gnn

    for i, c in enumerate(load_golden("segment_logsumexp")):
        out = ops_gnn.segment_logsumexp(_gpu(c["src"], cuda_device), _gpu(c["indptr"], cuda_device))
        assert out.dtype == c["src"].dtype
        assert_close(out, c["out"].to(c["src"].dtype), what=f"case {i} {c['src'].dtype}")


def test_convert_fixtures(cuda_device):
    import ops_gnn

    for c in load_golden("convert"):
        ptr = ops_gnn.ind2ptr(_gpu(c["ind"], cuda_device), c["rows"])
        assert_same(ptr, c["ptr"], "ind2ptr")
        assert_same(ops_gnn.ptr2ind(ptr, c["ind"].numel()), c["ind"], "ptr2ind")
    with pytest.raises(RuntimeError, match="ptr2ind"):
        ops_gnn.ptr2ind(torch.tensor([0, 3, 2, 5], device=cuda_device), 5)


def _config2(gen, rows, feat):
    """BASELINE config 2 shape: sorted index with geometric segment lengths (mean 8)."""
    lengths = 1 + torch.distributions.Geometric(probs=torch.tensor(1 / 8.0)).sample((rows // 4,)).long()
    ptr = torch.zeros(lengths.numel() + 1, dtype=torch.int64)
    ptr[1:] = lengths.cumsum(0)
    cut = int(torch.searchsorted(ptr, torch.tensor(rows), right=False))
    ptr = ptr[:cut + 1].clone()
    ptr[-1] = rows
    index = torch.repeat_interleave(torch.arange(ptr.numel() - 1), ptr[1:] - ptr[:-1])
    src = torch.randn(rows, feat, generator=gen)
    return src, ptr, index


@pytest.mark.parametrize("rows,feat", [(65536, 128), (1048576, 128)])
def test_config2_segments(cuda_device, rows, feat):
    import ops_gnn

    gen = torch.Generator().manual_seed(20261127)
    torch.manual_seed(20261127)
    src, ptr, index = _config2(gen, rows, feat)
    segments = ptr.numel() - 1
    d_src, d_ptr, d_index = src.to(cuda_device), ptr.to(cuda_device), index.to(cuda_device)
    for reduce in ("sum", "mean"):
        want = oracle.segment_csr_oracle(src, ptr, reduce)
        assert_close(ops_gnn.segment_csr(d_src, d_ptr, None, reduce), want, what="csr " + reduce)
        assert_close(ops_gnn.segment_coo(d_src, d_index, None, segments, reduce), want, what="coo " + reduce)
    for reduce, csr, coo in (("min", ops_gnn.segment_min_csr, ops_gnn.segment_min_coo),
                             ("max", ops_gnn.segment_max_csr, ops_gnn.segment_max_coo)):
        want, want_arg = oracle.segment_csr_oracle(src, ptr, reduce, return_arg=True)
        for name, got in (("csr", csr(d_src, d_ptr)), ("coo", coo(d_src, d_index, None, segments))):
            assert_same(got[0], want, f"{name} {reduce}")
            assert_same(got[1], want_arg, f"{name} {reduce} arg")
    assert_close(ops_gnn.segment_logsumexp(d_src, d_ptr), oracle.segment_logsumexp_oracle(src, ptr).float(),
                 what="segment_logsumexp")
    assert_same(ops_gnn.ind2ptr(d_index, segments), ptr, "ind2ptr")
    assert_same(ops_gnn.ptr2ind(d_ptr, rows), index, "ptr2ind")


def test_one_long_segment(cuda_device):
    """A single segment spanning every thread block: the carry chain across blocks decides the result."""
    import ops_gnn

    gen = torch.Generator().manual_seed(8)
    src = torch.randn(300000, 8, generator=gen)
    ptr = torch.tensor([0, 300000])
    d_src, d_ptr = src.to(cuda_device), ptr.to(cuda_device)
    out, arg = ops_gnn.segment_max_csr(d_src, d_ptr)
    want, want_arg = oracle.segment_csr_oracle(src, ptr, "max", return_arg=True)
    assert_same(out, want, "max")
    assert_same(arg, want_arg, "arg")
    total = ops_gnn.segment_csr(d_src, d_ptr, None, "sum")
    exact = src.double().sum(0, keepdim=True)
    assert float((total.cpu().double() - exact).abs().max()) <= 1e-5 * float(src.double().abs().sum(0).max())
    assert_close(ops_gnn.segment_logsumexp(d_src, d_ptr), oracle.segment_logsumexp_oracle(src, ptr).float())
