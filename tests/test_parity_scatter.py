"""GPU parity of scatter and the grouped softmax family against the reference's goldens (fixtures) and the oracle."""
import pytest
import torch

import oracle
from conftest import assert_close, assert_same, load_golden, requires_gpu

pytestmark = requires_gpu


def test_scatter_fixtures(cuda_device):
    import ops_gnn

    for i, c in enumerate(load_golden("scatter")):
        what = f"case {i} {c['reduce']} {c['src'].dtype} {tuple(c['src'].shape)} dim={c['dim']} {c['source']}"
        src, index = c["src"].to(cuda_device), c["index"].to(cuda_device)
        seed = None if c["out_in"] is None else c["out_in"].clone().to(cuda_device)
        if c["reduce"] in ("min", "max"):
            fn = ops_gnn.scatter_min if c["reduce"] == "min" else ops_gnn.scatter_max
            out, arg = fn(src, index, c["dim"], seed, c["dim_size"])
            assert_same(out, c["out"], what)
            assert_same(arg, c["arg"], what + " arg")
        else:
            out = ops_gnn.scatter(src, index, c["dim"], seed, c["dim_size"], c["reduce"])
            if c["src"].dtype.is_floating_point:
                # the golden adds one element at a time in the value dtype: its 16-bit sums drift with the order, so
                # sums and means are bounded by the magnitude that was summed (products by the product itself)
                magnitude = None
                if c["reduce"] != "mul":
                    start = None if c["out_in"] is None else c["out_in"].double().abs()
                    magnitude = oracle.scatter_oracle(c["src"].double().abs(), c["index"], c["dim"], start, c["dim_size"],
                                                      c["reduce"])
                assert_close(out, c["out"], what=what, magnitude=magnitude)
            else:
                assert_same(out, c["out"], what)
        if seed is not None:
            assert out.data_ptr() == seed.data_ptr(), what


def test_scatter_compact_index_and_errors(cuda_device):
    import ops_gnn

    gen = torch.Generator().manual_seed(21)
    src = torch.randn(5000, 128, generator=gen)
    index = torch.randint(0, 700, (5000,), generator=gen)
    d_src, d_index = src.to(cuda_device), index.to(cuda_device)
    for reduce in ("sum", "mean"):
        want = oracle.scatter_oracle(src.double(), index, 0, None, 700, reduce).float()
        assert_close(ops_gnn.scatter(d_src, d_index, 0, None, 700, reduce), want, what=reduce)
    for reduce, fn in (("min", ops_gnn.scatter_min), ("max", ops_gnn.scatter_max)):
        out, arg = fn(d_src, d_index, 0, None, 700)
        want, want_arg = oracle.scatter_oracle(src, index, 0, None, 700, reduce)
        assert_same(out, want, reduce)
        assert_same(arg, want_arg, reduce + " arg")
    with pytest.raises(IndexError, match="out of bounds"):
        ops_gnn.scatter(d_src, d_index, 0, None, 10, "sum")
    with pytest.raises(IndexError, match="negative"):
        ops_gnn.scatter(d_src, d_index - 5, 0, None, 700, "sum")
    with pytest.raises(ValueError, match="reduce must be"):
        ops_gnn.scatter(d_src, d_index, 0, None, 700, "prod")
    with pytest.raises(RuntimeError, match="CUDA"):
        ops_gnn.scatter(src, index, 0, None, 700, "sum")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.float64])
def test_scatter_extrema_negative_zero(cuda_device, dtype):
    """-0.0 among negative and positive values: its bit pattern is INT_MIN as a signed integer, so an atomic extremum
    that picks the integer view by `v >= 0` lets it beat every negative in a min and lose to everything in a max."""
    import ops_gnn

    src = torch.tensor([-5.0, -0.0, 3.0, -0.0, -1.0, -0.0, 0.0, -2.0, -0.0, -0.0, 2.0, -0.0], dtype=dtype)
    index = torch.tensor([0, 0, 0, 1, 1, 2, 2, 3, 3, 4, 4, 5])
    for order in (torch.arange(12), torch.arange(11, -1, -1)):       # both arrival orders
        s, i = src[order], index[order]
        for reduce, fn in (("min", ops_gnn.scatter_min), ("max", ops_gnn.scatter_max)):
            out, arg = fn(s.to(cuda_device), i.to(cuda_device), 0, None, 7)
            want, want_arg = oracle.scatter_oracle(s, i, 0, None, 7, reduce)
            assert_same(out, want, f"{reduce} {dtype}")               # == treats the two zeros as equal, as torch does
            assert_same(arg, want_arg, f"{reduce} {dtype} arg")
    big = torch.where(torch.rand(20000, 8, generator=torch.Generator().manual_seed(3)) < 0.3,
                      torch.tensor(-0.0), -torch.rand(20000, 8, generator=torch.Generator().manual_seed(4))).to(dtype)
    where = torch.randint(0, 50, (20000,), generator=torch.Generator().manual_seed(5))
    for reduce, fn in (("min", ops_gnn.scatter_min), ("max", ops_gnn.scatter_max)):
        out, arg = fn(big.to(cuda_device), where.to(cuda_device), 0, None, 50)
        want, want_arg = oracle.scatter_oracle(big, where, 0, None, 50, reduce)
        assert_same(out, want, f"{reduce} {dtype} many")
        assert_same(arg, want_arg, f"{reduce} {dtype} many arg")


def test_grouped_fixtures(cuda_device):
    import ops_gnn

    for i, c in enumerate(load_golden("grouped_softmax")):
        dtype = c["src"].dtype
        src, index = c["src"].to(cuda_device), c["index"].to(cuda_device)
        for name, fn in (("softmax", ops_gnn.scatter_softmax), ("log_softmax", ops_gnn.scatter_log_softmax),
                         ("logsumexp", ops_gnn.scatter_logsumexp)):
            for labels in (index, index.to(torch.int32)):
                got = fn(src, labels, c["dim"], c["dim_size"])
                assert got.dtype == dtype
                assert_close(got, c[name].to(dtype), what=f"case {i} {name} {dtype} {labels.dtype}")


def test_config2_softmax_sorted_and_shuffled(cuda_device):
    """BASELINE config 2 shape at 1/8 scale: sorted labels take the single-sweep path, shuffled labels the atomic one;
    both must agree with the float64 oracle, and the gradients with autograd through the oracle."""
    import ops_gnn

    gen = torch.Generator().manual_seed(22)
    rows, feat = 131072, 128
    lengths = 1 + torch.distributions.Geometric(probs=torch.tensor(1 / 8.0)).sample((rows // 4,)).long()
    index = torch.repeat_interleave(torch.arange(lengths.numel()), lengths)[:rows].contiguous()
    groups = int(index[-1]) + 1
    src = torch.randn(rows, feat, generator=gen) * 3
    perm = torch.randperm(rows, generator=gen)
    for name, labels, values in (("sorted", index, src), ("shuffled", index[perm], src[perm])):
        d_src, d_index = values.to(cuda_device), labels.to(cuda_device)
        assert_close(ops_gnn.scatter_softmax(d_src, d_index, 0, groups),
                     oracle.grouped_softmax_oracle(values, labels, 0, groups).float(), what=name + " softmax")
        assert_close(ops_gnn.scatter_log_softmax(d_src, d_index, 0, groups),
                     oracle.grouped_softmax_oracle(values, labels, 0, groups, log=True).float(),
                     what=name + " log_softmax")
        assert_close(ops_gnn.scatter_logsumexp(d_src, d_index, 0, groups),
                     oracle.grouped_logsumexp_oracle(values, labels, 0, groups).float(), what=name + " logsumexp")


def test_eight_column_sorted_sources(cuda_device):
    """[E, 8] fp32 sources under sorted labels (per-head attention logits) take the chunked sweep: groups inside one
    128-row chunk, groups that straddle chunks, a hub group spanning hundreds of chunks that opens in the middle of a
    chunk, empty groups, int32 labels, and the reference's +inf / -inf / NaN rules
    (test/scatter_softmax/grouped_softmax_golden.py:50-86)."""
    import ops_gnn

    gen = torch.Generator().manual_seed(88)
    lengths = torch.cat([torch.randint(0, 40, (3000,), generator=gen), torch.tensor([57, 40000, 0, 0, 3, 700, 129, 128, 1])])
    index = torch.repeat_interleave(torch.arange(lengths.numel()), lengths).contiguous()
    groups = lengths.numel() + 2                    # two more empty groups at the end
    src = torch.randn(index.numel(), 8, generator=gen) * 4
    first = int((index == 5).nonzero()[0]) if (index == 5).any() else 0
    src[first, 0] = float("inf")                    # a group with +inf: softmax NaN, logsumexp +inf
    where = (index == 9).nonzero().flatten()
    if where.numel():
        src[where, 1] = float("-inf")               # a column of a group all -inf: NaN / -inf
    src[int((index == 3001).nonzero()[100]), 2] = float("nan")   # NaN inside the hub group
    for labels in (index, index.to(torch.int32)):
        d_src, d_index = src.to(cuda_device), labels.to(cuda_device)
        assert_close(ops_gnn.scatter_logsumexp(d_src, d_index, 0, groups),
                     oracle.grouped_logsumexp_oracle(src, index, 0, groups).float(), what="[E, 8] logsumexp")
        assert_close(ops_gnn.scatter_softmax(d_src, d_index, 0, groups),
                     oracle.grouped_softmax_oracle(src, index, 0, groups).float(), what="[E, 8] softmax")
        assert_close(ops_gnn.scatter_log_softmax(d_src, d_index, 0, groups),
                     oracle.grouped_softmax_oracle(src, index, 0, groups, log=True).float(), what="[E, 8] log_softmax")
    twice = ops_gnn.scatter_softmax(src.to(cuda_device), index.to(cuda_device), 0, groups)
    assert torch.equal(twice.isnan(), ops_gnn.scatter_softmax(src.to(cuda_device), index.to(cuda_device), 0, groups).isnan())
    assert torch.equal(torch.nan_to_num(twice), torch.nan_to_num(ops_gnn.scatter_softmax(src.to(cuda_device), index.to(cuda_device), 0, groups)))


def test_grouped_gradients(cuda_device):
    import ops_gnn

    gen = torch.Generator().manual_seed(23)
    index = torch.randint(0, 9, (200,), generator=gen)
    src = torch.randn(200, 6, generator=gen)
    upstream = torch.randn(200, 6, generator=gen)
    reduced_upstream = torch.randn(9, 6, generator=gen)
    for fn, ref, up in (
        (ops_gnn.scatter_softmax, lambda x: oracle.grouped_softmax_oracle(x, index, 0, 9), upstream),
        (ops_gnn.scatter_log_softmax, lambda x: oracle.grouped_softmax_oracle(x, index, 0, 9, log=True), upstream),
        (ops_gnn.scatter_logsumexp, lambda x: oracle.grouped_logsumexp_oracle(x, index, 0, 9), reduced_upstream),
    ):
        x = src.to(cuda_device).requires_grad_(True)
        fn(x, index.to(cuda_device), 0, 9).backward(up.to(cuda_device))
        x64 = src.double().requires_grad_(True)
        ref(x64).backward(up.double())
        assert_close(x.grad, x64.grad.float(), what=fn.__name__ + " grad")
