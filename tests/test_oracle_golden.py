"""The CPU oracle against the reference's own goldens (committed fixtures) and known-answer vectors.

Every fixture case was produced by a golden function of the reference (see tests/golden/make_fixtures.py); the
known-answer vectors restate expectations written in the reference's test files, cited next to each.  Integers,
positions and extrema must match bit for bit; sums are compared at the documented tolerances because the oracle
accumulates in float64 where some goldens accumulate in the value dtype.
"""
import pytest
import torch

import oracle
from conftest import assert_close, assert_same, load_golden


def _close_or_same(got, want, what):
    if want.dtype.is_floating_point:
        assert got.dtype == want.dtype, what
        assert_close(got, want, what=what)
    else:
        assert_same(got, want, what)


def test_torch_sparse_spmm_fixtures():
    for i, c in enumerate(load_golden("torch_sparse_spmm")):
        out, arg = oracle.csr_spmm_oracle(c["ptr"], c["col"], c["value"], c["mat"], c["reduce"], c["outdtype"])
        what = f"case {i} {c['reduce']} {c['mat'].dtype}->{c['outdtype']}"
        if c["reduce"] in ("min", "max"):
            assert_same(out, c["out"], what)
            assert_same(arg, c["arg"], what + " arg")
        else:
            _close_or_same(out, c["out"], what)


def test_spmm_copy_fixtures():
    for i, c in enumerate(load_golden("spmm_copy")):
        what = f"case {i} {c['kind']} {c.get('op')} {c['reduce']}"
        if c["kind"] == "binary":
            continue  # message composition is host-side torch code, covered by the GPU tests
        op = c.get("op", "copy_lhs")
        got = oracle.spmm_copy_oracle(c["indptr"], c["indices"], c["x"], c["reduce"], op)
        if c["reduce"] in ("max", "min"):
            assert_same(got, c["out"], what)
        else:
            assert_close(got, c["out"], what=what)


def test_sddmm_fixtures():
    for i, c in enumerate(load_golden("sddmm_csr")):
        got = oracle.sddmm_oracle(c["indptr"], c["indices"], c["lhs"], c["rhs"], c["op"], c["lhs_target"], c["rhs_target"])
        assert_same(got, c["out"], f"case {i} {c['op']}")


def test_segment_csr_fixtures():
    for i, c in enumerate(load_golden("segment_csr")):
        what = f"case {i} {c['reduce']} {c['src'].dtype}"
        if c["reduce"] in ("min", "max"):
            out, arg = oracle.segment_csr_oracle(c["src"], c["indptr"], c["reduce"], return_arg=True)
            assert_same(out, c["out"], what)
            assert_same(arg, c["arg"], what + " arg")
        else:
            _close_or_same(oracle.segment_csr_oracle(c["src"], c["indptr"], c["reduce"]), c["out"], what)


def test_segment_coo_fixtures():
    for i, c in enumerate(load_golden("segment_coo")):
        what = f"case {i} {c['reduce']} {c['src'].dtype} out={c['out_in'] is not None}"
        got = oracle.segment_coo_oracle(c["src"], c["index"], c["out_in"], c["dim_size"], c["reduce"], return_arg=True)
        out, arg = got if isinstance(got, tuple) else (got, None)
        if c["reduce"] in ("min", "max"):
            assert_same(out, c["out"], what)
            assert_same(arg, c["arg"], what + " arg")
        else:
            _close_or_same(out, c["out"], what)


def test_scatter_fixtures():
    for i, c in enumerate(load_golden("scatter")):
        what = f"case {i} {c['reduce']} {c['src'].dtype} {c['source']}"
        got = oracle.scatter_oracle(c["src"], c["index"], c["dim"], c["out_in"], c["dim_size"], c["reduce"])
        out, arg = got if isinstance(got, tuple) else (got, None)
        if c["reduce"] in ("min", "max"):
            assert_same(out, c["out"], what)
            assert_same(arg, c["arg"], what + " arg")
        elif c["src"].dtype.is_floating_point:
            # the goldens add one element at a time in the value dtype; fp16/bf16 sums drift with the order, so sums
            # and means are bounded by the magnitude that was summed
            magnitude = None
            if c["reduce"] != "mul":
                start = None if c["out_in"] is None else c["out_in"].double().abs()
                magnitude = oracle.scatter_oracle(c["src"].double().abs(), c["index"], c["dim"], start, c["dim_size"],
                                                  c["reduce"])
            assert_close(out, c["out"], what=what, magnitude=magnitude)
        else:
            assert_same(out, c["out"], what)


def test_grouped_softmax_fixtures():
    for i, c in enumerate(load_golden("grouped_softmax")):
        args = (c["src"], c["index"], c["dim"], c["dim_size"])
        assert_close(oracle.grouped_softmax_oracle(*args), c["softmax"], torch.float64, f"case {i} softmax")
        assert_close(oracle.grouped_softmax_oracle(*args, log=True), c["log_softmax"], torch.float64,
                     f"case {i} log_softmax")
        assert_close(oracle.grouped_logsumexp_oracle(*args), c["logsumexp"], torch.float64, f"case {i} logsumexp")


def test_segment_logsumexp_fixtures():
    for i, c in enumerate(load_golden("segment_logsumexp")):
        assert_close(oracle.segment_logsumexp_oracle(c["src"], c["indptr"]), c["out"], torch.float64, f"case {i}")


def test_convert_fixtures():
    for c in load_golden("convert"):
        assert_same(oracle.ind2ptr_oracle(c["ind"], c["rows"]), c["ptr"], "ind2ptr")
        assert_same(oracle.ptr2ind_oracle(c["ptr"], c["ind"].numel()), c["back"], "ptr2ind")
        assert_same(oracle.ptr2ind_oracle(c["ptr"], c["ind"].numel()), c["ind"], "round trip")


def test_gather_fixtures():
    """gather_csr / gather_coo: the golden file's own known-answer table (every dtype it lists) and seeded cases."""
    for i, c in enumerate(load_golden("gather")):
        got = oracle.gather_csr_oracle(c["src"], c["indptr"])
        assert_same(got, c["out"], f"case {i} gather_csr {c['src'].dtype} {tuple(c['src'].shape)}")
        if "index" in c:
            assert_same(oracle.gather_coo_oracle(c["src"], c["index"]), c["out"], f"case {i} gather_coo")


# ---- known-answer vectors written in the reference's tests and docs ---------------------------------------------------
def test_ind2ptr_documented_example():
    # python/ops_gnn/ind2ptr.py:48-52 of the reference
    row = torch.tensor([2, 2, 4, 5, 5, 6])
    ptr = torch.tensor([0, 0, 0, 2, 2, 3, 5, 6, 6])
    assert_same(oracle.ind2ptr_oracle(row, 8), ptr)
    assert_same(oracle.ptr2ind_oracle(ptr, 6), row)


def test_torch_sparse_weight_example():
    # test/torch_sparse_spmm/arch35/test_torch_sparse_spmm.py:117-142: scalar and per-feature weights
    ptr, col = torch.tensor([0, 2]), torch.tensor([0, 1])
    mat = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    out, _ = oracle.csr_spmm_oracle(ptr, col, torch.tensor([2.0, 5.0]), mat, "sum")
    assert_same(out, torch.tensor([[22.0, 29.0, 36.0]]))
    out, _ = oracle.csr_spmm_oracle(ptr, col, torch.tensor([[2.0, 3.0, 4.0], [5.0, 6.0, 7.0]]), mat, "sum")
    assert_same(out, torch.tensor([[22.0, 36.0, 54.0]]))


def test_torch_sparse_extrema_special_values():
    # test_torch_sparse_spmm.py:518-534: NaN is skipped, an all-NaN or empty row gives (0, E), first tie wins
    ptr, col = torch.tensor([0, 3, 3, 5, 7]), torch.tensor([0, 1, 2, 3, 3, 0, 2])
    mat = torch.tensor([[float("nan")], [2.0], [2.0], [float("nan")]])
    out, arg = oracle.csr_spmm_oracle(ptr, col, None, mat, "max")
    assert_same(out, torch.tensor([[2.0], [0.0], [0.0], [2.0]]))
    assert_same(arg, torch.tensor([[1], [7], [7], [6]]))


def test_spmm_max_documented_example():
    # test/spmm_max/arch22/test_spmm_max.py:33-38: empty row gives 0, -inf survives, NaN propagates
    indptr, indices = torch.tensor([0, 2, 2, 3]), torch.tensor([0, 1, 2])
    x = torch.tensor([[1.0, float("nan")], [3.0, 0.0], [-float("inf"), 5.0]], dtype=torch.float16)
    got = oracle.spmm_copy_oracle(indptr, indices, x, "max")
    want = torch.tensor([[3.0, float("nan")], [0.0, 0.0], [-float("inf"), 5.0]], dtype=torch.float16)
    assert_same(got, want)


def test_segment_csr_first_occurrence():
    # test/segment_csr/arch35/test_segment_csr.py:435-445: ties keep the first position, empty gives src.size(dim)
    src = torch.tensor([[1.0], [3.0], [3.0], [2.0]])
    out, arg = oracle.segment_csr_oracle(src, torch.tensor([0, 3, 3, 4]), "max", return_arg=True)
    assert_same(out, torch.tensor([[3.0], [0.0], [2.0]]))
    assert_same(arg, torch.tensor([[1], [4], [3]]))


def test_scatter_documented_example():
    # test/scatter/arch35/test_scatter.py:95-118: later element wins ties, untouched targets report len(src)
    src = torch.tensor([5.0, 1.0, 1.0, 7.0, 7.0, 2.0])
    index = torch.tensor([0, 0, 0, 1, 1, 3])
    out, arg = oracle.scatter_oracle(src, index, 0, None, 4, "min")
    assert_same(out, torch.tensor([1.0, 7.0, 0.0, 2.0]))
    assert_same(arg, torch.tensor([2, 4, 6, 5]))
    out, arg = oracle.scatter_oracle(src, index, 0, None, 4, "max")
    assert_same(out, torch.tensor([5.0, 7.0, 0.0, 2.0]))
    assert_same(arg, torch.tensor([0, 4, 6, 5]))


def test_logsumexp_special_values():
    # test/common/test_grouped_log_softmax_suite.py:121-192: +inf member -> +inf, all -inf -> -inf, empty -> -inf
    src = torch.tensor([float("inf"), 1.0, -float("inf"), -float("inf"), 2.0])
    got = oracle.grouped_logsumexp_oracle(src, torch.tensor([0, 0, 1, 1, 3]), 0, 4)
    assert_same(got, torch.tensor([float("inf"), -float("inf"), -float("inf"), 2.0], dtype=torch.float64))
    got = oracle.segment_logsumexp_oracle(src, torch.tensor([0, 2, 4, 4, 5]))
    assert_same(got, torch.tensor([float("inf"), -float("inf"), -float("inf"), 2.0], dtype=torch.float64))


def test_vectorised_baseline_equals_oracle():
    """The function the benchmark times on the CPU computes the same SpMM-sum as the pinned oracle."""
    from oracle.spmm import csr_spmm_sum_vectorised

    c = load_golden("torch_sparse_spmm")[-8]
    assert c["reduce"] == "sum" and c["mat"].dim() == 2
    want, _ = oracle.csr_spmm_oracle(c["ptr"], c["col"], c["value"], c["mat"], "sum")
    got = csr_spmm_sum_vectorised(c["ptr"], c["col"], c["value"], c["mat"], edge_chunk=97)
    assert_close(got, want, what="vectorised baseline")
