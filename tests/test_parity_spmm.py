"""GPU parity of the SpMM family: the CUDA path (ops_gnn -> _pybind planners -> C ABI -> sm_100a kernels) against the
golden fixtures produced by the reference and against the CPU oracle on seeded inputs."""
import pytest
import torch

import oracle
from conftest import assert_close, assert_same, load_golden, requires_gpu, row_sum_magnitude

pytestmark = requires_gpu


def _gpu(t, device):
    return None if t is None else t.to(device)


def _conditioned_close(got, ptr, col, value, mat, expected, tol, what):
    """Sum tolerance relative to the magnitude that was summed (sum of |terms|), the condition-aware form of a
    relative error: hub rows cancel thousands of N(0,1) terms down to O(1)."""
    e = col.numel()
    rows = torch.repeat_interleave(torch.arange(ptr.numel() - 1), (ptr[1:] - ptr[:-1]).long(), output_size=e)
    terms = mat.double().abs()[..., col.long(), :]
    if value is not None:
        terms = terms * value.double().abs().reshape(e, -1)
    scale = torch.zeros(expected.shape, dtype=torch.float64).index_add_(-2, rows, terms).clamp(min=1.0)
    error = (got.cpu().double() - expected.double()).abs() / scale
    assert float(error.max()) <= tol, f"{what}: conditioned error {float(error.max()):.3g} > {tol:g}"


def test_torch_sparse_spmm_fixtures(cuda_device):
    import ops_gnn

    forward = ops_gnn._pybind.torch_sparse_spmm.forward
    codes = {"sum": 0, "mean": 1, "min": 2, "max": 3}
    types = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.int32: 4}
    for i, c in enumerate(load_golden("torch_sparse_spmm")):
        what = f"case {i} {c['reduce']} {c['mat'].dtype}->{c['outdtype']} batch={c['mat'].dim() > 2}"
        out, arg = forward(_gpu(c["ptr"], cuda_device), _gpu(c["col"], cuda_device), _gpu(c["value"], cuda_device),
                           _gpu(c["mat"], cuda_device), codes[c["reduce"]], types[c["outdtype"]])
        assert out.dtype == c["outdtype"]
        if c["reduce"] in ("min", "max"):
            assert_same(out, c["out"], what)
            assert_same(arg, c["arg"], what + " arg")
        elif c["outdtype"] == torch.int32:
            assert_same(out, c["out"], what)
        else:
            assert_close(out, c["out"], c["mat"].dtype if c["outdtype"] == torch.float32 and c["mat"].dtype != torch.int8
                         else c["outdtype"], what)


def test_csr_spmm_public_api(cuda_device):
    from ops_gnn.torch_sparse_spmm import csr_spmm

    c = load_golden("torch_sparse_spmm")[-4]  # k = 132, hub row of 600 edges, finite values
    ptr, col, value, mat = (_gpu(c[k], cuda_device) for k in ("ptr", "col", "value", "mat"))
    total = csr_spmm(ptr, col, value, mat, "sum")
    want, _ = oracle.csr_spmm_oracle(c["ptr"], c["col"], c["value"], c["mat"], "sum")
    _conditioned_close(total, c["ptr"], c["col"], c["value"], c["mat"], want, 1e-5, "csr_spmm sum")
    best, where = csr_spmm(ptr, col, value, mat, "max")
    want, want_arg = oracle.csr_spmm_oracle(c["ptr"], c["col"], c["value"], c["mat"], "max")
    assert_same(best, want, "csr_spmm max")
    assert_same(where, want_arg, "csr_spmm max arg")
    with pytest.raises(ValueError, match="invalid CSR"):
        csr_spmm(ptr, col.clone().fill_(10 ** 6), None, mat, "sum")
    with pytest.raises(ValueError, match="reduce must be"):
        csr_spmm(ptr, col, None, mat, "prod")


def test_config1_uniform_degree(cuda_device):
    """BASELINE config 1 at full size: 4096 x 4096, degree U{0..32}, sorted unique columns, weights U[-1,1)."""
    from ops_gnn.torch_sparse_spmm import csr_spmm

    gen = torch.Generator().manual_seed(20261126)
    n, k = 4096, 64
    degree = torch.randint(0, 33, (n,), generator=gen)
    ptr = torch.zeros(n + 1, dtype=torch.int64)
    ptr[1:] = degree.cumsum(0)
    col = torch.cat([torch.randperm(n, generator=gen)[:d].sort().values for d in degree.tolist()])
    value = torch.rand(col.numel(), generator=gen) * 2 - 1
    mat = torch.randn(n, k, generator=gen)
    args = [t.to(cuda_device) for t in (ptr, col, value, mat)]
    for reduce in ("sum", "mean", "min", "max"):
        got = csr_spmm(*args, reduce)
        want, want_arg = oracle.csr_spmm_oracle(ptr, col, value, mat, reduce)
        if reduce in ("min", "max"):
            assert_same(got[0], want, reduce)
            assert_same(got[1], want_arg, reduce + " arg")
        else:
            _conditioned_close(got, ptr, col, value, mat, want, 1e-5, reduce)
    unweighted = __import__("ops_gnn").spmm(args[0], args[1], args[3], reduce="max")
    assert_same(unweighted, oracle.spmm_copy_oracle(ptr, col, mat, "max"), "spmm max")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2), (torch.float16, 2e-3)])
def test_power_law_graph(cuda_device, dtype, tol):
    """Skewed degrees with hub rows that span many thread blocks, empty rows, F = 256 (the headline shape)."""
    from ops_gnn.torch_sparse_spmm import csr_spmm

    gen = torch.Generator().manual_seed(7)
    rows, cols, k = 20000, 15000, 256
    degree = torch.distributions.Geometric(probs=torch.tensor(1 / 9.0)).sample((rows,)).long()
    degree[0], degree[1], degree[17], degree[rows - 1] = 60000, 0, 9000, 4000
    ptr = torch.zeros(rows + 1, dtype=torch.int64)
    ptr[1:] = degree.cumsum(0)
    col = torch.randint(0, cols, (int(ptr[-1]),), generator=gen)
    value = torch.rand(col.numel(), generator=gen).to(dtype)
    mat = torch.randn(cols, k, generator=gen).to(dtype)
    dev = [t.to(cuda_device) for t in (ptr, col, value, mat)]
    first = csr_spmm(*dev, "sum")
    again = csr_spmm(*dev, "sum")
    assert torch.equal(first, again), "the reduction order must not depend on scheduling"
    want, _ = oracle.csr_spmm_oracle(ptr, col, value, mat, "sum", torch.float64)
    _conditioned_close(first, ptr, col, value, mat, want, tol, f"sum {dtype}")
    if dtype == torch.float32:
        best, where = csr_spmm(*dev, "min")
        want, want_arg = oracle.csr_spmm_oracle(ptr, col, value, mat, "min")
        assert_same(best, want, "min")
        assert_same(where, want_arg, "min arg")
        # linearity: A(x + y) = Ax + Ay within the tolerance of three sums
        other = torch.randn(cols, k, generator=gen).to(cuda_device)
        both = csr_spmm(dev[0], dev[1], dev[2], dev[3] + other, "sum")
        parts = first + csr_spmm(dev[0], dev[1], dev[2], other, "sum")
        scale = first.abs().max().item()
        assert float((both - parts).abs().max()) <= 1e-4 * max(scale, 1.0)


def _copy_magnitude(c):
    """Sum (mean) of the absolute messages of a spmm_copy fixture case, float64: what its row reductions summed."""
    ptr, col, x = c["indptr"].long(), c["indices"].long(), c["x"].double()
    if c["kind"] == "binary":
        lhs, rhs = x[col], c["rhs"].double()
        terms = {"add": lhs.abs() + rhs.abs(), "sub": lhs.abs() + rhs.abs(), "mul": (lhs * rhs).abs(),
                 "div": (lhs / rhs).abs()}[c["op"]]
    else:
        terms = (x if c.get("op") == "copy_rhs" else x[col]).abs()
    return row_sum_magnitude(ptr, terms, mean=c["reduce"] == "mean")


def test_spmm_copy_fixtures(cuda_device):
    import ops_gnn

    for i, c in enumerate(load_golden("spmm_copy")):
        what = f"case {i} {c['kind']} {c.get('op')} {c['reduce']} {c['x'].dtype}"
        indptr, indices, x = (_gpu(c[k], cuda_device) for k in ("indptr", "indices", "x"))
        if c["kind"] == "binary":
            got = ops_gnn.bspmm(indptr, indices, x, c["op"], c["reduce"], rhs=_gpu(c["rhs"], cuda_device))
        elif c["x"].dim() == 3:
            got = ops_gnn.bspmm(indptr, indices, x, reduce=c["reduce"])
        else:
            got = ops_gnn.spmm(indptr, indices, x, c.get("op", "copy_lhs"), c["reduce"])
        if c["reduce"] in ("max", "min"):
            assert_same(got, c["out"], what)
        else:
            assert_close(got, c["out"], what=what, magnitude=_copy_magnitude(c))


@pytest.mark.parametrize("dtype,heads,width", [(torch.float32, 8, 64), (torch.float32, 4, 32), (torch.float16, 8, 32),
                                               (torch.float16, 8, 64), (torch.float32, 3, 64)])
def test_fused_attention_aggregation(cuda_device, dtype, heads, width):
    """bspmm(op='mul') with one weight per (edge, head) runs fused and equals the materialised composition.  The
    shapes cover the instance whose weights are bulk-copied beside the gathered rows (8 x 64 fp32, 8 x 32 and 8 x 64 fp16), and
    shapes that stay on per-lane weight loads (odd head counts, narrow rows)."""
    import ops_gnn

    gen = torch.Generator().manual_seed(3)
    nodes = 3000
    degree = torch.randint(0, 40, (nodes,), generator=gen)
    degree[7], degree[8], degree[2000] = 9000, 0, 2500      # hub rows that span thread blocks, an empty row
    ptr = torch.zeros(nodes + 1, dtype=torch.int64)
    ptr[1:] = degree.cumsum(0)
    col = torch.randint(0, nodes, (int(ptr[-1]),), generator=gen)
    x = torch.randn(nodes, heads, width, generator=gen).to(dtype)
    alpha = torch.rand(col.numel(), heads, 1, generator=gen).to(dtype)
    args = (ptr.to(cuda_device), col.to(cuda_device), x.to(cuda_device), "mul", "sum")
    got = ops_gnn.bspmm(*args, rhs=alpha.to(cuda_device))
    assert torch.equal(got, ops_gnn.bspmm(*args, rhs=alpha.to(cuda_device))), "bitwise reproducible"
    rows = torch.repeat_interleave(torch.arange(nodes), degree)
    terms = x.double()[col] * alpha.double()
    want = torch.zeros(nodes, heads, width, dtype=torch.float64).index_add_(0, rows, terms)
    scale = torch.zeros(nodes, heads, width, dtype=torch.float64).index_add_(0, rows, terms.abs()).clamp(min=1.0)
    tol = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 1e-2}[dtype]
    error = ((got.cpu().double() - want).abs() / scale).max().item()
    assert error <= tol, f"u_mul_e_sum {dtype} {heads}x{width}: conditioned error {error:.3g} > {tol:g}"


def test_backward_matches_dense(cuda_device):
    from ops_gnn.torch_sparse_spmm import csr_spmm

    gen = torch.Generator().manual_seed(4)
    rows, cols, k = 60, 45, 20
    dense_mask = torch.rand(rows, cols, generator=gen) < 0.15
    weights = torch.randn(rows, cols, generator=gen) * dense_mask
    ptr = torch.zeros(rows + 1, dtype=torch.int64)
    ptr[1:] = dense_mask.sum(1).cumsum(0)
    r, c = dense_mask.nonzero(as_tuple=True)
    value = weights[r, c].to(cuda_device).requires_grad_(True)
    mat = torch.randn(cols, k, generator=gen).to(cuda_device).requires_grad_(True)
    out = csr_spmm(ptr.to(cuda_device), c.to(cuda_device), value, mat, "sum")
    upstream = torch.randn(rows, k, generator=gen).to(cuda_device)
    out.backward(upstream)
    dense = weights.double()
    want_mat = dense.t() @ upstream.cpu().double()
    want_value = (upstream.cpu().double() @ mat.detach().cpu().double().t())[r, c]
    assert_close(mat.grad, want_mat.float(), what="d mat")
    assert_close(value.grad, want_value.float(), what="d value")


@pytest.mark.parametrize("dtype,widths,tol", [
    (torch.float32, (4, 8, 16, 32, 64), 1e-5),
    (torch.float16, (8, 16, 32, 64, 128), 2e-3),
    (torch.bfloat16, (8, 64, 128), 1e-2),
])
def test_narrow_rows(cuda_device, dtype, widths, tol):
    """Rows of 16 to 256 bytes: several edges share one warp instruction and lane groups are merged at row ends.
    Ties, NaN and infinities are planted so the merge has to reproduce the first-occurrence and NaN rules."""
    import ops_gnn
    from ops_gnn.torch_sparse_spmm import csr_spmm

    gen = torch.Generator().manual_seed(11)
    rows, cols = 6000, 5000
    degree = torch.randint(0, 40, (rows,), generator=gen)
    degree[5], degree[6], degree[4000] = 30000, 0, 7000
    ptr = torch.zeros(rows + 1, dtype=torch.int64)
    ptr[1:] = degree.cumsum(0)
    col = torch.randint(0, cols, (int(ptr[-1]),), generator=gen)
    value = torch.rand(col.numel(), generator=gen).to(dtype)
    for k in widths:
        mat = torch.randn(cols, k, generator=gen)
        mat = (mat * 4).round() / 4          # many exact ties
        mat[17, 0], mat[18, k - 1], mat[19, 1] = float("nan"), float("inf"), float("-inf")
        mat = mat.to(dtype)
        dev = [t.to(cuda_device) for t in (ptr, col, value, mat)]
        got = csr_spmm(*dev, "sum")
        again = csr_spmm(*dev, "sum")
        assert torch.equal(torch.nan_to_num(got), torch.nan_to_num(again)), "the result must not depend on scheduling"
        want, _ = oracle.csr_spmm_oracle(ptr, col, value, mat, "sum", torch.float64)
        finite = torch.isfinite(want)
        assert torch.equal(torch.isnan(got.cpu()), torch.isnan(want)), f"NaN pattern, K={k}"
        assert torch.equal(got.cpu().double()[torch.isinf(want)], want[torch.isinf(want)]), f"infinities, K={k}"
        clean_mat = torch.nan_to_num(mat.float(), nan=0.0, posinf=0.0, neginf=0.0)
        clean_got = torch.where(finite, got.cpu().float(), torch.zeros(()))
        clean_want, _ = oracle.csr_spmm_oracle(ptr, col, value, clean_mat.to(dtype), "sum", torch.float64)
        _conditioned_close(clean_got, ptr, col, value, clean_mat, torch.where(finite, clean_want, torch.zeros((), dtype=torch.float64)),
                           tol, f"sum K={k} {dtype}")
        for reduce in ("max", "min"):
            best, where = csr_spmm(dev[0], dev[1], None, dev[3], reduce)
            want, want_arg = oracle.csr_spmm_oracle(ptr, col, None, mat, reduce)
            assert_same(best, want, f"{reduce} K={k} {dtype}")
            assert_same(where, want_arg, f"{reduce} arg K={k} {dtype}")
        if dtype != torch.bfloat16:
            unweighted = ops_gnn.spmm(dev[0], dev[1], dev[3], reduce="max")
            assert_same(unweighted, oracle.spmm_copy_oracle(ptr, col, mat, "max"), f"spmm max K={k}")
        # the segment forms of the same engine (consecutive source rows, contiguous stage copies)
        src = mat[col]                      # [E, k]
        d_src = src.to(cuda_device)
        seg_want, seg_arg = oracle.segment_csr_oracle(src, ptr, "max", return_arg=True)
        seg_got = ops_gnn.segment_max_csr(d_src, dev[0])
        assert_same(seg_got[0], seg_want, f"segment max K={k}")
        assert_same(seg_got[1], seg_arg, f"segment max arg K={k}")
        lse = ops_gnn.segment_logsumexp(d_src, dev[0])
        lse_want = oracle.segment_logsumexp_oracle(src, ptr)
        assert_close(lse, lse_want.to(lse.dtype), what=f"segment_logsumexp K={k} {dtype}")
