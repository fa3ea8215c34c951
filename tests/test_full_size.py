"""GPU checks at the full sizes of BASELINE configs 3, 4 and 5.

Two kinds.  (1) The CPU oracle itself, on three contiguous row ranges of every full-size launch - the first (hub) rows,
the rows around the median edge and the last rows, about two million edges each: the rows of the full-size GPU result
are copied to the host and compared with the float64 oracle of the same rows (sums within 1e-5 for fp32 and 1e-2 for
bf16 of the magnitude summed, extrema and their positions bit for bit).  The oracle sees the range as a graph of its
own: the dense rows its columns reference are gathered on the GPU and the columns relabelled, so no 17-GB matrix
crosses to the host.  (2) Size-independent properties over ALL rows that tie the kernels to independent computations
(column-weight checksums through torch.bincount, position consistency of extrema, the SDDMM / SpMM adjoint identity,
linearity)."""
import os
import sys

import pytest
import torch

from conftest import ROOT, requires_gpu

pytestmark = requires_gpu


def _rmat(scale, edge_factor, device, seed, index_dtype):
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    from bench import rmat_csr

    return rmat_csr(scale, edge_factor << scale, device, seed=seed, index_dtype=index_dtype)


def _needs(device, gigabytes):
    free, _ = torch.cuda.mem_get_info(device)
    if free < gigabytes * (1 << 30):
        pytest.skip(f"needs {gigabytes} GiB of free device memory")


SAMPLE_EDGES = 1 << 21


def _row_ranges(rowptr, target_edges=SAMPLE_EDGES):
    """Three contiguous row ranges holding about `target_edges` edges each: first rows, around the median edge, last rows."""
    rows, nnz = rowptr.numel() - 1, int(rowptr[-1])

    def row_of(edge, right):
        return int(torch.searchsorted(rowptr, torch.tensor([edge], device=rowptr.device, dtype=rowptr.dtype), right=right))

    head = (0, max(row_of(min(target_edges, nnz), False), 1))
    first = max(row_of(nnz // 2, True) - 1, 0)
    middle = (first, max(row_of(min(nnz // 2 + target_edges, nnz), False), first + 1))
    tail = (min(max(row_of(max(nnz - target_edges, 0), True) - 1, 0), rows - 1), rows)
    return [head, middle, tail]


def _local_graph(rowptr, col, first, last, *dense):
    """Rows [first, last) as a graph of their own on the host: pointers rebased, columns relabelled to the distinct
    rows they reference, and those rows of every matrix in `dense` (gathered on the GPU)."""
    lo, hi = int(rowptr[first]), int(rowptr[last])
    distinct, local_col = torch.unique(col[lo:hi].long(), return_inverse=True)
    ptr = (rowptr[first:last + 1].long() - lo).cpu()
    return ptr, local_col.cpu(), (lo, hi), [m[distinct].cpu() for m in dense]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
def test_config4_spmm_rows_against_oracle(cuda_device, dtype, tol):
    """BASELINE config 4 at full size (16.7M nodes, 263M edges, F = 256): rows of the GPU product against the oracle."""
    import oracle
    from ops_gnn.torch_sparse_spmm import csr_spmm

    _needs(cuda_device, 60)
    scale, feat = 24, 256
    rowptr, col = _rmat(scale, 16, cuda_device, 20261129, torch.int64)
    gen = torch.Generator(device=cuda_device).manual_seed(7)
    value = torch.rand(col.numel(), device=cuda_device, generator=gen).to(dtype)
    x = torch.randn(1 << scale, feat, device=cuda_device, generator=gen).to(dtype)
    out = csr_spmm(rowptr, col, value, x, "sum")
    narrow = x[:, :64].contiguous()
    best, where = csr_spmm(rowptr, col, None, narrow, "max") if dtype == torch.float32 else (None, None)
    for first, last in _row_ranges(rowptr):
        ptr, local_col, (lo, hi), (x_rows, narrow_rows) = _local_graph(rowptr, col, first, last, x, narrow)
        weights = value[lo:hi].cpu()
        want, _ = oracle.csr_spmm_oracle(ptr, local_col, weights, x_rows, "sum", torch.float64)
        magnitude, _ = oracle.csr_spmm_oracle(ptr, local_col, weights.double().abs(), x_rows.double().abs(), "sum", torch.float64)
        error = (out[first:last].cpu().double() - want).abs() / magnitude.clamp(min=1.0)
        assert float(error.max()) <= tol, f"rows [{first}, {last}) {dtype}: error {float(error.max()):.3g} of the magnitude summed"
        if best is not None:
            want_best, want_where = oracle.csr_spmm_oracle(ptr, local_col, None, narrow_rows, "max")
            assert torch.equal(best[first:last].cpu(), want_best), f"max values, rows [{first}, {last})"
            empty = want_where == local_col.numel()           # the oracle's "nothing selected" is its own edge count
            assert torch.equal(torch.where(empty, torch.full_like(want_where, col.numel()), want_where + lo),
                               where[first:last].cpu()), f"max positions, rows [{first}, {last})"


def test_config3_sddmm_edges_against_oracle(cuda_device):
    """BASELINE config 3 at full size (2.1M nodes, 63.5M edges, F = 64, int32): edge values against the oracle."""
    import oracle
    import ops_gnn

    _needs(cuda_device, 12)
    scale, feat = 21, 64
    indptr, indices = _rmat(scale, 32, cuda_device, 20261128, torch.int32)
    gen = torch.Generator(device=cuda_device).manual_seed(9)
    a = torch.randn(1 << scale, feat, device=cuda_device, generator=gen)
    b = torch.randn(1 << scale, feat, device=cuda_device, generator=gen)
    dots = ops_gnn.sddmm_csr(indptr, indices, a, b, "dot", "u", "v")
    for first, last in _row_ranges(indptr):
        ptr, local_col, (lo, hi), (b_rows,) = _local_graph(indptr, indices, first, last, b)
        a_rows = a[first:last].cpu()
        want = oracle.sddmm_oracle(ptr, local_col, a_rows.double(), b_rows.double(), "dot", "u", "v")
        magnitude = oracle.sddmm_oracle(ptr, local_col, a_rows.double().abs(), b_rows.double().abs(), "dot", "u", "v")
        error = (dots[lo:hi].cpu().double() - want).abs() / magnitude.clamp(min=1.0)
        assert float(error.max()) <= 1e-5, f"edges of rows [{first}, {last}): error {float(error.max()):.3g}"


def test_config5_attention_rows_against_oracle(cuda_device):
    """BASELINE config 5 at full size (2.1M nodes, 32M edges + self loops, 8 heads x 64): the composed layer (SDDMM add,
    LeakyReLU, scatter_softmax over destination rows, fused per-head aggregation) against the oracle composition."""
    import oracle
    import ops_gnn

    _needs(cuda_device, 30)
    scale, heads, width = 21, 8, 64
    nodes = 1 << scale
    indptr, indices = _rmat(scale, 16, cuda_device, 20261130, torch.int64)
    rows = ops_gnn.ptr2ind(indptr, indices.numel())
    loops = torch.arange(nodes, device=cuda_device)
    keys = torch.unique(torch.cat([(rows << scale) | indices, (loops << scale) | loops]))   # add the self loops, sorted
    rows, indices = keys >> scale, keys & (nodes - 1)
    indptr = ops_gnn.ind2ptr(rows, nodes)
    gen = torch.Generator(device=cuda_device).manual_seed(11)
    x = torch.randn(nodes, heads, width, device=cuda_device, generator=gen)
    left = torch.randn(nodes, heads, device=cuda_device, generator=gen)
    right = torch.randn(nodes, heads, device=cuda_device, generator=gen)
    logits = ops_gnn.sddmm_csr(indptr, indices, left, right, "add", "u", "v")
    alpha = ops_gnn.scatter_softmax(torch.nn.functional.leaky_relu(logits, 0.2), rows, 0, nodes)
    out = ops_gnn.bspmm(indptr, indices, x, "mul", "sum", rhs=alpha.unsqueeze(-1))
    fused = ops_gnn.gat_aggregate(indptr, indices, x, left, right, 0.2, edge_rows=rows)   # the same layer in two launches
    flat = x.view(nodes, heads * width)
    for first, last in _row_ranges(indptr, SAMPLE_EDGES // 2):
        ptr, local_col, (lo, hi), (x_rows, right_rows) = _local_graph(indptr, indices, first, last, flat, right)
        local_rows = oracle.ptr2ind_oracle(ptr, hi - lo)
        want_logits = oracle.sddmm_oracle(ptr, local_col, left[first:last].cpu().double(), right_rows.double(), "add", "u", "v")
        want_alpha = oracle.grouped_softmax_oracle(torch.nn.functional.leaky_relu(want_logits, 0.2), local_rows, 0, last - first)
        assert float((alpha[lo:hi].cpu().double() - want_alpha).abs().max()) <= 1e-5, f"attention weights, rows [{first}, {last})"
        terms = x_rows.double().view(-1, heads, width)[local_col] * want_alpha.unsqueeze(-1)
        want = torch.zeros(last - first, heads, width, dtype=torch.float64).index_add_(0, local_rows, terms)
        magnitude = torch.zeros_like(want).index_add_(0, local_rows, terms.abs()).clamp(min=1.0)
        error = (out[first:last].cpu().double() - want).abs() / magnitude
        assert float(error.max()) <= 1e-5, f"aggregated features, rows [{first}, {last}): error {float(error.max()):.3g}"
        error = (fused[first:last].cpu().double() - want).abs() / magnitude
        assert float(error.max()) <= 1e-5, f"fused layer, rows [{first}, {last}): error {float(error.max()):.3g}"


def test_config4_spmm_checksums(cuda_device):
    """263M edges x 256 features, fp32: sum over output rows == sum over columns of (column weight x X row)."""
    from ops_gnn.torch_sparse_spmm import csr_spmm

    _needs(cuda_device, 80)
    scale, feat = 24, 256
    rowptr, col = _rmat(scale, 16, cuda_device, 20261129, torch.int64)
    gen = torch.Generator(device=cuda_device).manual_seed(7)
    value = torch.rand(col.numel(), device=cuda_device, generator=gen)
    x = torch.randn(1 << scale, feat, device=cuda_device, generator=gen)
    out = csr_spmm(rowptr, col, value, x, "sum")
    column_weight = torch.bincount(col, weights=value.double(), minlength=1 << scale)
    want = torch.zeros(feat, dtype=torch.float64, device=cuda_device)
    magnitude = torch.zeros(feat, dtype=torch.float64, device=cuda_device)
    for start in range(0, 1 << scale, 1 << 21):                     # chunked: keeps the fp64 temporaries small
        block = x[start:start + (1 << 21)].double() * column_weight[start:start + (1 << 21), None]
        want += block.sum(0)
        magnitude += block.abs().sum(0)
    got = torch.zeros(feat, dtype=torch.float64, device=cuda_device)
    for start in range(0, 1 << scale, 1 << 21):
        got += out[start:start + (1 << 21)].double().sum(0)
    assert float(((got - want).abs() / magnitude).max()) <= 1e-6, "checksum of the full-size SpMM"
    # degrees through the same kernel: A @ 1 with unit weights is the row length, exactly
    ones = torch.ones(1 << scale, 4, device=cuda_device)
    degree = csr_spmm(rowptr, col, None, ones, "sum")[:, 0]
    assert torch.equal(degree.long(), rowptr[1:] - rowptr[:-1])
    del out, ones, degree
    # extrema: the reported position must hold the reported value, and lie inside the row
    best, where = csr_spmm(rowptr, col, None, x[:, :64].contiguous(), "max")
    rows_with_edges = (rowptr[1:] > rowptr[:-1])
    picked = torch.where(rows_with_edges[:, None], where, torch.zeros_like(where))
    gathered = x[:, :64].contiguous()[col[picked.reshape(-1)], torch.arange(64, device=cuda_device).repeat(1 << scale)]
    assert torch.equal(torch.where(rows_with_edges[:, None], gathered.view(-1, 64), torch.zeros_like(best)), best)
    inside = (where >= rowptr[:-1, None]) & (where < rowptr[1:, None])
    assert bool((inside | ~rows_with_edges[:, None]).all())
    assert bool((where[~rows_with_edges] == col.numel()).all()) and bool((best[~rows_with_edges] == 0).all())


def test_config3_sddmm_adjoint_identity(cuda_device):
    """63.5M edges, F = 64, int32: sum_e <A[row e], B[col e]> == sum_r <A[r], (Adj @ B)[r]> ties SDDMM to SpMM."""
    import ops_gnn

    _needs(cuda_device, 12)
    scale, feat = 21, 64
    indptr, indices = _rmat(scale, 32, cuda_device, 20261128, torch.int32)
    gen = torch.Generator(device=cuda_device).manual_seed(9)
    a = torch.randn(1 << scale, feat, device=cuda_device, generator=gen)
    b = torch.randn(1 << scale, feat, device=cuda_device, generator=gen)
    dots = ops_gnn.sddmm_csr(indptr, indices, a, b, "dot", "u", "v")
    gathered = ops_gnn.spmm(indptr, indices, b, reduce="sum")        # (Adj @ B), unweighted copy_lhs
    lhs = float(dots.double().sum())
    rhs = float((a.double() * gathered.double()).sum())
    scale_of_terms = float(dots.double().abs().sum())
    assert abs(lhs - rhs) <= 1e-6 * scale_of_terms
    # swapping the operands and the targets gives the same edge values (the kernel caches the row-side operand)
    swapped = ops_gnn.sddmm_csr(indptr, indices, b, a, "dot", "v", "u")
    assert torch.equal(dots, swapped)
    # linearity on a slice of rows: dot(u, v1 + v2) = dot(u, v1) + dot(u, v2) within fp32 rounding
    other = torch.randn(1 << scale, feat, device=cuda_device, generator=gen)
    both = ops_gnn.sddmm_csr(indptr, indices, a, b + other, "dot", "u", "v")
    parts = dots + ops_gnn.sddmm_csr(indptr, indices, a, other, "dot", "u", "v")
    assert float((both - parts).abs().max()) <= 1e-4 * float(both.abs().max())
