"""GPU checks at the full sizes of BASELINE configs 3 and 4, where no CPU oracle finishes: size-independent
properties that tie the kernels to independent computations (column-weight checksums through torch.bincount,
position consistency of extrema, the SDDMM / SpMM adjoint identity, linearity on a row slice)."""
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
