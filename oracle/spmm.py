"""Oracle of CSR SpMM.  Test infrastructure; see the package docstring.

`csr_spmm_oracle` follows `golden` of the reference's test/torch_sparse_spmm/arch35/golden.py:91-116: products are
formed and reduced in float64; min/max ignore NaN products, report the first edge that attains the extremum and
give (0, E) for rows with no selectable product; mean divides by the row's edge count; int32 output truncates.
`spmm_copy_oracle` follows `unified_spmm_reference` (test/unified_spmm/arch22/golden.py:42-92) and
`spmm_{sum,max}_reference` (test/spmm_sum/arch22/golden.py:13-22, test/spmm_max/arch22/golden.py:13-24): unweighted
gather (`copy_lhs`) or edge rows (`copy_rhs`), fp16 computed in fp32, max/min through `scatter_reduce_` (NaN
propagates), rows without edges are 0.
"""
import torch

from ._rows import edge_rows, first_extremum


def csr_spmm_oracle(ptr, col, value, mat, reduce, outdtype=None):
    ptr, col = ptr.cpu().to(torch.int64), col.cpu().to(torch.int64)
    mat = mat.cpu()
    outdtype = outdtype or (torch.int32 if mat.dtype == torch.int8 else mat.dtype)
    m, k, e = ptr.numel() - 1, mat.size(-1), col.numel()
    rows = edge_rows(ptr, e)
    lead = mat.shape[:-2]
    # [E, B, K] so that dim 0 is the edge axis
    flat = mat.double().reshape(-1, mat.size(-2), k)
    product = flat[:, col, :].permute(1, 0, 2).contiguous()
    if value is not None:
        product = product * value.cpu().double().reshape(e, 1, -1)
    b = flat.size(0)
    arg = torch.full((m, b, k), e, dtype=torch.int64)
    if reduce in ("sum", "add", "mean"):
        out = torch.zeros((m, b, k), dtype=torch.float64).index_add_(0, rows, product)
        if reduce == "mean":
            # Matches product.mean(-2): float64 sum divided by the row's edge count (rows without edges stay 0).
            degree = (ptr[1:] - ptr[:-1]).clamp(min=1).double().reshape(m, 1, 1)
            out = out / degree
    else:
        out, arg = first_extremum(product, rows, m, reduce == "min", ~torch.isnan(product), e)
    out = out.permute(1, 0, 2).reshape(*lead, m, k)
    arg = arg.permute(1, 0, 2).reshape(*lead, m, k)
    if outdtype == torch.int32:
        out = out.trunc()
    return out.to(outdtype), arg


def spmm_copy_oracle(indptr, indices, x, reduce="sum", op="copy_lhs"):
    indptr, x = indptr.cpu(), x.cpu()
    m = indptr.numel() - 1
    values = x if op == "copy_rhs" else x[indices.cpu().long()]
    compute = values.float() if values.dtype in (torch.float16, torch.bfloat16) else values
    rows = edge_rows(indptr, compute.size(0))
    shape = (m,) + tuple(compute.shape[1:])
    degree = (indptr[1:] - indptr[:-1]).long()
    if reduce in ("sum", "mean"):
        out = torch.zeros(shape, dtype=compute.dtype).index_add_(0, rows, compute)
        if reduce == "mean":
            out = out / degree.clamp(min=1).to(compute.dtype).reshape((m,) + (1,) * (compute.dim() - 1))
    else:
        init = -float("inf") if reduce == "max" else float("inf")
        out = torch.full(shape, init, dtype=compute.dtype)
        idx = rows.reshape((-1,) + (1,) * (compute.dim() - 1)).expand_as(compute)
        out.scatter_reduce_(0, idx, compute, "amax" if reduce == "max" else "amin", include_self=True)
        out[degree == 0] = 0
    return out.to(values.dtype)


def csr_spmm_sum_vectorised(ptr, col, value, mat, edge_chunk=1 << 20):
    """Weighted CSR SpMM-sum in the value dtype the way the reference's vectorised goldens do it: gather the source
    rows of a run of edges, scale them, `index_add_` them into the output rows (test/spmm_sum/arch22/golden.py:13-22,
    test/unified_spmm/arch22/golden.py:42-49).  Edges are processed in chunks so the gathered block stays bounded;
    this is the function the benchmark times as the CPU baseline.  `mat` is [N, K]; returns [rows, K] in mat's dtype.
    """
    ptr = ptr.to(torch.int64)
    rows_total = ptr.numel() - 1
    edges = col.numel()
    rows = edge_rows(ptr, edges)
    out = torch.zeros((rows_total, mat.size(-1)), dtype=mat.dtype)
    for start in range(0, edges, edge_chunk):
        stop = min(start + edge_chunk, edges)
        block = mat.index_select(0, col[start:stop].long())
        if value is not None:
            block.mul_(value[start:stop].reshape(-1, 1).to(mat.dtype))
        out.index_add_(0, rows[start:stop], block)
    return out
