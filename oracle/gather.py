"""Oracle of `gather_csr` / `gather_coo`.  Test infrastructure; see the package docstring.

Follows `gather_csr_cpu` and `gather_csr_coo_cpu` of the reference's test/gather_csr/arch35/golden.py:61-110: the segment
dimension is `indptr.dim() - 1`, `indptr` broadcasts over the leading dimensions, output row `e` of a batch copies the
segment `s` with `indptr[s] <= e < indptr[s + 1]`, rows before `indptr[0]` stay zero and the output has `indptr[-1]`
rows; `gather_coo` is the same copy driven by an explicit (sorted) row index.
"""
import math

import torch


def gather_coo_oracle(src, index):
    src, index = src.cpu(), index.cpu().long()
    dim = index.dim() - 1
    batches = math.prod(src.shape[:dim])
    features = math.prod(src.shape[dim + 1:])
    flat = src.contiguous().reshape(batches, src.size(dim), features)
    picks = index.contiguous().reshape(batches, index.size(dim))
    out = torch.gather(flat, 1, picks.unsqueeze(-1).expand(batches, picks.size(1), features)) if picks.numel() else \
        flat.new_zeros((batches, picks.size(1), features))
    shape = list(src.shape)
    shape[dim] = index.size(dim)
    return out.reshape(shape)


def gather_csr_oracle(src, indptr):
    src, indptr = src.cpu(), indptr.cpu().long()
    dim = indptr.dim() - 1
    shape = list(src.shape)
    if src.numel() == 0 or indptr.size(-1) == 0:
        shape[dim] = int(indptr.flatten()[-1]) if indptr.numel() else 0
        return torch.zeros(shape, dtype=src.dtype)
    expanded = list(indptr.shape)
    for axis in range(dim):
        expanded[axis] = src.size(axis)
    ptr = indptr.expand(expanded).contiguous().reshape(-1, indptr.size(-1))
    rows = int(ptr[0, -1])
    position = torch.arange(rows).unsqueeze(0).expand(ptr.size(0), rows).contiguous()
    segment = torch.searchsorted(ptr, position, right=True) - 1          # -1 before ptr[0]
    covered = (segment >= 0) & (segment < src.size(dim))
    features = math.prod(src.shape[dim + 1:])
    flat = src.contiguous().reshape(ptr.size(0), src.size(dim), features)
    picked = torch.gather(flat, 1, segment.clamp(0, src.size(dim) - 1).unsqueeze(-1).expand(-1, -1, features))
    out = torch.where(covered.unsqueeze(-1), picked, torch.zeros((), dtype=src.dtype))
    shape[dim] = rows
    return out.reshape(shape)
