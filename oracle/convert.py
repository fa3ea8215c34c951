"""Oracle of the index conversions.  Test infrastructure; see the package docstring.

`ind2ptr_oracle` / `ptr2ind_oracle` give the results of `ind2ptr_cpu` / `ptr2ind_cpu` in the reference's
test/sparse/arch35/golden.py:14-51 (ptr[i] = number of sorted entries smaller than i; every edge of row i maps to i,
edges past ptr[-1] stay 0) with `searchsorted` / `repeat_interleave` instead of Python loops.
"""
import torch


def ind2ptr_oracle(ind, num_rows):
    ind = ind.cpu().to(torch.int64)
    if ind.numel() == 0:
        return torch.zeros(num_rows + 1, dtype=torch.int64)
    return torch.searchsorted(ind, torch.arange(num_rows + 1, dtype=torch.int64), right=False)


def ptr2ind_oracle(ptr, num_edges):
    ptr = ptr.cpu().to(torch.int64)
    counts = ptr[1:] - ptr[:-1]
    rows = torch.repeat_interleave(torch.arange(counts.numel(), dtype=torch.int64), counts)
    out = torch.zeros(num_edges, dtype=torch.int64)
    start = int(ptr[0]) if ptr.numel() else 0
    n = min(rows.numel(), max(num_edges - start, 0))
    out[start:start + n] = rows[:n]
    return out
