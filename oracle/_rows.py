"""Shared helpers of the oracle: row ids of CSR edges and first-winner extremum reduction along dim 0."""
import torch


def edge_rows(ptr: torch.Tensor, edges: int) -> torch.Tensor:
    """Row id of every edge of a CSR pointer array (int64, CPU)."""
    ptr = ptr.to(torch.int64)
    counts = ptr[1:] - ptr[:-1]
    return torch.repeat_interleave(torch.arange(counts.numel(), dtype=torch.int64), counts, output_size=edges)


def first_extremum(values: torch.Tensor, rows: torch.Tensor, row_count: int, is_min: bool, valid: torch.Tensor,
                   none: int, positions: torch.Tensor = None):
    """Per-row extremum of `values[E, ...]` grouped by `rows[E]`, restricted to `valid` entries.

    Returns (value, arg): the extremum over the valid entries of each row and the position (default: edge id) of its
    first occurrence; rows without a valid entry give (0, none).
    """
    e = values.size(0)
    shape = (row_count,) + tuple(values.shape[1:])
    idx = rows.reshape((-1,) + (1,) * (values.dim() - 1)).expand_as(values)
    fill = float("inf") if is_min else -float("inf")
    if not values.dtype.is_floating_point:
        info = torch.iinfo(values.dtype)
        fill = info.max if is_min else info.min
    masked = torch.where(valid, values, torch.full_like(values, fill))
    best = torch.full(shape, fill, dtype=values.dtype)
    best = best.scatter_reduce(0, idx, masked, "amin" if is_min else "amax", include_self=True)
    if positions is None:
        positions = torch.arange(e, dtype=torch.int64)
    pos = positions.reshape((-1,) + (1,) * (values.dim() - 1)).expand_as(values)
    big = torch.iinfo(torch.int64).max
    hit = valid & (values == best.gather(0, idx))
    candidate = torch.where(hit, pos, torch.full_like(pos, big))
    arg = torch.full(shape, big, dtype=torch.int64).scatter_reduce(0, idx, candidate, "amin", include_self=True)
    found = arg != big
    value = torch.where(found, best, torch.zeros_like(best))
    arg = torch.where(found, arg, torch.full_like(arg, none))
    return value, arg
