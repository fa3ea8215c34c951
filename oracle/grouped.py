"""Oracle of the grouped softmax family.  Test infrastructure; see the package docstring.

`grouped_softmax_oracle` follows `grouped_reference` of the reference's test/common/grouped_softmax_golden.py:50-63:
`torch.softmax` / `torch.log_softmax` over the members of every group of an unsorted 1-D index along `dim`, in
float64.  `grouped_logsumexp_oracle` follows `grouped_logsumexp_reference` (:66-86): one row per (batch, group), a
group without members is -inf.  Special values behave as the torch operators do: a group holding +inf gives NaN for
softmax, a group of only -inf gives NaN; logsumexp gives +inf / -inf for those groups; NaN spreads over its group.
"""
import torch


def _prepare(src, index, dim, dim_size):
    index = torch.as_tensor(index).cpu().to(torch.int64).reshape(-1)
    values = src.cpu().to(torch.float64)
    dim = dim + values.dim() if dim < 0 else dim
    groups = int(dim_size) if dim_size is not None else (int(index.max()) + 1 if index.numel() else 0)
    moved = values.movedim(dim, 0).contiguous()
    return index, moved, dim, groups


def _group_max_sum(index, moved, groups):
    flat = moved.reshape(moved.size(0), -1)
    k = flat.size(1)
    spread = index.reshape(-1, 1).expand(-1, k)
    top = torch.full((groups, k), -float("inf"), dtype=torch.float64)
    if flat.numel():
        top = top.scatter_reduce(0, spread, flat, "amax", include_self=True)
    return flat, spread, top


def grouped_softmax_oracle(src, index, dim=0, dim_size=None, log=False):
    index, moved, dim, groups = _prepare(src, index, dim, dim_size)
    flat, spread, top = _group_max_sum(index, moved, groups)
    if flat.numel() == 0:
        return src.cpu().to(torch.float64).clone()
    shifted = flat - top[index]              # +inf - +inf and -inf - -inf are NaN, as in torch.softmax
    total = torch.zeros_like(top).index_add_(0, index, torch.exp(shifted))
    result = shifted - torch.log(total[index]) if log else torch.exp(shifted) / total[index]
    return result.reshape(moved.shape).movedim(0, dim)


def grouped_logsumexp_oracle(src, index, dim=0, dim_size=None):
    index, moved, dim, groups = _prepare(src, index, dim, dim_size)
    flat, spread, top = _group_max_sum(index, moved, groups)
    shift = torch.where(torch.isfinite(top), top, torch.zeros_like(top))
    total = torch.zeros_like(top)
    if flat.numel():
        total.index_add_(0, index, torch.exp(flat - shift[index]))
    result = shift + torch.log(total)
    return result.reshape((groups,) + tuple(moved.shape[1:])).movedim(0, dim)
