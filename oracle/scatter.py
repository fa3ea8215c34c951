"""Oracle of `scatter` (unsorted index).  Test infrastructure; see the package docstring.

Follows `scatter_cpu` of the reference's test/scatter/arch35/golden.py:127-143 and `_reference_forward` of
python/ops_gnn/scatter.py:320-335: elements are applied in source order along `dim`; sum/mul/mean accumulate in the
value dtype; integer mean is a floor division by the count (narrow dtypes wrap the count and clamp it to at least 1);
min/max start from the dtype extremes (or from `out`), a later element wins ties (`<=` / `>=`), `arg` is the winning
source position and `src.size(dim)` where nothing won; without `out`, positions nothing reached are 0.
"""
import math

import torch

_NARROW = (torch.uint8, torch.int8, torch.int16)


def scatter_oracle(src, index, dim=-1, out=None, dim_size=None, reduce="sum"):
    src, index = src.cpu(), index.cpu().long()
    dim = dim % src.dim()
    if index.dim() == 1 and src.dim() > 1:
        view = [1] * src.dim()
        view[dim] = index.numel()
        index = index.reshape(view)
    index = index.expand_as(src) if index.shape != src.shape else index
    if dim_size is None:
        dim_size = out.size(dim) if out is not None else (int(index.max()) + 1 if index.numel() else 0)
    shape = list(src.shape)
    shape[dim] = dim_size
    before, length, after = math.prod(src.shape[:dim]), src.size(dim), math.prod(src.shape[dim + 1:])
    s3 = src.reshape(before, length, after)
    i3 = index.reshape(before, length, after)
    dtype = src.dtype
    floating = dtype.is_floating_point
    wide = torch.float64 if floating else torch.int64
    info = torch.finfo(dtype) if floating else torch.iinfo(dtype)
    if out is not None:
        result = out.cpu().clone().contiguous().reshape(before, dim_size, after)
    elif reduce == "mul":
        result = torch.ones((before, dim_size, after), dtype=dtype)
    elif reduce == "min":
        result = torch.full((before, dim_size, after), info.max, dtype=dtype)
    elif reduce == "max":
        result = torch.full((before, dim_size, after), info.min, dtype=dtype)
    else:
        result = torch.zeros((before, dim_size, after), dtype=dtype)
    arg = torch.full((before, dim_size, after), length, dtype=torch.int64)
    if src.numel() == 0 or result.numel() == 0:
        full = result.reshape(shape)
        return (full, arg.reshape(shape)) if reduce in ("min", "max") else full
    if reduce in ("sum", "add", "mean"):
        total = result.to(wide).scatter_add(1, i3, s3.to(wide))
        if reduce == "mean":
            count = torch.zeros((before, dim_size, after), dtype=torch.int64).scatter_add(1, i3, torch.ones_like(i3))
            if floating:
                total = torch.where(count > 0, total / count.clamp(min=1).to(wide), total)
            else:
                denominator = count.to(dtype).clamp(min=1).to(torch.int64) if dtype in _NARROW else count.clamp(min=1)
                total = torch.where(count > 0, torch.div(total.to(dtype).to(torch.int64), denominator,
                                                          rounding_mode="floor"), total)
        result = total.to(dtype)
    elif reduce == "mul":
        result = result.to(wide).scatter_reduce(1, i3, s3.to(wide), "prod", include_self=True).to(dtype)
    else:
        is_min = reduce == "min"
        start = result.clone()
        bar = start.gather(1, i3)
        valid = (s3 <= bar) if is_min else (s3 >= bar)
        fill = info.max if is_min else info.min
        if floating:
            fill = float("inf") if is_min else -float("inf")
        masked = torch.where(valid, s3, torch.full_like(s3, fill))
        best = torch.full_like(start, fill).scatter_reduce(1, i3, masked, "amin" if is_min else "amax",
                                                           include_self=True)
        position = torch.arange(length, dtype=torch.int64).reshape(1, length, 1).expand_as(i3)
        hit = valid & (s3 == best.gather(1, i3))
        last = torch.full_like(arg, -1).scatter_reduce(1, i3, torch.where(hit, position, torch.full_like(position, -1)),
                                                       "amax", include_self=True)
        won = last >= 0
        result = torch.where(won, best, start)
        arg = torch.where(won, last, arg)
        if out is None:
            result = torch.where(won, result, torch.zeros_like(result))
    full = result.reshape(shape)
    return (full, arg.reshape(shape)) if reduce in ("min", "max") else full
