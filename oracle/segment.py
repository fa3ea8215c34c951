"""Oracle of the segment reductions.  Test infrastructure; see the package docstring.

`segment_csr_oracle` follows `segment_csr_cpu` / `segment_argminmax_cpu` of the reference's
test/segment_csr/arch35/golden.py:67-103: reduction along `indptr.dim() - 1`, pointers broadcast over leading
dimensions, segment ends clamped to the source length, empty segments give 0 and arg = source length, min/max are
`torch.min/max` (first occurrence, NaN propagates), float mean = typed sum / typed count in fp32, integer mean wraps
the count to the value dtype and truncates (zero count gives 0).

`segment_coo_oracle` follows `segment_coo_reference` of test/segment_coo/arch35/golden.py:42-161: sorted int64
index broadcast over leading dimensions; fp16/bf16 accumulate in fp32; without `out`, min/max start from the finite
dtype extreme, only strictly better values win (NaN never does), an unbeaten seed becomes 0 with arg = length; with
`out`, its contents seed the segments that receive elements (the segment that contains position 0 is seeded from
`out[..., 0, :]`, golden.py:131-133) and other segments keep their contents.

`segment_logsumexp_oracle` follows `reference` of test/segment_logsumexp/golden.py:25-43: float64 log-sum-exp per
CSR segment, empty segments are -inf, rows before indptr[0] are ignored.
"""
import math

import torch

from ._rows import first_extremum


def _typed_mean(total, counts):
    if total.is_floating_point():
        return total.float() / counts.to(total.dtype).float()
    count = counts.to(total.dtype)
    safe = torch.where(count != 0, count, torch.ones_like(count))
    return torch.where(count != 0, torch.div(total, safe, rounding_mode="trunc"), torch.zeros_like(total))


def _segment_ids(ptr, length):
    """Segment id of every source position (or -1) for one non-decreasing pointer row clamped to `length`."""
    ptr = ptr.clamp(max=length)
    position = torch.arange(length, dtype=torch.int64)
    seg = torch.searchsorted(ptr, position, right=True) - 1
    inside = (seg >= 0) & (seg < ptr.numel() - 1)
    return torch.where(inside, seg, torch.full_like(seg, -1))


def segment_csr_oracle(src, indptr, reduce="sum", return_arg=False):
    src, indptr = src.cpu(), indptr.cpu().long()
    dim = indptr.dim() - 1
    pointer_shape = list(src.shape[:dim]) + [indptr.size(-1)]
    pointers = indptr.expand(pointer_shape).contiguous().reshape(-1, indptr.size(-1))
    batches = math.prod(src.shape[:dim])
    length = src.size(dim)
    feat = math.prod(src.shape[dim + 1:])
    segments = indptr.size(-1) - 1
    out_shape = list(src.shape)
    out_shape[dim] = segments
    values = src.contiguous().reshape(batches, length, feat)
    out = torch.zeros((batches, segments, feat), dtype=src.dtype)
    arg = torch.full((batches, segments, feat), length, dtype=torch.int64)
    for b in range(batches):
        seg = _segment_ids(pointers[b], length)
        keep = seg >= 0
        rows, vals = seg[keep], values[b][keep]
        position = torch.arange(length, dtype=torch.int64)[keep]
        if rows.numel() == 0:
            continue
        if reduce in ("sum", "add", "mean"):
            wide = torch.float64 if src.is_floating_point() else torch.int64
            total = torch.zeros((segments, feat), dtype=wide).index_add_(0, rows, vals.to(wide)).to(src.dtype)
            if reduce == "mean":
                counts = torch.bincount(rows, minlength=segments).reshape(-1, 1).expand(-1, feat)
                mean = _typed_mean(total, counts.clamp(min=1)).to(src.dtype)
                total = torch.where(counts > 0, mean, torch.zeros_like(mean))
            out[b] = total
        else:
            is_min = reduce == "min"
            if src.is_floating_point():
                # torch.min/max: the first NaN of a segment wins; otherwise the first extremum.
                nan = torch.isnan(vals)
                nan_value, nan_arg = first_extremum(torch.zeros_like(vals), rows, segments, True, nan, length, position)
                clean_value, clean_arg = first_extremum(vals, rows, segments, is_min, ~nan, length, position)
                has_nan = nan_arg != length
                out[b] = torch.where(has_nan, torch.full_like(clean_value, float("nan")), clean_value)
                arg[b] = torch.where(has_nan, nan_arg, clean_arg)
            else:
                out[b], arg[b] = first_extremum(vals, rows, segments, is_min, torch.ones_like(vals, dtype=torch.bool),
                                                length, position)
    out, arg = out.reshape(out_shape), arg.reshape(out_shape)
    return (out, arg) if return_arg else out


def segment_coo_oracle(src, index, out=None, dim_size=None, reduce="sum", return_arg=False):
    src, index = src.cpu(), index.cpu()
    mode = "sum" if reduce == "add" else reduce
    dim = index.dim() - 1
    expanded = index.expand(src.shape[:index.dim()]).contiguous()
    length = src.size(dim)
    batches = math.prod(src.shape[:dim])
    feat = math.prod(src.shape[dim + 1:])
    if out is not None:
        segments = out.size(dim)
    elif dim_size is not None:
        segments = int(dim_size)
    else:
        segments = int(expanded.max()) + 1 if expanded.numel() else 0
    shape = list(src.shape)
    shape[dim] = segments
    has_out = out is not None
    result = torch.zeros(shape, dtype=src.dtype) if not has_out else out.cpu().clone().contiguous()
    args = torch.full(shape, length, dtype=torch.int64)
    res3 = result.reshape(batches, segments, feat)
    arg3 = args.reshape(batches, segments, feat)
    values = src.contiguous().reshape(batches, length, feat)
    rows_all = expanded.reshape(batches, length)
    dtype = src.dtype
    acc_dtype = torch.float32 if dtype in (torch.float16, torch.bfloat16) else dtype
    wide = torch.float64 if dtype.is_floating_point else torch.int64
    limits = torch.finfo(dtype) if dtype.is_floating_point else torch.iinfo(dtype)
    for b in range(batches):
        rows = rows_all[b]
        if rows.numel() == 0 or segments == 0:
            continue
        vals = values[b].to(acc_dtype)
        counts = torch.bincount(rows, minlength=segments)
        touched = (counts > 0).reshape(-1, 1).expand(-1, feat)
        seed = res3[b].clone()
        if has_out:
            seed[rows[0]] = res3[b][0]  # the segment holding position 0 is seeded from out[0]
        if mode in ("sum", "mean"):
            total = torch.zeros((segments, feat), dtype=wide).index_add_(0, rows, vals.to(wide))
            total = (total + seed.to(wide)) if has_out else total
            total = total.to(acc_dtype).to(dtype)
            if mode == "mean":
                divisor = counts.to(dtype).reshape(-1, 1).expand(-1, feat)
                if dtype.is_floating_point:
                    mean = (total / torch.where(touched, divisor, torch.ones_like(divisor))).to(dtype)
                else:
                    safe = torch.where(divisor != 0, divisor, torch.ones_like(divisor)).to(torch.int64)
                    mean = torch.div(total.to(torch.int64), safe, rounding_mode="trunc").to(dtype)
                    mean = torch.where(divisor != 0, mean, torch.zeros_like(mean))
                total = mean
            res3[b] = torch.where(touched, total, res3[b])
        else:
            is_min = mode == "min"
            if has_out:
                start = seed.to(acc_dtype)
            else:
                start = torch.full((segments, feat), limits.max if is_min else limits.min, dtype=dtype).to(acc_dtype)
            bar = start[rows]
            valid = (vals < bar) if is_min else (vals > bar)
            best, where = first_extremum(vals, rows, segments, is_min, valid, length)
            won = where != length
            merged = torch.where(won, best, start).to(dtype)
            if not has_out:
                merged = torch.where(won, merged, torch.zeros_like(merged))
            res3[b] = torch.where(touched, merged, res3[b])
            arg3[b] = torch.where(touched & won, where, torch.full_like(where, length))
    if return_arg and mode in ("min", "max"):
        return result, args
    return result


def segment_logsumexp_oracle(src, indptr):
    src, indptr = src.cpu(), torch.as_tensor(indptr).cpu().long()
    segments = indptr.numel() - 1
    feat_shape = tuple(src.shape[1:])
    flat = src.double().reshape(src.size(0), -1)
    seg = _segment_ids(indptr, src.size(0))
    keep = seg >= 0
    rows, vals = seg[keep], flat[keep]
    k = flat.size(1)
    top = torch.full((segments, k), -float("inf"), dtype=torch.float64)
    if rows.numel():
        top = top.scatter_reduce(0, rows.reshape(-1, 1).expand(-1, k), vals, "amax", include_self=True)
    shift = torch.where(torch.isfinite(top), top, torch.zeros_like(top))
    total = torch.zeros((segments, k), dtype=torch.float64)
    if rows.numel():
        total.index_add_(0, rows, torch.exp(vals - shift[rows]))
    return (shift + torch.log(total)).reshape((segments,) + feat_shape)
