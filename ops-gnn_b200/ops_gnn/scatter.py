"""torch_scatter-compatible ``scatter`` with an unsorted index: ``ops_gnn.scatter`` and its per-reduction aliases.

API of python/ops_gnn/scatter.py:603-674 in ops-gnn: ``scatter(src, index, dim=-1, out=None, dim_size=None,
reduce="sum")`` with ``reduce`` in ``sum/add/mul/mean/min/max``; ``scatter_min`` / ``scatter_max`` return
``(out, arg)``.  ``index`` (int64) follows torch_scatter's broadcasting: a 1-D index runs along ``dim``, anything else
is expanded to ``src``'s shape.  Semantics kept from the reference: elements are applied as if in source order, so a
later element wins min/max ties and ``arg`` is its position (``src.size(dim)`` where nothing was written); without
``out`` untouched positions are 0; integer ``mean`` is a floor division and 8/16-bit dtypes wrap the count into their
own range (at least 1); an index outside ``[0, out.size(dim))`` raises ``IndexError`` before anything is launched.

Every dtype, float64 and int64 included, runs on the GPU (the reference sends those two to a synchronous CPU
fallback); CPU tensors are rejected because this build has no CPU path.
"""
from __future__ import annotations

import weakref
from typing import NamedTuple, Optional, Tuple

import torch

from . import _pybind

_DTYPES = (torch.float16, torch.bfloat16, torch.float32, torch.float64, torch.int8, torch.int16, torch.int32,
           torch.int64, torch.uint8)
_REDUCE_CODE = {"sum": 0, "add": 0, "mul": 1, "mean": 2, "min": 3, "max": 4}
_BOUNDS_CACHE = {}
_BOUNDS_CACHE_LIMIT = 256


class _Request(NamedTuple):
    dim: int
    out: Optional[torch.Tensor]
    dim_size: Optional[int]
    reduce: str


def native_available() -> bool:
    """The CUDA extension is a hard requirement of this build, so importing the package already proved it."""
    return True


def broadcast(src: torch.Tensor, other: torch.Tensor, dim: int) -> torch.Tensor:
    """Expand ``src`` to ``other``'s shape with torch_scatter's rule: a 1-D tensor lies along ``dim``."""
    if dim < 0:
        dim += other.dim()
    if src.dim() == 1:
        src = src.reshape((1,) * dim + (-1,))
    src = src.reshape(tuple(src.shape) + (1,) * (other.dim() - src.dim()))
    return src.expand(other.size())


def _index_bounds(index: torch.Tensor) -> Tuple[int, int]:
    """Exact (min, max) of the index: one fused kernel and one small read, remembered per tensor version."""
    if index.numel() == 0:
        return 0, -1
    try:
        version = index._version
    except RuntimeError:  # inference tensors carry no version counter
        version = None
    key = id(index)
    if version is not None:
        hit = _BOUNDS_CACHE.get(key)
        if hit is not None and hit[0]() is index and hit[1] == version:
            return hit[2], hit[3]
    low, high, _ = _pybind.index_stats(index.contiguous()).tolist()
    if version is not None:
        if len(_BOUNDS_CACHE) >= _BOUNDS_CACHE_LIMIT:
            for stale in [k for k, v in _BOUNDS_CACHE.items() if v[0]() is None]:
                _BOUNDS_CACHE.pop(stale, None)
            if len(_BOUNDS_CACHE) >= _BOUNDS_CACHE_LIMIT:
                _BOUNDS_CACHE.pop(next(iter(_BOUNDS_CACHE)))
        _BOUNDS_CACHE[key] = (weakref.ref(index), version, low, high)
    return low, high


def _check(src, index, request: _Request) -> int:
    if not isinstance(src, torch.Tensor) or not isinstance(index, torch.Tensor):
        raise TypeError("src and index must be torch.Tensor instances")
    if not isinstance(request.dim, int) or isinstance(request.dim, bool):
        raise TypeError("dim must be an int")
    if not 1 <= src.dim() <= 8:
        raise ValueError("src must have between 1 and 8 dimensions")
    if not -src.dim() <= request.dim < src.dim():
        raise IndexError(
            f"Dimension out of range (expected to be in range of [-{src.dim()}, {src.dim() - 1}], but got {request.dim})")
    if index.dtype != torch.int64:
        raise TypeError(f"index must have dtype torch.int64, got {index.dtype}")
    if src.dtype not in _DTYPES:
        raise TypeError(
            "src dtype must be one of float16, bfloat16, float32, float64, int8, int16, int32, int64, or uint8")
    if src.device != index.device:
        raise ValueError("src and index must be on the same device")
    if src.device.type != "cuda":
        raise RuntimeError("ops_gnn.scatter requires CUDA tensors (this build has no CPU path)")
    if request.dim_size is not None:
        if not isinstance(request.dim_size, int) or isinstance(request.dim_size, bool):
            raise TypeError("dim_size must be an int or None")
        if request.dim_size < 0:
            raise ValueError("dim_size must be non-negative")
    return request.dim % src.dim()


def _initial_output(src: torch.Tensor, reduce: str, shape) -> torch.Tensor:
    if src.numel() == 0 or reduce in ("sum", "add", "mean"):
        return torch.zeros(shape, dtype=src.dtype, device=src.device)
    if reduce == "mul":
        return torch.ones(shape, dtype=src.dtype, device=src.device)
    info = torch.finfo(src.dtype) if src.dtype.is_floating_point else torch.iinfo(src.dtype)
    return torch.full(shape, info.max if reduce == "min" else info.min, dtype=src.dtype, device=src.device)


def _scatter_forward(src: torch.Tensor, index: torch.Tensor, request: _Request):
    dim = _check(src, index, request)
    if (request.out is None and request.reduce in ("min", "max") and dim == 0 and index.dim() == 1 and index.dtype == torch.int64
            and src.dtype in (torch.float32, torch.float16, torch.bfloat16) and index.numel() == src.size(0) and src.numel() > 0
            and src.is_contiguous() and index.is_contiguous()):
        # Extrema over a 1-D index along the leading dimension: sorted once (a stable argsort the planner caches with the
        # index's other facts) and reduced by the CSR engine, no atomics.  Nothing between the two native calls is a tensor
        # operation, so back-to-back calls reuse the permutation.
        low, high, _, _ = _pybind.index_facts(index, True)
        if low < 0:
            raise IndexError(f"index contains a negative value ({low})")
        length = high + 1 if request.dim_size is None else request.dim_size
        if high >= length:
            raise IndexError(f"index value {high} is out of bounds for output size {length} at dimension {dim}")
        done = _pybind.scatter_extremum_sorted(src, index, length, request.reduce == "min")
        if done is not None:
            return done
    try:
        expanded = broadcast(index, src, dim)
    except RuntimeError as exc:
        raise ValueError(
            f"index with shape {tuple(index.shape)} cannot broadcast to src shape {tuple(src.shape)} at dim={dim}"
        ) from exc
    low, high = _index_bounds(index) if expanded.numel() > 0 else (0, -1)
    if low < 0:
        raise IndexError(f"index contains a negative value ({low})")

    out = request.out
    if out is None:
        length = request.dim_size
        if length is None:
            length = 0 if expanded.numel() == 0 else high + 1
        shape = list(src.shape)
        shape[dim] = length
        work = _initial_output(src, request.reduce, shape)
    else:
        if not isinstance(out, torch.Tensor):
            raise TypeError("out must be a torch.Tensor or None")
        if out.dtype != src.dtype:
            raise TypeError("out dtype must match src dtype")
        if out.device != src.device:
            raise ValueError("out must be on the same device as src")
        if out.dim() != src.dim():
            raise ValueError("out and src must have the same rank")
        if any(axis != dim and out.size(axis) != src.size(axis) for axis in range(src.dim())):
            raise ValueError("out shape must match src outside the scatter dim")
        length = out.size(dim)
        work = out if out.is_contiguous() else out.contiguous()
    if high >= length:
        raise IndexError(f"index value {high} is out of bounds for output size {length} at dimension {dim}")

    source = src.contiguous()
    labels = index.contiguous() if index.dim() == 1 else expanded.contiguous()
    if out is not None:
        if source.data_ptr() == work.data_ptr():
            source = source.clone()
        if labels.data_ptr() == work.data_ptr():
            labels = labels.clone()
    result, arg = _pybind.scatter_forward(source, labels, dim, work, _REDUCE_CODE[request.reduce], out is not None)
    if out is not None and result is not out and result.data_ptr() != out.data_ptr():
        out.copy_(result)
        result = out
    elif out is not None:
        result = out
    return result, (arg if request.reduce in ("min", "max") else None)


def scatter_sum(src: torch.Tensor, index: torch.Tensor, dim: int = -1, out: Optional[torch.Tensor] = None,
                dim_size: Optional[int] = None) -> torch.Tensor:
    return _scatter_forward(src, index, _Request(dim, out, dim_size, "sum"))[0]


def scatter_add(src: torch.Tensor, index: torch.Tensor, dim: int = -1, out: Optional[torch.Tensor] = None,
                dim_size: Optional[int] = None) -> torch.Tensor:
    return scatter_sum(src, index, dim, out, dim_size)


def scatter_mul(src: torch.Tensor, index: torch.Tensor, dim: int = -1, out: Optional[torch.Tensor] = None,
                dim_size: Optional[int] = None) -> torch.Tensor:
    return _scatter_forward(src, index, _Request(dim, out, dim_size, "mul"))[0]


def scatter_mean(src: torch.Tensor, index: torch.Tensor, dim: int = -1, out: Optional[torch.Tensor] = None,
                 dim_size: Optional[int] = None) -> torch.Tensor:
    return _scatter_forward(src, index, _Request(dim, out, dim_size, "mean"))[0]


def scatter_min(src: torch.Tensor, index: torch.Tensor, dim: int = -1, out: Optional[torch.Tensor] = None,
                dim_size: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    return _scatter_forward(src, index, _Request(dim, out, dim_size, "min"))


def scatter_max(src: torch.Tensor, index: torch.Tensor, dim: int = -1, out: Optional[torch.Tensor] = None,
                dim_size: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    return _scatter_forward(src, index, _Request(dim, out, dim_size, "max"))


def scatter(src: torch.Tensor, index: torch.Tensor, dim: int = -1, out: Optional[torch.Tensor] = None,
            dim_size: Optional[int] = None, reduce: str = "sum") -> torch.Tensor:
    """``torch_scatter.scatter(src, index, dim, out, dim_size, reduce)`` on CUDA tensors; values only."""
    if reduce not in _REDUCE_CODE:
        raise ValueError("reduce must be one of 'sum', 'add', 'mul', 'mean', 'min', or 'max'")
    return _scatter_forward(src, index, _Request(dim, out, dim_size, reduce))[0]
