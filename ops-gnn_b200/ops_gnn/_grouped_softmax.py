"""Shared front-end of ``scatter_softmax``, ``scatter_log_softmax`` and ``scatter_logsumexp``.

The three operators take ``(src, index, dim=0, dim_size=None)``: ``src`` is fp16 / fp32 / bf16 on a CUDA device,
``index`` a 1-D int32 / int64 group label per position along ``dim``, not necessarily sorted.  They validate the same
way and raise the same exception types as the reference front-end (python/ops_gnn/_grouped_softmax.py:33-155 of
ops-gnn).  Differences that matter on the GPU: the index keeps its width (no narrowing copy), and negative labels,
the largest label and sortedness come from ONE statistics kernel with a single small read instead of two reductions.
"""
from typing import Optional, Tuple

import torch

from . import _pybind

SUPPORTED_DTYPES = (torch.float16, torch.float32, torch.bfloat16)
SUPPORTED_INDEX_DTYPES = (torch.int32, torch.int64)
_INT32_MAX = 2 ** 31 - 1


def normalize_dim(dim: int, rank: int) -> int:
    if not isinstance(dim, int) or isinstance(dim, bool):
        raise TypeError(f"dim must be an int, got {type(dim).__name__}")
    if not -rank <= dim < rank:
        raise IndexError(
            f"Dimension out of range (expected to be in range of [-{rank}, {rank - 1}], but got {dim})")
    return dim % rank


def check_inputs(op: str, src: torch.Tensor, index: torch.Tensor, dim: int) -> None:
    if src.dim() < 1:
        raise ValueError("src must have at least one dimension")
    if index.dim() != 1:
        raise ValueError(f"index must be 1-D, got {index.dim()}-D")
    if src.dtype not in SUPPORTED_DTYPES:
        raise TypeError(f"src dtype must be one of float16, float32, bfloat16; got {src.dtype}")
    if index.dtype not in SUPPORTED_INDEX_DTYPES:
        raise TypeError(f"index dtype must be int32 or int64, got {index.dtype}")
    if src.device != index.device:
        raise ValueError(f"src and index must be on the same device, got {src.device} and {index.device}")
    if src.device.type != "cuda":
        raise RuntimeError(f"{op} requires CUDA tensors")
    if index.numel() != src.size(dim):
        raise ValueError(f"index length ({index.numel()}) must match src.size({dim}) ({src.size(dim)})")


def index_bounds(index: torch.Tensor) -> Tuple[int, int]:
    """(minimum, maximum) of a non-empty index.  One device pass whose facts (range, sortedness, largest group) the
    native planner reuses a moment later, as long as no other tensor operation runs in between."""
    labels = index if index.is_contiguous() else index.contiguous()
    low, high, _, _ = _pybind.index_facts(labels, True)
    return low, high


def resolve_groups(index: torch.Tensor, dim_size: Optional[int]) -> int:
    """Validate ``dim_size`` and the index range; return the number of groups."""
    if dim_size is not None:
        if not isinstance(dim_size, int) or isinstance(dim_size, bool):
            raise TypeError(f"dim_size must be an int, got {type(dim_size).__name__}")
        if dim_size < 0:
            raise ValueError(f"dim_size must be non-negative, got {dim_size}")
        if dim_size > _INT32_MAX:
            raise ValueError(f"dim_size must fit the int32 index range, got {dim_size}")
    if index.numel() == 0:
        return 0 if dim_size is None else dim_size
    low, high = index_bounds(index)
    groups = high + 1 if dim_size is None else dim_size
    if low < 0:
        raise ValueError("index must be non-negative")
    if high >= groups:
        raise ValueError(f"index values must be smaller than dim_size ({groups})")
    return groups


def build_autograd(op_name: str):
    """Autograd bridge of one same-shape operator: ``<op_name>_forward`` / ``<op_name>_backward`` of the extension.

    The backward of both softmax flavours needs only the forward output and the index; the grouped Jacobian is
    applied by the device kernel.
    """
    forward = getattr(_pybind, f"{op_name}_forward")
    backward = getattr(_pybind, f"{op_name}_backward")

    class _Grouped(torch.autograd.Function):
        @staticmethod
        def forward(ctx, src, index, dim, groups):
            labels = index.contiguous()
            out = torch.zeros_like(src) if src.numel() == 0 else forward(src.contiguous(), labels, dim, groups)
            ctx.dim, ctx.groups = dim, groups
            ctx.save_for_backward(out, labels)
            return out

        @staticmethod
        def backward(ctx, grad_out):
            out, labels = ctx.saved_tensors
            upstream = grad_out.contiguous()
            if out.numel() == 0:
                return torch.zeros_like(upstream), None, None, None
            return backward(out, upstream, labels, ctx.dim, ctx.groups), None, None, None

    _Grouped.native_name = op_name
    _Grouped.__name__ = _Grouped.__qualname__ = f"_{op_name}"
    return _Grouped


def run(op: str, function, src, index, dim: int, dim_size: Optional[int]) -> torch.Tensor:
    if not isinstance(src, torch.Tensor):
        raise TypeError(f"src must be a torch.Tensor, got {type(src).__name__}")
    if not isinstance(index, torch.Tensor):
        raise TypeError(f"index must be a torch.Tensor, got {type(index).__name__}")
    dim = normalize_dim(dim, src.dim())
    check_inputs(op, src, index, dim)
    groups = resolve_groups(index, dim_size)
    if not (torch.is_grad_enabled() and src.requires_grad) and src.numel() and src.is_contiguous() and index.is_contiguous():
        # Nothing to differentiate: call the planner directly.  (An autograd node or a needless `.contiguous()` is a
        # tensor operation, and any tensor operation makes the planner re-derive the index facts cached just above.)
        return getattr(_pybind, f"{function.native_name}_forward")(src, index, dim, groups)
    return function.apply(src, index, dim, groups)
