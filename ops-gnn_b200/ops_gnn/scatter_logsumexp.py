"""Grouped log-sum-exp along one dimension: ``ops_gnn.scatter_logsumexp`` (python/ops_gnn/scatter_logsumexp.py:76-127
of ops-gnn).

The output is reduced: ``src.size(dim)`` is replaced by the number of groups.  A group without members, or made only
of ``-inf``, is ``-inf``; a group that holds ``+inf`` is ``+inf``; NaN spreads over its group.  The gradient is
``grad_out[group] * exp(src - out[group])``, read from the saved source and the reduced output.
"""
from typing import Optional

import torch

from . import _pybind
from ._grouped_softmax import check_inputs, normalize_dim, resolve_groups


class _ScatterLogSumExp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, src, index, dim, groups):
        labels, source = index.contiguous(), src.contiguous()
        out = _pybind.scatter_logsumexp_forward(source, labels, dim, groups)
        ctx.dim, ctx.groups = dim, groups
        ctx.save_for_backward(source, out, labels)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        source, out, labels = ctx.saved_tensors
        grad = _pybind.scatter_logsumexp_backward(source, out, grad_out.contiguous(), labels, ctx.dim, ctx.groups)
        return grad, None, None, None


def scatter_logsumexp(src: torch.Tensor, index: torch.Tensor, dim: int = 0,
                      dim_size: Optional[int] = None) -> torch.Tensor:
    """``out[g] = log(sum_{j: index[j] == g} exp(src[j]))`` along ``dim`` for fp16 / fp32 / bf16 CUDA tensors.

    ``index`` is a 1-D int32/int64 label per position along ``dim``; ``dim_size`` defaults to ``index.max() + 1`` and
    may be larger to leave empty groups (``-inf``).  Raises ``TypeError`` / ``ValueError`` / ``IndexError`` for bad
    arguments and ``RuntimeError`` for tensors that are not on a CUDA device.
    """
    if not isinstance(src, torch.Tensor):
        raise TypeError(f"src must be a torch.Tensor, got {type(src).__name__}")
    if not isinstance(index, torch.Tensor):
        raise TypeError(f"index must be a torch.Tensor, got {type(index).__name__}")
    dim = normalize_dim(dim, src.dim())
    check_inputs("scatter_logsumexp", src, index, dim)
    groups = resolve_groups(index, dim_size)
    if not (torch.is_grad_enabled() and src.requires_grad) and src.numel() and src.is_contiguous() and index.is_contiguous():
        # Nothing to differentiate: call the planner directly.  (An autograd node or a needless `.contiguous()` is a
        # tensor operation, and any tensor operation makes the planner re-derive the index facts cached just above.)
        return _pybind.scatter_logsumexp_forward(src, index, dim, groups)
    return _ScatterLogSumExp.apply(src, index, dim, groups)
