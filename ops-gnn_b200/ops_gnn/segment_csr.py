"""torch_scatter-compatible ``segment_csr`` family (python/ops_gnn/segment_csr.py:35-91 of ops-gnn).

Signatures match ``torch_scatter.segment_csr``; there is no ``dim_size`` because the pointers define the segment
count.  Reduction runs along ``dim = indptr.dim() - 1``.
"""
from typing import Optional, Tuple

import torch

from . import _pybind

_REDUCE_OPS = ("sum", "add", "mean", "min", "max")


def _check_reduce(reduce: str) -> None:
    if reduce not in _REDUCE_OPS:
        raise ValueError(f"reduce value '{reduce}' is not valid (use one of {_REDUCE_OPS})")


def segment_sum_csr(src: torch.Tensor, indptr: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _pybind.segment_csr_value(src, indptr, out, "sum")


def segment_add_csr(src: torch.Tensor, indptr: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _pybind.segment_csr_value(src, indptr, out, "add")


def segment_mean_csr(src: torch.Tensor, indptr: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _pybind.segment_csr_value(src, indptr, out, "mean")


def segment_min_csr(src: torch.Tensor, indptr: torch.Tensor,
                    out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    result = _pybind.segment_csr(src, indptr, out, "min")
    return result[0], result[1]


def segment_max_csr(src: torch.Tensor, indptr: torch.Tensor,
                    out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Return per-segment maxima and the first position that attains them (``src.size(dim)`` for empty segments)."""
    result = _pybind.segment_csr(src, indptr, out, "max")
    return result[0], result[1]


def segment_csr(src: torch.Tensor, indptr: torch.Tensor, out: Optional[torch.Tensor] = None,
                reduce: str = "sum") -> torch.Tensor:
    """Reduce CSR segments and return values only; min/max positions come from the sub-operators."""
    _check_reduce(reduce)
    return _pybind.segment_csr_value(src, indptr, out, reduce)
