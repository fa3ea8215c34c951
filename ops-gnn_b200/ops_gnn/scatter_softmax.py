"""Grouped softmax along one dimension: ``ops_gnn.scatter_softmax`` (python/ops_gnn/scatter_softmax.py:46-75 of
ops-gnn; torch_scatter.composite.scatter_softmax semantics)."""
from typing import Optional

import torch

from . import _grouped_softmax

_FUNCTION = _grouped_softmax.build_autograd("scatter_softmax")


def scatter_softmax(src: torch.Tensor, index: torch.Tensor, dim: int = 0,
                    dim_size: Optional[int] = None) -> torch.Tensor:
    """``out[i] = exp(src[i]) / sum_{j: index[j] == index[i]} exp(src[j])`` along ``dim``, computed in fp32.

    ``index`` is a 1-D int32/int64 label per position along ``dim`` (any order); ``dim_size`` defaults to
    ``index.max() + 1``.  The result has ``src``'s shape and dtype and is differentiable.  A group that holds
    ``+inf`` or only ``-inf`` is NaN, as with ``torch.softmax``.  Raises ``TypeError`` / ``ValueError`` /
    ``IndexError`` for bad arguments and ``RuntimeError`` for tensors that are not on a CUDA device.
    """
    return _grouped_softmax.run("scatter_softmax", _FUNCTION, src, index, dim, dim_size)
