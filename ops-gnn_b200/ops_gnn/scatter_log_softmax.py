"""Grouped log-softmax along one dimension: ``ops_gnn.scatter_log_softmax`` (python/ops_gnn/scatter_log_softmax.py of
ops-gnn; torch_scatter.composite.scatter_log_softmax semantics)."""
from typing import Optional

import torch

from . import _grouped_softmax

_FUNCTION = _grouped_softmax.build_autograd("scatter_log_softmax")


def scatter_log_softmax(src: torch.Tensor, index: torch.Tensor, dim: int = 0,
                        dim_size: Optional[int] = None) -> torch.Tensor:
    """``out[i] = src[i] - log(sum_{j: index[j] == index[i]} exp(src[j]))`` along ``dim``, computed in fp32.

    Arguments, result shape, special values and exceptions are those of :func:`ops_gnn.scatter_softmax`.
    """
    return _grouped_softmax.run("scatter_log_softmax", _FUNCTION, src, index, dim, dim_size)
