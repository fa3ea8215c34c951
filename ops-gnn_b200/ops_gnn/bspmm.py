"""Batched CSR SpMM aggregation (python/ops_gnn/bspmm.py:15-28 of ops-gnn)."""
from typing import Optional

import torch

from .spmm import _SpmmRequest, _parse_call_options, _spmm


def bspmm(indptr: torch.Tensor, indices: torch.Tensor, x: Optional[torch.Tensor] = None, *args,
          **kwargs) -> torch.Tensor:
    """Generalized batched CSR aggregation: at least one feature tensor has rank three or higher.

    Trailing feature dimensions broadcast with missing dimensions inserted right after the item axis; message ops
    and reductions are those of :func:`ops_gnn.spmm`.  ``bspmm(indptr, indices, X[V, H, D], op="mul",
    rhs=alpha[E, H, 1])`` (attention-weighted aggregation) runs as one fused kernel.
    """
    op, reduce, out, rhs = _parse_call_options("bspmm", args, kwargs)
    return _spmm(_SpmmRequest(indptr, indices, x, op, reduce, out, rhs, True))
