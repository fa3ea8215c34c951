"""Fused graph-attention aggregation.  An addition: the reference has no counterpart and composes the layer from
``sddmm_csr``, ``leaky_relu``, ``scatter_softmax`` and ``spmm`` / ``bspmm`` (python/ops_gnn/spmm.py:148-208, 283-289)."""
from typing import Optional, Tuple

import torch

from . import _pybind
from .ptr2ind import ptr2ind


def gat_aggregate(indptr: torch.Tensor, indices: torch.Tensor, x: torch.Tensor, left: torch.Tensor, right: torch.Tensor,
                  negative_slope: float = 0.2, edge_rows: Optional[torch.Tensor] = None,
                  return_lse: bool = False):
    """One GAT layer over a CSR graph (rows = destination nodes) in two launches; of the per-edge tensors only the logits
    are written (once) and read (once), the LeakyReLU output and the softmax weights never exist in memory.

    ``logit[e, h] = leaky_relu(left[row(e), h] + right[indices[e], h])``; the weights are the softmax of the logits over
    the edges of each row, per head; ``out[r, h, :] = sum_e weight[e, h] * x[indices[e], h, :]``.  ``x`` is ``[N, H, D]``,
    ``left`` ``[M, H]``, ``right`` ``[N, H]``, all float32 on one GPU; ``indptr`` / ``indices`` are int32 or int64.
    ``edge_rows`` is ``ptr2ind(indptr, E)``: pass it when it is already at hand (a layer stack computes it once).
    Rows without edges give 0.  It equals, within fp32 rounding::

        e = sddmm_csr(indptr, indices, left, right, "add", "u", "v")
        a = scatter_softmax(leaky_relu(e, negative_slope), edge_rows, 0, M)
        out = bspmm(indptr, indices, x, "mul", "sum", rhs=a.unsqueeze(-1))

    Shapes the fused kernel does not take (``H * D`` not a multiple of 256, ``H`` not a multiple of 4 or above 21) raise
    ``RuntimeError``; compose the layer as above for them.  No autograd.  ``return_lse`` also returns the ``[M, H]``
    log-sum-exp of the logits (``-inf`` for rows without edges).
    """
    if edge_rows is None:
        edge_rows = ptr2ind(indptr.to(torch.int64), indices.numel()).to(indptr.dtype)
    out, lse = _pybind.gat_aggregate(indptr, indices, edge_rows, x, left, right, float(negative_slope))
    return (out, lse) if return_lse else out
