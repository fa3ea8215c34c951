"""Public ind2ptr API (python/ops_gnn/ind2ptr.py:25-72 of ops-gnn)."""
import torch

from . import _pybind
from .typing import Tensor


def ind2ptr(ind: Tensor, num_rows: int) -> Tensor:
    """Convert sorted row indices to a CSR row-pointer tensor.

    Drop-in for ``torch.ops.torch_sparse.ind2ptr(ind, M)``: ``ind`` is a 1-D ``torch.long`` CUDA tensor of
    non-decreasing row ids, the result has ``num_rows + 1`` entries.  The kernel is enqueued on the current stream
    and the call returns without synchronising.

        >>> row = torch.tensor([2, 2, 4, 5, 5, 6], device="cuda")
        >>> ops_gnn.ind2ptr(row, 8)
        tensor([0, 0, 0, 2, 2, 3, 5, 6, 6], device='cuda:0')
    """
    if not ind.is_contiguous():
        ind = ind.contiguous()
    return _pybind.ind2ptr(ind, int(num_rows))
