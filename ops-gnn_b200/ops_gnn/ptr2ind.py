"""Public ptr2ind API (python/ops_gnn/ptr2ind.py of ops-gnn)."""
import torch

from . import _pybind
from .typing import Tensor


def ptr2ind(ptr: Tensor, num_edges: int) -> Tensor:
    """Expand a CSR row pointer into one row id per edge.

    Drop-in for ``torch.ops.torch_sparse.ptr2ind(ptr, E)``: ``ptr`` is a 1-D ``torch.long`` CUDA tensor that starts
    at 0, never decreases and ends at ``num_edges``; a pointer that breaks this raises ``RuntimeError`` (checked on
    the device, four bytes return to the host).

        >>> ops_gnn.ptr2ind(torch.tensor([0, 0, 0, 2, 2, 3, 5, 6, 6], device="cuda"), 6)
        tensor([2, 2, 4, 5, 5, 6], device='cuda:0')
    """
    if not ptr.is_contiguous():
        ptr = ptr.contiguous()
    return _pybind.ptr2ind(ptr, int(num_edges))
