"""``gather_coo``: gather rows by a sorted COO index (python/ops_gnn/gather_coo.py:20-47 of the reference)."""
from typing import Optional

from . import _pybind
from .typing import Tensor


def gather_coo(src: Tensor, index: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """``out[..., i, :] = src[..., index[..., i], :]`` along dimension ``index.dim() - 1``.

    ``index`` is int64 with the same leading shape as ``src``; the gathered dimension of ``src`` is replaced by
    ``index.size(-1)`` and trailing dimensions are copied unchanged.  A raw copy without autograd, as in the reference.
    ``out``, when given, must have the exact output shape and matching dtype / device and is returned as the same object.
    """
    return _pybind.gather_coo(src, index, out)
