"""``gather_csr``: expand segment rows by CSR pointers (python/ops_gnn/gather_csr.py:15-26 of the reference)."""
from typing import Optional

from . import _pybind
from .typing import Tensor


def gather_csr(src: Tensor, indptr: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """``out[..., e, :] = src[..., s, :]`` for ``indptr[..., s] <= e < indptr[..., s + 1]``.

    The segment dimension is ``indptr.dim() - 1``; ``indptr`` is int64 and broadcasts over the leading dimensions of
    ``src``; the output has ``indptr[..., -1]`` rows along that dimension and rows before ``indptr[..., 0]`` are zero.
    It is the inverse data movement of ``segment_csr`` (the gradient of a segment sum).  ``src`` and ``indptr`` are CUDA
    tensors; ``out``, when given, must have the inferred shape, dtype and device and is returned as the same object.
    """
    return _pybind.gather_csr(src, indptr, out)
