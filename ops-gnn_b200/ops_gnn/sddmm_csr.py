"""Generalized sampled dense-dense matrix multiplication on a CSR graph: ``ops_gnn.sddmm_csr``.

API of python/ops_gnn/sddmm_csr.py:126-173 in ops-gnn.  For every stored edge ``e`` of the CSR matrix

    out[e] = op(lhs[t_l(e)], rhs[t_r(e)])

where a target picks the CSR row of the edge (``0`` / ``"u"`` / ``"src"``), the edge itself (``1`` / ``"e"`` /
``"edge"``) or its column (``2`` / ``"v"`` / ``"dst"``).  ``dot`` reduces the feature axis and returns ``(nnz,)``;
``add, sub, mul, div, copy_lhs, copy_rhs`` return ``(nnz, feature_dim)``.  One-dimensional operands act as
``(rows, 1)`` and the trailing axis is squeezed again.  fp16 (and bf16) compute in fp32 and round once.
"""
from typing import Optional

import torch

from . import _pybind

_BOTH, _LEFT, _RIGHT = (True, True), (True, False), (False, True)
_OPERANDS = {"dot": _BOTH, "add": _BOTH, "sub": _BOTH, "mul": _BOTH, "div": _BOTH, "copy_lhs": _LEFT,
             "copy_rhs": _RIGHT}
_TARGETS = {"u": 0, "src": 0, "e": 1, "edge": 1, "v": 2, "dst": 2}
_FEATURE_DTYPES = (torch.float16, torch.float32)


def _target_code(target, name: str) -> int:
    code = None
    if isinstance(target, str):
        code = _TARGETS.get(target.lower())
    elif isinstance(target, int) and not isinstance(target, bool) and target in (0, 1, 2):
        code = target
    if code is None:
        raise ValueError(f"sddmm_csr: {name} must be 0, 1, 2, u, e or v")
    return code


def _as_matrix(name: str, value, used: bool):
    """Validate one operand and return it as a 2-D tensor plus whether it came in 1-D."""
    if not used:
        if value is not None:
            raise ValueError(f"sddmm_csr: {name} is not used by this op")
        return None, False
    if value is None:
        raise ValueError(f"sddmm_csr: {name} is required by this op")
    if not isinstance(value, torch.Tensor):
        raise TypeError(f"sddmm_csr: {name} must be a Tensor")
    if value.dim() not in (1, 2):
        raise ValueError(f"sddmm_csr: {name} must be one- or two-dimensional")
    if value.dtype not in _FEATURE_DTYPES:
        raise ValueError(f"sddmm_csr: {name} must be float16 or float32")
    return (value.unsqueeze(-1), True) if value.dim() == 1 else (value, False)


def sddmm_csr(indptr: torch.Tensor, indices: torch.Tensor, lhs: Optional[torch.Tensor] = None,
              rhs: Optional[torch.Tensor] = None, op: str = "dot", lhs_target=0, rhs_target=2,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Run generalized SDDMM on a CSR graph held on a CUDA device.

    ``indptr`` / ``indices`` are 1-D int32 or int64 tensors of one dtype on the same GPU (``indptr`` nonempty,
    non-decreasing, from 0 to ``nnz``).  ``lhs`` / ``rhs`` share device, dtype and feature width.  ``out``, if given,
    must have the result's shape, dtype and device, be contiguous, not require grad and not alias an input; it is
    returned.  Autograd is not supported.
    """
    if not isinstance(indptr, torch.Tensor):
        raise TypeError("sddmm_csr: indptr must be a Tensor")
    if not isinstance(indices, torch.Tensor):
        raise TypeError("sddmm_csr: indices must be a Tensor")
    if op not in _OPERANDS:
        raise ValueError("sddmm_csr: op must be dot, add, sub, mul, div, copy_lhs or copy_rhs")
    use_lhs, use_rhs = _OPERANDS[op]
    left, left_1d = _as_matrix("lhs", lhs, use_lhs)
    right, right_1d = _as_matrix("rhs", rhs, use_rhs)
    if use_lhs and use_rhs:
        if left.device != right.device:
            raise ValueError("sddmm_csr: lhs and rhs must be on the same device")
        if left.dtype != right.dtype:
            raise ValueError("sddmm_csr: lhs and rhs must have the same dtype")
        if left.size(1) != right.size(1):
            raise ValueError("sddmm_csr: lhs and rhs must have the same feature dim")
    lhs_code = _target_code(lhs_target, "lhs_target")
    rhs_code = _target_code(rhs_target, "rhs_target")

    width = (left if use_lhs else right).size(1)
    nnz = indices.numel()
    squeeze = op != "dot" and (left_1d or not use_lhs) and (right_1d or not use_rhs)
    final_shape = (nnz,) if (op == "dot" or squeeze) else (nnz, width)
    native_out = None
    if out is not None:
        if not isinstance(out, torch.Tensor):
            raise TypeError("sddmm_csr: out must be a Tensor")
        if tuple(out.shape) != final_shape:
            raise ValueError(f"sddmm_csr: out must have shape {tuple(final_shape)}, got {tuple(out.shape)}")
        native_out = out.unsqueeze(-1) if squeeze else out
    result = _pybind.sddmm_csr(indptr, indices, left, right, op, lhs_code, rhs_code, native_out)
    if out is not None:
        return out
    return result.squeeze(-1) if squeeze else result
