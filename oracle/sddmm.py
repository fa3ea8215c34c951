"""Oracle of CSR SDDMM.  Test infrastructure; see the package docstring.

Follows `sddmm_reference` of the reference's test/sddmm_csr/arch22/golden.py:74-97: each operand is gathered by the
edge's row ("u", 0), the edge itself ("e", 1) or its column ("v", 2); `dot` multiplies and sums over the feature
axis, the other ops are elementwise; fp16 computes in fp32 and rounds once; 1-D operands are treated as [n, 1] and
squeezed again when every used operand was 1-D.
"""
import torch

from ._rows import edge_rows

_TARGETS = {"u": 0, "src": 0, "e": 1, "edge": 1, "v": 2, "dst": 2}


def _target(t):
    return _TARGETS[t.lower()] if isinstance(t, str) else int(t)


def _select(indptr, indices, target):
    target = _target(target)
    if target == 0:
        return edge_rows(indptr, indices.numel())
    if target == 1:
        return torch.arange(indices.numel(), dtype=torch.int64)
    return indices.long()


def sddmm_oracle(indptr, indices, lhs=None, rhs=None, op="dot", lhs_target=0, rhs_target=2):
    indptr, indices = indptr.cpu(), indices.cpu()
    use_lhs, use_rhs = op != "copy_rhs", op != "copy_lhs"
    lhs_1d = rhs_1d = False
    if use_lhs:
        lhs = lhs.cpu()
        if lhs.dim() == 1:
            lhs, lhs_1d = lhs.unsqueeze(-1), True
    if use_rhs:
        rhs = rhs.cpu()
        if rhs.dim() == 1:
            rhs, rhs_1d = rhs.unsqueeze(-1), True
    dtype = lhs.dtype if use_lhs else rhs.dtype
    compute = torch.float32 if dtype in (torch.float16, torch.bfloat16) else dtype
    squeeze = (lhs_1d or not use_lhs) and (rhs_1d or not use_rhs)
    left = lhs[_select(indptr, indices, lhs_target)] if use_lhs else None
    right = rhs[_select(indptr, indices, rhs_target)] if use_rhs else None
    if op == "dot":
        return (left.to(compute) * right.to(compute)).sum(dim=-1).to(dtype)
    if op == "copy_lhs":
        result = left
    elif op == "copy_rhs":
        result = right
    else:
        a, b = left.to(compute), right.to(compute)
        result = {"add": a + b, "sub": a - b, "mul": a * b, "div": a / b}[op].to(dtype)
    return result.squeeze(-1) if squeeze else result
