"""Generalized CSR SpMM aggregation: ``ops_gnn.spmm`` (API of python/ops_gnn/spmm.py:309-322 in ops-gnn).

For every CSR row ``r``::

    out[r] = reduce over the edges e of r of  message(x[indices[e]], rhs[e])

Message ops: ``copy_lhs`` (gather a source row), ``copy_rhs`` (take the edge row), ``add/sub/mul/div`` (combine both,
with missing feature dimensions inserted right after the item axis).  Reductions: ``sum``, ``mean``, ``max``, ``min``;
rows without edges give 0.

A call is handled by the first strategy of ``_STRATEGIES`` that accepts it:

* ``_NativeGather`` / ``_NativeEdgeRows``: no-grad ``copy_lhs`` / ``copy_rhs`` with sum, max or min run on the CSR
  reduce engine through the same ``_pybind`` functions the reference binds (``spmm_{sum,max,min}_csr`` for fp16,
  ``unified_spmm_csr`` for fp32).
* ``_NativeScaledGather``: no-grad ``mul`` whose edge operand is constant over trailing feature dimensions
  (``rhs [E]``, ``[E, 1]``, or ``[E, H, 1]`` against ``x [V, H, D]``: attention weights) is fused into the gather;
  the reference materialises the ``[E, ...]`` messages for this case (spmm.py:148-162).
* ``_TorchComposition``: everything else, and everything that needs autograd, is composed from differentiable torch
  operators on the same GPU.  There is no CPU path.
"""
from typing import NamedTuple, Optional

import torch

from . import _pybind

_MESSAGE_OPS = ("copy_lhs", "copy_rhs", "add", "sub", "mul", "div")
_REDUCTIONS = ("sum", "max", "min", "mean")


class _SpmmRequest(NamedTuple):
    indptr: torch.Tensor
    indices: torch.Tensor
    x: Optional[torch.Tensor]
    op: str
    reduce: str
    out: Optional[torch.Tensor]
    rhs: Optional[torch.Tensor]
    batched: bool

    @property
    def api(self) -> str:
        return "bspmm" if self.batched else "spmm"


class _Operands(NamedTuple):
    node: Optional[torch.Tensor]  # rows selected by indices[e]
    edge: Optional[torch.Tensor]  # rows selected by e
    needs_grad: bool


def _split_operands(request: _SpmmRequest) -> _Operands:
    x, rhs, op = request.x, request.rhs, request.op
    if op == "copy_lhs":
        if x is None or rhs is not None:
            raise ValueError("copy_lhs requires x and does not accept rhs")
        node, edge = x, None
    elif op == "copy_rhs":
        if rhs is not None and x is not None:
            raise ValueError("copy_rhs accepts edge features through either x or rhs, not both")
        if rhs is None and x is None:
            raise ValueError("copy_rhs requires edge features")
        node, edge = None, rhs if rhs is not None else x
    else:
        if x is None or rhs is None:
            raise ValueError(f"{op} requires both x and rhs")
        node, edge = x, rhs
    tracked = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (node, edge))
    if not tracked:
        # Detach only what carries autograd state: a needless `detach()` is an ATen call, and any ATen call between two
        # native calls makes the planners re-derive their cached CSR facts (they cannot tell it from a write).
        node = node.detach() if node is not None and node.requires_grad else node
        edge = edge.detach() if edge is not None and edge.requires_grad else edge
    return _Operands(node, edge, tracked)


def _check_tensors(request: _SpmmRequest, operands: _Operands) -> None:
    """Type, device, dtype and rank rules shared by every strategy that does not defer them to C++."""
    features = [t for t in (operands.node, operands.edge) if t is not None]
    if not features:
        raise ValueError("at least one feature tensor is required")
    device = features[0].device
    if device.type != "cuda" or any(t.device != device for t in features):
        raise RuntimeError("spmm: feature tensors must be on the same GPU")
    indptr, indices = request.indptr, request.indices
    if indptr.device != device or indices.device != device:
        raise RuntimeError("spmm: CSR tensors and features must be on the same GPU")
    if indptr.dim() != 1 or indices.dim() != 1:
        raise RuntimeError("spmm: CSR tensors must be one-dimensional")
    if indptr.numel() == 0:
        raise RuntimeError("spmm: indptr must be nonempty")
    if indptr.dtype not in (torch.int32, torch.int64) or indices.dtype != indptr.dtype:
        raise RuntimeError("spmm: CSR tensors must have the same int32 or int64 dtype")
    if any(t.dtype not in (torch.float16, torch.float32) for t in features):
        raise RuntimeError("spmm: features must use float16 or float32")
    if len(features) == 2 and features[0].dtype != features[1].dtype:
        raise RuntimeError("x and rhs must have the same dtype")
    ranks = [t.dim() for t in features]
    if min(ranks) < 1:
        raise RuntimeError("spmm feature tensors must have at least one dimension")
    if request.batched and max(ranks) < 3:
        raise RuntimeError("bspmm requires at least one feature tensor with rank 3 or higher")
    if not request.batched and max(ranks) > 2:
        raise RuntimeError("spmm supports scalar or two-dimensional features; use bspmm for higher-rank features")


def _check_structure(request: _SpmmRequest, operands: _Operands) -> None:
    """CSR contents, checked by one device pass; a 4-byte mask returns to the host (cached per tensor version)."""
    rows, edges = request.indptr.numel() - 1, request.indices.numel()
    node = operands.node
    mask = int(_pybind.csr_facts(request.indptr, request.indices if node is not None else None, rows,
                                 node.size(0) if node is not None else 0, edges))
    if mask & 1:
        raise RuntimeError("indptr must start at zero and end at indices.numel()")
    if mask & 6:
        raise RuntimeError("indptr must be non-decreasing")
    if mask & 8:
        raise RuntimeError("indices are out of range for x")
    if operands.edge is not None and operands.edge.size(0) != edges:
        raise RuntimeError("rhs.size(0) must equal indices.numel()")


def _deliver(result: torch.Tensor, out: Optional[torch.Tensor], tracked: bool) -> torch.Tensor:
    if out is None:
        return result
    if tracked:
        raise RuntimeError("out is not supported when feature tensors require gradients")
    if out.shape != result.shape or out.dtype != result.dtype or out.device != result.device:
        raise RuntimeError("out must match the result shape, dtype and device")
    if not out.is_contiguous() or out.requires_grad:
        raise RuntimeError("out must be contiguous and must not require gradients")
    out.copy_(result)
    return out


# ---- strategies ---------------------------------------------------------------------------------------------------------
class _NativeGather:
    """copy_lhs + sum/max/min without autograd: the engine gathers source rows itself."""

    HALF = {"sum": _pybind.spmm_sum_csr, "max": _pybind.spmm_max_csr, "min": _pybind.spmm_min_csr}

    @classmethod
    def run(cls, request: _SpmmRequest, operands: _Operands):
        node = operands.node
        if operands.needs_grad or request.op != "copy_lhs" or request.reduce not in cls.HALF:
            return None
        if not isinstance(node, torch.Tensor):
            return None
        wanted_rank = 3 if request.batched else 2
        if node.dim() != wanted_rank:
            return None
        if node.dtype == torch.float16:
            return cls.HALF[request.reduce](request.indptr, request.indices, node, request.out)
        if node.dtype == torch.float32 and not request.batched:
            return _pybind.unified_spmm_csr(request.indptr, request.indices, node, "copy_lhs", request.reduce,
                                            request.out)
        return None


class _NativeEdgeRows:
    """copy_rhs + sum/max/min on fp32 [E, F] edge features: a segment reduction over consecutive rows."""

    @staticmethod
    def run(request: _SpmmRequest, operands: _Operands):
        edge = operands.edge
        if operands.needs_grad or request.batched or request.op != "copy_rhs" or request.reduce == "mean":
            return None
        if not isinstance(edge, torch.Tensor) or edge.dim() != 2 or edge.dtype != torch.float32:
            return None
        return _pybind.unified_spmm_csr(request.indptr, request.indices, edge, "copy_rhs", request.reduce, request.out)


class _NativeScaledGather:
    """mul with an edge operand that is constant over trailing feature dimensions, fused into the gather."""

    @staticmethod
    def weights_per_edge(node: torch.Tensor, edge: torch.Tensor) -> Optional[int]:
        features = tuple(node.shape[1:])
        missing = len(features) - (edge.dim() - 1)
        if missing < 0:
            return None
        aligned = (1,) * missing + tuple(edge.shape[1:])
        count, tail = 1, False
        for full, have in zip(features, aligned):
            if tail and have != 1:
                return None
            if not tail:
                if have == full:
                    count *= full
                elif have == 1:
                    tail = True
                else:
                    return None
        return count

    @classmethod
    def run(cls, request: _SpmmRequest, operands: _Operands):
        node, edge = operands.node, operands.edge
        if operands.needs_grad or request.op != "mul":
            return None
        if not (isinstance(node, torch.Tensor) and isinstance(edge, torch.Tensor)):
            return None
        if node.dim() < 1 or edge.dim() < 1 or node.dtype != edge.dtype or node.numel() == 0:
            return None
        if edge.size(0) != request.indices.numel():
            return None
        groups = cls.weights_per_edge(node, edge)
        if groups is None:
            return None
        _check_tensors(request, operands)
        width = node.numel() // node.size(0)
        flat = _pybind.spmm_weighted_csr(request.indptr, request.indices, node.reshape(node.size(0), width),
                                         edge.reshape(edge.size(0), groups), request.reduce)
        shaped = flat.reshape((request.indptr.numel() - 1,) + tuple(node.shape[1:]))
        return _deliver(shaped, request.out, False)


class _TorchComposition:
    """Materialise the messages and reduce them with differentiable torch operators on the device."""

    @staticmethod
    def messages(request: _SpmmRequest, operands: _Operands) -> torch.Tensor:
        if request.op == "copy_rhs":
            return operands.edge
        picked = operands.node.index_select(0, request.indices.to(torch.int64))
        if request.op == "copy_lhs":
            return picked
        edge = operands.edge
        rank = max(picked.dim(), edge.dim())

        def pad(t):  # insert singleton feature dimensions right after the item axis
            return t.reshape((t.shape[0],) + (1,) * (rank - t.dim()) + tuple(t.shape[1:]))

        picked, edge = pad(picked), pad(edge)
        if request.op == "add":
            return picked + edge
        if request.op == "sub":
            return picked - edge
        if request.op == "mul":
            return picked * edge
        return picked / edge

    @staticmethod
    def reduce(indptr: torch.Tensor, messages: torch.Tensor, how: str) -> torch.Tensor:
        rows = indptr.numel() - 1
        degree = (indptr[1:] - indptr[:-1]).to(torch.int64)
        owner = torch.repeat_interleave(torch.arange(rows, device=indptr.device), degree,
                                        output_size=messages.size(0))
        shape = (rows,) + tuple(messages.shape[1:])
        if how in ("sum", "mean"):
            widen = how == "mean" and messages.dtype == torch.float16
            total = (messages.float() if widen else messages).new_zeros(shape)
            total = total.index_add(0, owner, messages.float() if widen else messages)
            if how == "sum":
                return total
            # The divisor stays in fp32: fp16 cannot represent degrees above 65504.
            divisor = degree.clamp(min=1).to(torch.float32).reshape((rows,) + (1,) * (messages.dim() - 1))
            return (total.to(torch.float32) / divisor).to(messages.dtype)
        if rows == 0:
            return messages.new_empty(shape)
        spread = owner.reshape((-1,) + (1,) * (messages.dim() - 1)).expand_as(messages)
        return messages.new_zeros(shape).scatter_reduce(0, spread, messages, "amax" if how == "max" else "amin",
                                                        include_self=False)

    @classmethod
    def run(cls, request: _SpmmRequest, operands: _Operands):
        _check_tensors(request, operands)
        if request.op == "copy_rhs" and operands.edge.dtype != torch.float32:
            raise RuntimeError("copy_rhs supports only float32")
        _check_structure(request, operands)
        result = cls.reduce(request.indptr, cls.messages(request, operands), request.reduce)
        return _deliver(result, request.out, operands.needs_grad)


_STRATEGIES = (_NativeGather, _NativeEdgeRows, _NativeScaledGather, _TorchComposition)


def _spmm(request: _SpmmRequest) -> torch.Tensor:
    api = request.api
    for name in ("indptr", "indices", "x", "rhs", "out"):
        value = getattr(request, name)
        if value is not None and not isinstance(value, torch.Tensor):
            raise TypeError(f"{api}: {name} must be a Tensor")
    if not isinstance(request.op, str) or request.op not in _MESSAGE_OPS:
        raise RuntimeError(f"{api}: op must be copy_lhs, copy_rhs, add, sub, mul or div")
    if not isinstance(request.reduce, str) or request.reduce not in _REDUCTIONS:
        raise RuntimeError(f"{api}: reduce must be sum, max, min or mean")
    operands = _split_operands(request)
    for strategy in _STRATEGIES:
        result = strategy.run(request, operands)
        if result is not None:
            return result
    raise AssertionError("unreachable: the torch composition accepts every valid request")


def _parse_call_options(api: str, args: tuple, kwargs: dict) -> tuple:
    """Resolve the optional ``op, reduce, out, rhs`` arguments given positionally and/or by keyword."""
    order = ("op", "reduce", "out", "rhs")
    if len(args) > len(order):
        raise TypeError(f"{api} accepts at most seven positional arguments")
    resolved = {"op": "copy_lhs", "reduce": "sum", "out": None, "rhs": None}
    for name, value in zip(order, args):
        if name in kwargs:
            raise TypeError(f"{api} got multiple values for argument '{name}'")
        resolved[name] = value
    for name in sorted(kwargs):
        if name not in resolved:
            raise TypeError(f"{api} got an unexpected keyword argument '{name}'")
        resolved[name] = kwargs[name]
    return tuple(resolved[name] for name in order)


def spmm(indptr: torch.Tensor, indices: torch.Tensor, x: Optional[torch.Tensor] = None, *args,
         **kwargs) -> torch.Tensor:
    """Generalized CSR aggregation on CUDA tensors.

    ``x`` holds source features for ``copy_lhs`` and the left operand of the binary message ops; ``rhs`` holds
    CSR-ordered edge features (``copy_rhs`` also accepts them through ``x``).  Optional arguments in positional
    order: ``op='copy_lhs'``, ``reduce='sum'``, ``out=None``, ``rhs=None``.
    """
    op, reduce, out, rhs = _parse_call_options("spmm", args, kwargs)
    return _spmm(_SpmmRequest(indptr, indices, x, op, reduce, out, rhs, False))
