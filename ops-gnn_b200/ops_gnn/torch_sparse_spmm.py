"""torch_sparse-compatible CSR / COO SpMM on CUDA.

Drop-in for the module of the same name in ops-gnn (python/ops_gnn/torch_sparse_spmm.py:222-342): ``csr_spmm``,
``coo_spmm``, ``coo_to_csr``, ``clear_validation_cache`` and ``validation_cache_info`` keep their signatures,
results and ``ValueError`` messages.

Semantics of ``csr_spmm(rowptr, col, value, mat, reduce)``: ``out[..., r, :] = reduce_e value[e] * mat[..., col[e], :]``
over the edges of row ``r``; sum/mean return ``out``, min/max return ``(out, arg)`` where ``arg`` is the winning edge
(first among ties, NaN products never win) and ``E`` for rows without a winner, whose value is 0.

How this file is organised: three identity-keyed LRU caches (validated CSR pairs, validated backward metadata, COO
layouts) share one small class; ``_Graph`` owns the pointer/column pair plus the optional backward metadata and knows
how to build what is missing on the GPU; ``_SpmmFunction`` is the autograd bridge.  When ``torch_sparse`` is
installed its dispatcher operators and ``SparseTensor`` front-ends are pointed here for CUDA tensors by
``_install_torch_sparse_hooks`` (the reference does the same for its device keys, :406-459).
"""
__all__ = ["csr_spmm", "coo_spmm", "coo_to_csr", "clear_validation_cache", "validation_cache_info"]

import importlib
import importlib.util
import weakref
from collections import OrderedDict, namedtuple
from numbers import Integral
from typing import Optional, Tuple, Union

import torch

from . import _pybind

try:
    import torch_sparse  # type: ignore  # optional front-end
except ImportError:  # pragma: no cover - depends on the environment
    torch_sparse = None

_native = _pybind.torch_sparse_spmm
_REDUCE_CODE = {"sum": 0, "add": 0, "mean": 1, "min": 2, "max": 3}
_DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.int8: 3, torch.int32: 4}
_VALUE_DTYPES = (torch.float32, torch.float16, torch.bfloat16, torch.int8)


class _IdentityLru:
    """LRU keyed by ``(id, version)`` of tensors; an entry is live only while every keyed tensor object is.

    Tensors without a version counter (inference tensors) are never stored, so a write that PyTorch cannot see can
    not leave a stale entry behind.  Writes through foreign pointers are outside what the cache can observe.
    """

    def __init__(self, capacity: int):
        self.capacity = capacity
        self.entries = OrderedDict()

    @staticmethod
    def stamp(tensor):
        return None if tensor is None else (id(tensor), _native.tensor_version(tensor))

    def lookup(self, key, tensors):
        hit = self.entries.get(key)
        if hit is None:
            return None
        refs, payload = hit
        if len(refs) != len(tensors) or any(ref() is not t for ref, t in zip(refs, tensors)):
            return None
        self.entries.move_to_end(key)
        return payload

    def store(self, key, tensors, payload=True, on_release=None):
        stamps = [self.stamp(t) for t in tensors]
        if any(s[1] is None for s in stamps):
            return
        refs = tuple(weakref.ref(t, on_release) if on_release else weakref.ref(t) for t in tensors)
        self.entries[key] = (refs, payload)
        while len(self.entries) > self.capacity:
            self.entries.popitem(last=False)

    def __len__(self):
        return len(self.entries)

    def clear(self):
        self.entries.clear()


_csr_cache = _IdentityLru(128)
_metadata_cache = _IdentityLru(128)
_coo_cache = _IdentityLru(32)
_CacheInfo = namedtuple("_CacheInfo", ("csr_entries", "metadata_entries", "coo_entries"))


def clear_validation_cache() -> None:
    for cache in (_csr_cache, _metadata_cache, _coo_cache):
        cache.clear()
    _pybind.clear_native_caches()


def validation_cache_info() -> _CacheInfo:
    """Entry counts of the three caches; no tensor is exposed."""
    return _CacheInfo(len(_csr_cache), len(_metadata_cache), len(_coo_cache))


# ---- argument checks ------------------------------------------------------------------------------------------------
def _require_dense(mat) -> None:
    if mat.device.type != "cuda" or mat.dim() < 2 or mat.dtype not in _VALUE_DTYPES:
        raise ValueError("mat must be a CUDA fp32/fp16/bf16/int8 tensor [...,N,K]")


def _weights_per_edge(value) -> int:
    count = 1
    for extent in value.shape[1:]:
        count *= extent
    return count


def _require_value(value, edges: int, mat) -> None:
    if value is None:
        return
    if value.dtype not in _VALUE_DTYPES or value.dtype != mat.dtype:
        raise ValueError("value dtype must be supported and match mat dtype")
    if value.device != mat.device or value.dim() < 1 or value.size(0) != edges:
        raise ValueError("value must be on the same GPU and have leading length E")
    if _weights_per_edge(value) not in (1, mat.size(-1)):
        raise ValueError("value must contain 1 or K weights per edge")


def _require_same_device(ptr, col, mat) -> None:
    if ptr.device != mat.device or col.device != mat.device:
        raise ValueError("indices and mat must be on the same GPU")


def _reduce_code(reduce) -> int:
    if not isinstance(reduce, str) or reduce not in _REDUCE_CODE:
        raise ValueError("reduce must be sum/add/mean/min/max")
    return _REDUCE_CODE[reduce]


def _validate_structure(ptr, col, columns: int) -> None:
    """Device-side CSR check; one 4-byte status comes back, and only the first time a (ptr, col) pair is seen."""
    key = (_IdentityLru.stamp(ptr), _IdentityLru.stamp(col), columns)
    if _csr_cache.lookup(key, (ptr, col)) is not None:
        return
    if int(_native.validate(ptr, col, columns).max().item()) != 0:
        raise ValueError("invalid CSR rowptr or column index out of range")
    _csr_cache.store(key, (ptr, col))


class _Graph:
    """A CSR structure and the metadata its backward pass needs (row ids, row counts, CSC pointer, CSR->CSC map)."""

    FIELDS = ("row", "rowcount", "colptr", "csr2csc")

    def __init__(self, ptr, col, row=None, rowcount=None, colptr=None, csr2csc=None):
        self.ptr, self.col = ptr, col
        self.row, self.rowcount, self.colptr, self.csr2csc = row, rowcount, colptr, csr2csc

    @property
    def edges(self) -> int:
        return self.col.numel()

    @property
    def rows(self) -> int:
        return self.ptr.numel() - 1

    def complete_for(self, value, mat, reduce_code: int) -> None:
        """Build on the GPU whatever the coming backward will read and the caller did not supply."""
        if reduce_code >= 2 or not torch.is_grad_enabled():
            return
        wants_value = value is not None and value.requires_grad
        if not (mat.requires_grad or wants_value):
            return
        if self.row is None:
            self.row = _native.convert(self.ptr, self.edges, False)
        if mat.requires_grad:
            if self.csr2csc is None:
                self.csr2csc = torch.argsort(self.col, stable=True)
            if self.colptr is None:
                self.colptr = _native.convert(self.col[self.csr2csc], mat.size(-2) + 1, True)
            if self.rowcount is None:
                self.rowcount = self.ptr[1:] - self.ptr[:-1]

    def _expect(self, tensor, length: int, name: str) -> None:
        device = self.col.device
        ok = (tensor is not None and tensor.dtype == torch.int64 and tensor.device == device
              and tuple(tensor.shape) == (length,))
        if not ok:
            raise ValueError(f"{name} must be int64 [{length}] on {device}")

    def check_metadata(self, value, mat, reduce_code: int) -> None:
        """Supplied metadata is checked even when no backward follows; required metadata must be present."""
        grads = torch.is_grad_enabled() and reduce_code < 2
        wants_value = grads and value is not None and value.requires_grad
        wants_mat = grads and mat.requires_grad
        columns = mat.size(-2)
        if self.row is not None or wants_value or wants_mat:
            self._expect(self.row, self.edges, "row")
        if self.colptr is not None or wants_mat:
            self._expect(self.colptr, columns + 1, "colptr")
        if self.csr2csc is not None or wants_mat:
            self._expect(self.csr2csc, self.edges, "csr2csc")
        if self.rowcount is not None or (wants_mat and reduce_code == 1):
            self._expect(self.rowcount, self.rows, "rowcount")
        extras = [getattr(self, name) for name in self.FIELDS]
        if all(t is None for t in extras):
            return
        slots = (self.ptr, self.col, *extras)
        present = tuple(t for t in slots if t is not None)
        key = (columns, tuple(_IdentityLru.stamp(t) for t in slots))
        if _metadata_cache.lookup(key, present) is not None:
            return
        self._check_contents(columns)
        _metadata_cache.store(key, present)

    def _check_contents(self, columns: int) -> None:
        if self.row is not None and not torch.equal(self.row, _native.convert(self.ptr, self.edges, False)):
            raise ValueError("row disagrees with rowptr")
        if self.rowcount is not None and not torch.equal(self.rowcount, self.ptr[1:] - self.ptr[:-1]):
            raise ValueError("rowcount disagrees with rowptr")
        by_column = None
        if self.csr2csc is not None:
            identity = torch.arange(self.edges, device=self.col.device)
            if not torch.equal(self.csr2csc.sort().values, identity):
                raise ValueError("csr2csc must be a permutation of [0,E)")
            by_column = self.col[self.csr2csc]
            if self.edges > 1 and bool((by_column[1:] < by_column[:-1]).any().item()):
                raise ValueError("csr2csc must order edges by column")
        if self.colptr is not None:
            if by_column is None:
                by_column = self.col.sort().values
            if not torch.equal(self.colptr, _native.convert(by_column, columns + 1, True)):
                raise ValueError("colptr disagrees with col and csr2csc")


class _SpmmFunction(torch.autograd.Function):
    """Forward = engine launch.  Backward (sum/mean only): d value = SDDMM-style kernel over the edges,
    d mat = SpMM over the transposed graph (CSC pointer, permuted rows and weights) in fp32."""

    @staticmethod
    def forward(ctx, value, mat, graph, reduce_code, out_code):
        out, arg = _native.forward(graph.ptr, graph.col, value, mat, reduce_code, out_code)
        ctx.graph, ctx.reduce_code = graph, reduce_code
        ctx.save_for_backward(value, mat)
        ctx.mark_non_differentiable(arg)
        return out, arg

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_out, _grad_arg):
        if ctx.reduce_code >= 2:
            raise NotImplementedError("min/max backward is outside this extension's supported contract")
        value, mat = ctx.saved_tensors
        graph = ctx.graph
        grad_value = grad_mat = None
        if value is not None and ctx.needs_input_grad[0]:
            raw = _native.value_backward(graph.ptr, graph.col, mat, grad_out, ctx.reduce_code,
                                         _weights_per_edge(value))
            grad_value = raw.reshape_as(value).to(value.dtype)
        if ctx.needs_input_grad[1]:
            upstream = grad_out.float()
            if ctx.reduce_code == 1:
                upstream = upstream / (graph.ptr[1:] - graph.ptr[:-1]).clamp_min(1).float().unsqueeze(-1)
            weights = None if value is None else value[graph.csr2csc].float()
            grad_mat = _native.forward(graph.colptr, graph.row[graph.csr2csc], weights, upstream, 0, 0)[0].to(mat.dtype)
        return grad_value, grad_mat, None, None, None


def _run(graph: _Graph, value, mat, reduce_code: int, output_dtype=None):
    """Shared tail of every entry point: checks, validation, then the plain or the differentiable launch."""
    _require_dense(mat)
    _require_value(value, graph.edges, mat)
    _require_same_device(graph.ptr, graph.col, mat)
    _validate_structure(graph.ptr, graph.col, mat.size(-2))
    if reduce_code < 2:
        graph.check_metadata(value, mat, reduce_code)
    dtype = output_dtype or (torch.int32 if mat.dtype == torch.int8 else mat.dtype)
    if dtype not in _DTYPE_CODE:
        raise ValueError("unsupported output dtype")
    differentiable = torch.is_grad_enabled() and (mat.requires_grad or (value is not None and value.requires_grad))
    if not differentiable:
        return _native.forward(graph.ptr, graph.col, value, mat, reduce_code, _DTYPE_CODE[dtype])
    return _SpmmFunction.apply(value, mat, graph, reduce_code, _DTYPE_CODE[dtype])


def csr_spmm(
    rowptr: torch.Tensor,
    col: torch.Tensor,
    value: Optional[torch.Tensor],
    mat: torch.Tensor,
    reduce: str = "sum",
    *,
    output_dtype: Optional[torch.dtype] = None,
) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """CSR SpMM on int64 ``rowptr``/``col``; ``value`` is ``None``, ``[E]`` or ``[E, K]`` with ``mat``'s dtype.

    ``output_dtype`` is an extension-only precision choice (fp32 output for 16-bit inputs; int32 or fp32 for int8).
    Missing backward metadata is constructed on the GPU.  Min/max return ``(out, arg)``, sum/mean return ``out``.
    """
    _require_dense(mat)
    _require_value(value, col.numel(), mat)
    _require_same_device(rowptr, col, mat)
    code = _reduce_code(reduce)
    _validate_structure(rowptr, col, mat.size(-2))
    graph = _Graph(rowptr, col)
    graph.complete_for(value, mat, code)
    out, arg = _run(graph, value, mat, code, output_dtype)
    return (out, arg) if code >= 2 else out


# ---- COO front-end ------------------------------------------------------------------------------------------------------
def _coo_layout(index, rows: int):
    """(rowptr, col, permutation or None) for COO indices; rows already sorted need no permutation."""
    row = index[0]
    if bool(((row < 0) | (row >= rows)).any().item()):
        raise ValueError("COO row out of range")
    already_sorted = row.numel() < 2 or not bool((row[1:] < row[:-1]).any().item())
    if already_sorted:
        return _native.convert(row, rows + 1, True), index[1].clone(), None
    order = torch.argsort(row, stable=True)
    return _native.convert(row[order], rows + 1, True), index[1][order], order


def coo_to_csr(index: torch.Tensor, value: Optional[torch.Tensor],
               m: int) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """COO ``[2, E]`` int64 indices (+ optional values) to ``(rowptr, col, value)`` with columns stably ordered by
    row.  Nothing is cached and dense-input compatibility is not checked (conversion profiling helper)."""
    ptr, col, order = _coo_layout(index, m)
    if value is None:
        return ptr, col, None
    return ptr, col, value.clone() if order is None else value[order]


def _coo_layout_cached(index, rows: int):
    """Only topology is reused; edge values and dense inputs are read on every call."""
    stamp = _IdentityLru.stamp(index)
    if stamp[1] is None:
        return _coo_layout(index, rows)
    key = (stamp, rows)
    layout = _coo_cache.lookup(key, (index,))
    if layout is None:
        layout = _coo_layout(index, rows)
        _coo_cache.store(key, (index,), layout, on_release=lambda _ref, key=key: _coo_cache.entries.pop(key, None))
    return layout


def coo_spmm(index: torch.Tensor, value: Optional[torch.Tensor], m: int, n: int, matrix: torch.Tensor) -> torch.Tensor:
    """``torch_sparse.spmm(index, value, m, n, matrix)`` (sum reduction) for CUDA inputs."""
    if matrix.device.type != "cuda":
        if _upstream_coo_spmm is None:
            raise ValueError("mat must be a CUDA fp32/fp16/bf16/int8 tensor [...,N,K]")
        return _upstream_coo_spmm(index, value, m, n, matrix)
    _require_dense(matrix)
    for extent in (m, n):
        if isinstance(extent, bool) or not isinstance(extent, Integral) or extent < 0:
            raise ValueError("COO m and n must be nonnegative integers")
    if index.dtype != torch.int64 or index.dim() != 2 or index.size(0) != 2:
        raise ValueError("COO index must be int64 [2,E] and dimensions nonnegative")
    if index.device != matrix.device or matrix.dim() < 2 or matrix.size(-2) != n:
        raise ValueError("COO device or dense shape mismatch")
    _require_value(value, index.size(1), matrix)  # before a permutation could hide surplus entries
    ptr, col, order = _coo_layout_cached(index, m)
    tracked = torch.is_grad_enabled() and value is not None and value.requires_grad
    if value is None:
        weights = None
    elif order is not None:
        weights = value[order] if tracked else _native.permute_values(value, order)
    elif tracked or (torch.is_grad_enabled() and matrix.requires_grad):
        weights = value.clone()
    else:
        weights = value
    return csr_spmm(ptr, col, weights, matrix)


# ---- optional torch_sparse / PyG hooks ------------------------------------------------------------------------------------
_LIBRARIES = []
_upstream_coo_spmm = None


def _remember_original(owner, name):
    """First-seen attribute of ``owner``, kept across ``importlib.reload`` of this module."""
    return owner.__dict__.setdefault("_ops_gnn_originals", {}).setdefault(name, owner.__dict__[name])


def register_dispatcher_kernels():
    """Implement the six ``torch_sparse`` dispatcher operators of the SpMM path for CUDA tensors.

    The reference registers ``spmm_sum``, ``spmm_mean``, ``spmm_min``, ``spmm_max``, ``ind2ptr`` and ``ptr2ind`` for its
    device keys from Python (python/ops_gnn/torch_sparse_spmm.py:406-431); here the keys are ``CUDA`` and
    ``AutogradCUDA``.  Only the operator SCHEMAS have to exist in the dispatcher (``torch_sparse`` defines them when it
    is installed); an existing CUDA kernel of a CUDA build of ``torch_sparse`` is never shadowed.  Returns the names
    that received a kernel, per key.  Called at import when ``torch_sparse`` is importable.
    """
    def op_sum(row, ptr, col, value, colptr, csr2csc, mat):
        return _run(_Graph(ptr, col, row=row, colptr=colptr, csr2csc=csr2csc), value, mat, 0)[0]

    def op_mean(row, ptr, col, value, rowcount, colptr, csr2csc, mat):
        return _run(_Graph(ptr, col, row=row, rowcount=rowcount, colptr=colptr, csr2csc=csr2csc), value, mat, 1)[0]

    table = {
        "spmm_sum": op_sum,
        "spmm_mean": op_mean,
        "spmm_min": lambda ptr, col, value, mat: _run(_Graph(ptr, col), value, mat, 2),
        "spmm_max": lambda ptr, col, value, mat: _run(_Graph(ptr, col), value, mat, 3),
        "ind2ptr": lambda ind, rows: _native.convert(ind, rows + 1, True),
        "ptr2ind": lambda ptr, edges: _native.convert(ptr, edges, False),
    }
    registered = {}
    for key in ("CUDA", "AutogradCUDA"):
        library = torch.library.Library("torch_sparse", "IMPL", key)
        registered[key] = []
        for name, implementation in table.items():
            # A CUDA build of torch_sparse owns its own CUDA kernels; never shadow an existing registration.
            if key == "CUDA" and _pybind.has_private_use1_kernel("torch_sparse::" + name):
                continue
            try:
                library.impl(name, implementation)
                registered[key].append(name)
            except RuntimeError:
                pass
        _LIBRARIES.append(library)
    return registered


def _install_torch_sparse_hooks():  # pragma: no cover - needs the third-party package
    global _upstream_coo_spmm
    _upstream_coo_spmm = _remember_original(torch_sparse, "spmm")
    matmul_module = importlib.import_module("torch_sparse.matmul")
    upstream_matmul = _remember_original(matmul_module, "matmul")
    upstream_spmm = _remember_original(matmul_module, "spmm")

    def storage_graph(src, other):
        storage = src.storage
        if not storage.has_rowptr():
            row = storage.row() if storage.has_row() else None
            if row is None or row.dtype != torch.int64 or row.device != other.device:
                raise ValueError("SparseTensor row must be int64 on the same GPU")
            if bool(((row < 0) | (row >= src.sparse_size(0))).any().item()):
                raise ValueError("SparseTensor row out of range")
            if row.numel() > 1 and bool((row[1:] < row[:-1]).any().item()):
                raise ValueError("SparseTensor row must be sorted")
        return _Graph(
            storage.rowptr(), storage.col(),
            row=storage.row() if storage.has_row() else None,
            rowcount=storage.rowcount() if storage.has_rowcount() else None,
            colptr=storage.colptr() if storage.has_colptr() else None,
            csr2csc=storage.csr2csc() if storage.has_csr2csc() else None)

    def sparse_tensor_spmm(src, other, reduce="sum"):
        if other.device.type != "cuda":
            return upstream_spmm(src, other, reduce)
        _require_dense(other)
        code = _reduce_code(reduce)
        if other.size(-2) != src.sparse_size(1):
            raise ValueError("sparse columns must match dense N")
        graph = storage_graph(src, other)
        value = src.storage.value()
        _require_value(value, graph.edges, other)
        _validate_structure(graph.ptr, graph.col, other.size(-2))
        with torch.no_grad():
            graph.check_metadata(value, other, code)
        result = csr_spmm(graph.ptr, graph.col, value, other, reduce)
        return result[0] if code >= 2 else result

    def matmul(src, other, reduce="sum"):
        if isinstance(other, torch.Tensor):
            return sparse_tensor_spmm(src, other, reduce)
        return upstream_matmul(src, other, reduce)

    register_dispatcher_kernels()

    torch_sparse.spmm = coo_spmm
    importlib.import_module("torch_sparse.spmm").spmm = coo_spmm
    torch_sparse.matmul = matmul_module.matmul = matmul
    matmul_module.spmm = sparse_tensor_spmm
    sparse_tensor = torch_sparse.SparseTensor
    sparse_tensor.spmm = sparse_tensor_spmm
    sparse_tensor.matmul = matmul
    sparse_tensor.__matmul__ = lambda self, other: matmul(self, other, "sum")

    # PyG routes non-CUDA-looking sparse matmuls elsewhere; point its helper and the aliases captured by GCN/GIN here.
    if importlib.util.find_spec("torch_geometric") is not None:
        pyg_module = importlib.import_module("torch_geometric.utils._spmm")
        upstream_pyg = _remember_original(pyg_module, "spmm")

        def pyg_spmm(src, other, reduce="sum"):
            if isinstance(src, sparse_tensor) and other.device.type == "cuda":
                return sparse_tensor_spmm(src, other, reduce)
            return upstream_pyg(src, other, reduce)

        importlib.import_module("torch_geometric.utils").spmm = pyg_spmm
        pyg_module.spmm = pyg_spmm
        for conv in ("gcn_conv", "gin_conv"):
            importlib.import_module("torch_geometric.nn.conv." + conv).spmm = pyg_spmm


if torch_sparse is not None:  # pragma: no cover - needs the third-party package
    _install_torch_sparse_hooks()
