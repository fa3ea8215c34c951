"""ctypes view of ``libopsgnn_b200.so`` (the C ABI declared in ``include/opsgnn_b200.h``).

The torch extension ``_pybind`` is the product path; this module exists so tests, the benchmark and
foreign-language callers can drive the same entry points with raw device pointers.  Nothing here computes:
a missing library raises ``ImportError`` instead of falling back to another implementation.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_int, c_int32, c_int64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_HERE, "sm100", "libopsgnn_b200.so")

# dtype ids (include/opsgnn_b200.h)
F32, F16, BF16, I8, I32, I64, U8, I16, F64 = range(9)
REDUCE_SUM, REDUCE_MEAN, REDUCE_MIN, REDUCE_MAX, REDUCE_LOGSUMEXP = range(5)
EXTREMUM_IGNORE_NAN, EXTREMUM_PROPAGATE_NAN, EXTREMUM_SEEDED, EXTREMUM_SEEDED_LAST = range(4)
SDDMM_OPS = {"dot": 0, "add": 1, "sub": 2, "mul": 3, "div": 4, "copy_lhs": 5, "copy_rhs": 6}
SCATTER_SUM, SCATTER_MUL, SCATTER_MEAN, SCATTER_MIN, SCATTER_MAX = range(5)
GROUPED_SOFTMAX, GROUPED_LOG_SOFTMAX, GROUPED_LOGSUMEXP = range(3)

EXPORTS = (
    "opsgnn_status_string", "opsgnn_sm_count",
    "opsgnn_csr_plan_bytes", "opsgnn_csr_plan_build", "opsgnn_csr_reduce_workspace_bytes", "opsgnn_csr_reduce",
    "opsgnn_csr_reduce_status", "opsgnn_set_status_sink", "opsgnn_set_wait_polls",
    "opsgnn_csr_integer_mean", "opsgnn_sddmm_workspace_bytes", "opsgnn_sddmm_csr", "opsgnn_sddmm_csr_static",
    "opsgnn_spmm_value_grad",
    "opsgnn_attention_lse_workspace_bytes", "opsgnn_attention_lse", "opsgnn_attention_aggregate",
    "opsgnn_sorted_lse8_workspace_bytes", "opsgnn_sorted_lse8",
    "opsgnn_grouped_prepare", "opsgnn_grouped_forward_prepared",
    "opsgnn_gather_rows", "opsgnn_gather_expand",
    "opsgnn_ind2ptr", "opsgnn_ptr2ind", "opsgnn_csr_validate", "opsgnn_permute_values", "opsgnn_index_stats",
    "opsgnn_index_longest_run",
    "opsgnn_scatter_workspace_bytes", "opsgnn_scatter",
    "opsgnn_grouped_workspace_bytes", "opsgnn_grouped_forward", "opsgnn_grouped_forward_permuted", "opsgnn_grouped_backward",
)


class CsrReduceDesc(Structure):
    _fields_ = [
        ("rows", c_int64), ("src_rows", c_int64), ("feat", c_int64), ("nnz", c_int64), ("batches", c_int64),
        ("value_width", c_int64), ("arg_none", c_int64),
        ("reduce", c_int32), ("extremum", c_int32), ("ptr_type", c_int32), ("col_type", c_int32),
        ("in_type", c_int32), ("out_type", c_int32),
    ]


class SddmmDesc(Structure):
    _fields_ = [
        ("rows", c_int64), ("nnz", c_int64), ("feat", c_int64), ("lhs_rows", c_int64), ("rhs_rows", c_int64),
        ("op", c_int32), ("lhs_target", c_int32), ("rhs_target", c_int32), ("index_type", c_int32),
        ("dtype", c_int32),
    ]


class AttentionDesc(Structure):
    _fields_ = [
        ("rows", c_int64), ("src_rows", c_int64), ("heads", c_int64), ("width", c_int64), ("nnz", c_int64),
        ("negative_slope", ctypes.c_float), ("index_type", c_int32), ("dtype", c_int32),
    ]


class ScatterDesc(Structure):
    _fields_ = [
        ("before", c_int64), ("dim_len", c_int64), ("after", c_int64), ("out_len", c_int64),
        ("index_full", c_int64), ("reduce", c_int32), ("dtype", c_int32), ("has_out", c_int32),
    ]


class GroupedDesc(Structure):
    _fields_ = [
        ("batch", c_int64), ("dim_len", c_int64), ("after", c_int64), ("groups", c_int64),
        ("mode", c_int32), ("dtype", c_int32), ("sorted", c_int32), ("index_type", c_int32),
    ]


_PROTOTYPES = {
    "opsgnn_status_string": (c_char_p, [c_int]),
    "opsgnn_sm_count": (c_int, [POINTER(c_int)]),
    "opsgnn_csr_plan_bytes": (c_int, [c_int64, c_int64, POINTER(c_int64)]),
    "opsgnn_csr_plan_build": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p]),
    "opsgnn_csr_reduce_workspace_bytes": (c_int, [POINTER(CsrReduceDesc), POINTER(c_int64)]),
    "opsgnn_csr_reduce": (c_int, [POINTER(CsrReduceDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "opsgnn_csr_reduce_status": (c_int, [c_void_p, c_void_p, POINTER(c_int64)]),
    "opsgnn_set_status_sink": (c_int, [c_void_p]),
    "opsgnn_set_wait_polls": (c_int, [c_int64]),
    "opsgnn_csr_integer_mean": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p]),
    "opsgnn_sddmm_workspace_bytes": (c_int, [POINTER(SddmmDesc), POINTER(c_int64)]),
    "opsgnn_sddmm_csr": (c_int, [POINTER(SddmmDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                 c_void_p]),
    "opsgnn_sddmm_csr_static": (c_int, [POINTER(SddmmDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "opsgnn_spmm_value_grad": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64,
                                       c_int64, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "opsgnn_gather_rows": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int, POINTER(c_int64),
                                   POINTER(c_void_p), c_int, c_void_p]),
    "opsgnn_sorted_lse8_workspace_bytes": (c_int, [c_int64, POINTER(c_int64)]),
    "opsgnn_sorted_lse8": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p]),
    "opsgnn_attention_lse_workspace_bytes": (c_int, [POINTER(AttentionDesc), POINTER(c_int64)]),
    "opsgnn_attention_lse": (c_int, [POINTER(AttentionDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_int64, c_void_p]),
    "opsgnn_attention_aggregate": (c_int, [POINTER(AttentionDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_int64, c_void_p]),
    "opsgnn_gather_expand": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "opsgnn_ind2ptr": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p]),
    "opsgnn_ptr2ind": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p]),
    "opsgnn_csr_validate": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "opsgnn_permute_values": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "opsgnn_index_stats": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p]),
    "opsgnn_index_longest_run": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_void_p, c_void_p]),
    "opsgnn_scatter_workspace_bytes": (c_int, [POINTER(ScatterDesc), POINTER(c_int64)]),
    "opsgnn_scatter": (c_int, [POINTER(ScatterDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                               c_void_p]),
    "opsgnn_grouped_workspace_bytes": (c_int, [POINTER(GroupedDesc), POINTER(c_int64)]),
    "opsgnn_grouped_forward": (c_int, [POINTER(GroupedDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                       c_void_p]),
    "opsgnn_grouped_prepare": (c_int, [POINTER(GroupedDesc), c_void_p, c_void_p, c_void_p, c_void_p]),
    "opsgnn_grouped_forward_prepared": (c_int, [POINTER(GroupedDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                c_void_p, c_int64, c_void_p]),
    "opsgnn_grouped_forward_permuted": (c_int, [POINTER(GroupedDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                c_int64, c_void_p]),
    "opsgnn_grouped_backward": (c_int, [POINTER(GroupedDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int64, c_void_p]),
}

_LIB = None


def load():
    """Return the loaded library with argument types set; raise ImportError when it is absent."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(LIBRARY_PATH):
        raise ImportError(
            f"{LIBRARY_PATH} is missing: build it with `python ops-gnn_b200/build.py` (there is no CPU fallback)")
    lib = ctypes.CDLL(LIBRARY_PATH)
    for name, (restype, argtypes) in _PROTOTYPES.items():
        if not hasattr(lib, name):
            continue  # optional symbols (for example the fixed-scratch variant) are probed by their users
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _LIB = lib
    return lib


def check(status: int, what: str) -> None:
    if status != 0:
        text = load().opsgnn_status_string(status).decode()
        raise RuntimeError(f"{what} failed: {text} (status {status})")


def torch_dtype_id(dtype) -> int:
    import torch

    table = {
        torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int8: I8, torch.int32: I32,
        torch.int64: I64, torch.uint8: U8, torch.int16: I16, torch.float64: F64,
    }
    return table[dtype]


def _ptr(tensor):
    return None if tensor is None else c_void_p(tensor.data_ptr())


def _stream(device):
    import torch

    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def csr_reduce(ptr, col, val, mat, reduce, *, rows=None, out_dtype=None, extremum=EXTREMUM_IGNORE_NAN,
               arg_none=None, plan=None, return_workspace=False):
    """Drive plan build + opsgnn_csr_reduce on CUDA tensors; returns (out, arg or None).

    ``mat`` is ``[..., N, K]``; ``col`` may be None (segment reduction over consecutive rows).  With
    ``return_workspace`` the launch's workspace comes back as a third value (its head is the status word that
    ``opsgnn_csr_reduce_status`` reads).
    """
    import torch

    lib = load()
    device = mat.device
    m = ptr.numel() - 1 if rows is None else rows
    n, k = mat.size(-2), mat.size(-1)
    batches = 1
    for s in mat.shape[:-2]:
        batches *= s
    nnz = col.numel() if col is not None else int(ptr[-1].item())
    out_dtype = out_dtype or mat.dtype
    width = 0
    if val is not None:
        width = 1
        for s in val.shape[1:]:
            width *= s
    desc = CsrReduceDesc(m, n, k, nnz, batches, width, nnz if arg_none is None else arg_none, reduce, extremum,
                         torch_dtype_id(ptr.dtype), torch_dtype_id(col.dtype if col is not None else ptr.dtype),
                         torch_dtype_id(mat.dtype), torch_dtype_id(out_dtype))
    stream = _stream(device)
    if plan is None:
        nbytes = c_int64()
        check(lib.opsgnn_csr_plan_bytes(m, nnz, ctypes.byref(nbytes)), "csr_plan_bytes")
        plan = torch.empty(nbytes.value // 8, dtype=torch.int64, device=device)
        check(lib.opsgnn_csr_plan_build(_ptr(ptr), desc.ptr_type, m, nnz, _ptr(plan), stream), "csr_plan_build")
    nbytes = c_int64()
    check(lib.opsgnn_csr_reduce_workspace_bytes(ctypes.byref(desc), ctypes.byref(nbytes)), "workspace_bytes")
    workspace = torch.empty(max(nbytes.value, 256), dtype=torch.uint8, device=device)
    out = torch.empty((*mat.shape[:-2], m, k), dtype=out_dtype, device=device)
    arg = None
    if reduce in (REDUCE_MIN, REDUCE_MAX):
        arg = torch.empty(out.shape, dtype=torch.int64, device=device)
    check(lib.opsgnn_csr_reduce(ctypes.byref(desc), _ptr(ptr), _ptr(col), _ptr(val), _ptr(mat), _ptr(out), _ptr(arg),
                                _ptr(plan), _ptr(workspace), workspace.numel(), stream), "csr_reduce")
    if return_workspace:
        return out, arg, workspace
    return out, arg


def csr_reduce_status(workspace) -> int:
    """Number of device-side waits that ran out in the launch that used ``workspace`` (synchronises its stream)."""
    lib = load()
    count = c_int64()
    status = lib.opsgnn_csr_reduce_status(_ptr(workspace), _stream(workspace.device), ctypes.byref(count))
    if status not in (0, -5):
        check(status, "csr_reduce_status")
    return count.value
