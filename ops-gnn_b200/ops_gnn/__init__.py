"""ops_gnn for NVIDIA B200: sparse message-passing operators behind the ops-gnn Python API.

The native extension is loaded from ``<package>/<target>/_pybind.so`` exactly as the reference does
(python/ops_gnn/__init__.py:27-42 of ops-gnn); the single CUDA build exports the union of the operators the two
Ascend builds expose for this path.  There is no CPU fallback: importing without the built extension fails.
"""
import importlib.util
import os
import sys

import torch

from ._device import select_target
from .typing import OptTensor, Tensor

__version__ = "0.1.0"

try:
    _target = select_target()
    _library = os.path.join(os.path.dirname(__file__), _target, "_pybind.so")
    _spec = importlib.util.spec_from_file_location(__name__ + "._pybind", _library)
    _pybind = importlib.util.module_from_spec(_spec)
    sys.modules[_spec.name] = _pybind
    _spec.loader.exec_module(_pybind)
except (ImportError, OSError, RuntimeError, ValueError, AttributeError) as exc:
    raise ImportError(
        "cannot import the ops_gnn._pybind native extension; the CUDA operators are unavailable. Check that "
        "(1) `python ops-gnn_b200/build.py` has been run for this Python / PyTorch, "
        "(2) libopsgnn_b200.so sits next to _pybind.so, and (3) the GPU is an sm_100a device. "
        f"Original error: {exc}"
    ) from exc

from .ind2ptr import ind2ptr
from .ptr2ind import ptr2ind
from .segment_csr import (
    segment_add_csr, segment_csr, segment_max_csr, segment_mean_csr, segment_min_csr, segment_sum_csr,
)
from .segment_reduce import segment_reduce
from .segment_coo import (
    segment_add_coo, segment_coo, segment_max_coo, segment_mean_coo, segment_min_coo, segment_sum_coo,
)
from .segment_logsumexp import segment_logsumexp
from .gather_csr import gather_csr
from .gather_coo import gather_coo
from .gat_aggregate import gat_aggregate
from .spmm import spmm
from .sddmm_csr import sddmm_csr
from .bspmm import bspmm
from .scatter import (
    native_available, scatter, scatter_add, scatter_max, scatter_mean, scatter_min, scatter_mul, scatter_sum,
)
from .scatter_softmax import scatter_softmax
from .scatter_log_softmax import scatter_log_softmax
from .scatter_logsumexp import scatter_logsumexp
from . import torch_sparse_spmm


def check_device_status(device=None) -> None:
    """Synchronise ``device`` and raise ``RuntimeError`` if a device-side wait of this library ran out since the last look.

    Every wait inside the kernels is bounded; a wait that runs out makes its launch return with rows unwritten and
    leaves a mark the host can read without a fault.  The operators look at the mark on every call (a stall of an
    earlier launch raises there); this function is the explicit form for the end of a step.  No counterpart in the
    reference, whose runtime reports device errors through its stream synchronisation.
    """
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    count = _pybind.device_stall_count(int(index or 0), True)
    if count:
        raise RuntimeError(f"ops_gnn: device wait timed out on cuda:{index} (a bulk-copy wait of the reduce kernel ran "
                           "out of polls; the output of that launch is incomplete)")


__all__ = [
    "check_device_status",
    "ind2ptr",
    "ptr2ind",
    "spmm",
    "bspmm",
    "sddmm_csr",
    "segment_csr", "segment_sum_csr", "segment_add_csr", "segment_mean_csr", "segment_min_csr", "segment_max_csr",
    "segment_reduce",
    "segment_logsumexp",
    "gather_csr", "gather_coo", "gat_aggregate",
    "segment_coo", "segment_sum_coo", "segment_add_coo", "segment_mean_coo", "segment_min_coo", "segment_max_coo",
    "scatter", "scatter_sum", "scatter_add", "scatter_mul", "scatter_mean", "scatter_min", "scatter_max",
    "native_available",
    "scatter_softmax", "scatter_log_softmax", "scatter_logsumexp",
    "torch_sparse_spmm",
    "Tensor",
    "OptTensor",
]
