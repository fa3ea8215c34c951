"""Failure detection of the bounded device-side waits, without a GPU fault.

Every wait inside the reduce kernels has a poll limit.  A wait that runs out makes its warp count itself in the status
word at the head of the launch's workspace and return; the launch ends normally with rows unwritten and the host turns
the count into an error.  The tests make the waits run out on a healthy GPU by setting the poll limit to zero (the
kernel then gives up before it looks at the barrier; copies already in flight are still awaited with the full limit
before a block exits), check that the report arrives through the C ABI and through the Python API, and that the next
launch with the default limit is correct again.  The reference states the same contract for its device kernels:
a device error surfaces as a status the host reads (the error code of its stream synchronisation after a launch).
"""
import pytest
import torch

import oracle
from conftest import requires_gpu

pytestmark = requires_gpu


def _inputs(device):
    gen = torch.Generator().manual_seed(77)
    rows, cols, feat = 4000, 3000, 256            # 1-KiB rows: the bulk-copy instance with mbarrier waits
    degree = torch.randint(1, 30, (rows,), generator=gen)
    ptr = torch.zeros(rows + 1, dtype=torch.int64)
    ptr[1:] = degree.cumsum(0)
    col = torch.randint(0, cols, (int(ptr[-1]),), generator=gen)
    value = torch.rand(col.numel(), generator=gen)
    mat = torch.randn(cols, feat, generator=gen)
    return (ptr, col, value, mat), [t.to(device) for t in (ptr, col, value, mat)]


def test_stalled_wait_is_reported_through_the_c_abi(cuda_device):
    from ops_gnn import _cabi

    lib = _cabi.load()
    host, dev = _inputs(cuda_device)
    try:
        assert lib.opsgnn_set_wait_polls(0) == 0
        _, _, workspace = _cabi.csr_reduce(*dev, _cabi.REDUCE_SUM, return_workspace=True)
        stalled = _cabi.csr_reduce_status(workspace)          # synchronises: the launch has returned
        assert stalled > 0, "a wait with no polls must be reported"
        assert b"wait" in lib.opsgnn_status_string(-5)
    finally:
        assert lib.opsgnn_set_wait_polls(-1) == 0
        import ops_gnn

        ops_gnn._pybind.device_stall_count(cuda_device.index or 0, True)   # the planner's sink saw the stall too: clear it
    got, _, workspace = _cabi.csr_reduce(*dev, _cabi.REDUCE_SUM, return_workspace=True)
    assert _cabi.csr_reduce_status(workspace) == 0
    want, _ = oracle.csr_spmm_oracle(*host, "sum", torch.float64)
    assert float((got.cpu().double() - want).abs().max()) <= 1e-4


def test_stalled_wait_raises_in_python(cuda_device):
    import ops_gnn
    from ops_gnn.torch_sparse_spmm import csr_spmm

    host, dev = _inputs(cuda_device)
    ops_gnn._pybind.device_stall_count(cuda_device.index or 0, True)   # start from a clean mark
    try:
        ops_gnn._pybind.set_wait_polls(0)
        csr_spmm(*dev, "sum")                                 # returns: the launch ends by itself
        with pytest.raises(RuntimeError, match="device wait timed out"):
            ops_gnn.check_device_status()
        csr_spmm(*dev, "sum")
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="device wait timed out"):
            csr_spmm(*dev, "sum")                             # the next call reports the earlier launch's stall
    finally:
        ops_gnn._pybind.set_wait_polls(-1)
        torch.cuda.synchronize()
        ops_gnn._pybind.device_stall_count(cuda_device.index or 0, True)   # the raising call above launched nothing
    got = csr_spmm(*dev, "sum")
    ops_gnn.check_device_status()
    want, _ = oracle.csr_spmm_oracle(*host, "sum", torch.float64)
    assert float((got.cpu().double() - want).abs().max()) <= 1e-4
