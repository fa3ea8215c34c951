"""GPU parity driven through the C ABI alone: ctypes -> libopsgnn_b200.so with raw device pointers, no torch extension
in between.  This is the call sequence a foreign-language binding makes (plan bytes, plan build, workspace bytes,
reduce), checked against the CPU oracle."""
import ctypes

import torch

import oracle
from conftest import assert_close, assert_same, requires_gpu

pytestmark = requires_gpu


def _graph(gen, rows=5000, cols=4000):
    degree = torch.randint(0, 30, (rows,), generator=gen)
    degree[11], degree[12] = 20000, 0
    ptr = torch.zeros(rows + 1, dtype=torch.int64)
    ptr[1:] = degree.cumsum(0)
    col = torch.randint(0, cols, (int(ptr[-1]),), generator=gen)
    return ptr, col


def test_csr_reduce_entry_point(cuda_device):
    from ops_gnn import _cabi

    gen = torch.Generator().manual_seed(23)
    ptr, col = _graph(gen)
    value = torch.rand(col.numel(), generator=gen)
    for width in (256, 64, 100):           # bulk ring, narrow rows, ragged width (register gathers)
        mat = torch.randn(4000, width, generator=gen)
        dev = [t.to(cuda_device) for t in (ptr, col, value, mat)]
        got, _ = _cabi.csr_reduce(dev[0], dev[1], dev[2], dev[3], _cabi.REDUCE_SUM)
        want, _ = oracle.csr_spmm_oracle(ptr, col, value, mat, "sum", torch.float64)
        magnitude = torch.zeros_like(want).index_add_(
            0, torch.repeat_interleave(torch.arange(ptr.numel() - 1), ptr[1:] - ptr[:-1]),
            (mat.double()[col] * value.double().unsqueeze(-1)).abs()).clamp(min=1.0)
        assert float(((got.cpu().double() - want).abs() / magnitude).max()) <= 1e-5, f"sum, width {width}"
        best, where = _cabi.csr_reduce(dev[0], dev[1], None, dev[3], _cabi.REDUCE_MAX)
        want, want_arg = oracle.csr_spmm_oracle(ptr, col, None, mat, "max")
        assert_same(best, want, f"max, width {width}")
        assert_same(where, want_arg, f"max positions, width {width}")
    # segment form: no column array, log-sum-exp with fp32 output
    src = torch.randn(int(ptr[-1]), 16, generator=gen)
    got, _ = _cabi.csr_reduce(dev[0], None, None, src.to(cuda_device), _cabi.REDUCE_LOGSUMEXP,
                              extremum=_cabi.EXTREMUM_PROPAGATE_NAN)
    assert_close(got, oracle.segment_logsumexp_oracle(src, ptr).float(), what="segment log-sum-exp")


def test_sddmm_and_conversions_entry_points(cuda_device):
    from ops_gnn import _cabi

    lib = _cabi.load()
    gen = torch.Generator().manual_seed(29)
    ptr, col = _graph(gen, rows=3000, cols=3000)
    nnz = col.numel()
    a, b = torch.randn(3000, 64, generator=gen), torch.randn(3000, 64, generator=gen)
    d_ptr, d_col, d_a, d_b = (t.to(cuda_device) for t in (ptr, col, a, b))
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    desc = _cabi.SddmmDesc(3000, nnz, 64, 3000, 3000, _cabi.SDDMM_OPS["dot"], 0, 2, _cabi.I64, _cabi.F32)
    nbytes = ctypes.c_int64()
    _cabi.check(lib.opsgnn_sddmm_workspace_bytes(ctypes.byref(desc), ctypes.byref(nbytes)), "sddmm_workspace_bytes")
    workspace = torch.empty(max(nbytes.value, 8), dtype=torch.uint8, device=cuda_device)
    out = torch.empty(nnz, device=cuda_device)
    _cabi.check(lib.opsgnn_sddmm_csr(ctypes.byref(desc), d_ptr.data_ptr(), d_col.data_ptr(), d_a.data_ptr(), d_b.data_ptr(),
                                     out.data_ptr(), workspace.data_ptr(), workspace.numel(), stream), "sddmm_csr")
    assert_close(out, oracle.sddmm_oracle(ptr, col, a, b, "dot", "u", "v"), what="sddmm dot")

    rows = torch.repeat_interleave(torch.arange(3000), ptr[1:] - ptr[:-1])
    d_rows = rows.to(cuda_device)
    made_ptr = torch.empty(3001, dtype=torch.int64, device=cuda_device)
    _cabi.check(lib.opsgnn_ind2ptr(d_rows.data_ptr(), nnz, made_ptr.data_ptr(), 3000, stream), "ind2ptr")
    assert_same(made_ptr, ptr, "ind2ptr")
    made_rows = torch.empty(nnz, dtype=torch.int64, device=cuda_device)
    _cabi.check(lib.opsgnn_ptr2ind(d_ptr.data_ptr(), 3000, made_rows.data_ptr(), nnz, stream), "ptr2ind")
    assert_same(made_rows, rows, "ptr2ind")


def test_gather_rows_entry_point(cuda_device):
    """opsgnn_gather_rows through ctypes: segmented outputs in separate buffers, both index dtypes, row widths from one
    16-byte vector to beyond one 512-byte piece, capped and uncapped grids; bit-exact against an index_select."""
    from ops_gnn import _cabi

    lib = _cabi.load()
    gen = torch.Generator().manual_seed(31)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for dtype, width in ((torch.float32, 256), (torch.float32, 4), (torch.bfloat16, 200), (torch.float16, 520), (torch.float32, 100)):
        src = torch.randn(3000, width, generator=gen).to(dtype).to(cuda_device)
        for index_dtype, cap in ((torch.int64, 0), (torch.int32, 8), (torch.int64, 1)):
            index = torch.randint(0, 3000, (7001,), generator=gen).to(index_dtype).to(cuda_device)
            counts = [0, 2500, 1, 0, 4500]
            outs = [torch.full((n, width), 7, dtype=dtype, device=cuda_device) for n in counts]
            rows = (ctypes.c_int64 * len(counts))(*counts)
            bases = (ctypes.c_void_p * len(counts))(*[o.data_ptr() if o.numel() else None for o in outs])
            _cabi.check(lib.opsgnn_gather_rows(src.data_ptr(), index.data_ptr(), _cabi.torch_dtype_id(index_dtype), 7001, 3000,
                                               width * src.element_size(), len(counts), rows, bases, cap, stream), "gather_rows")
            assert_same(torch.cat(outs), src[index.long()], f"gather {dtype} width {width} cap {cap}")
    bad = (ctypes.c_int64 * 1)(5)
    base = (ctypes.c_void_p * 1)(outs[1].data_ptr())
    assert lib.opsgnn_gather_rows(src.data_ptr(), index.data_ptr(), _cabi.I64, 6, 3000, 400, 1, bad, base, 0, stream) == -1
    assert lib.opsgnn_gather_rows(src.data_ptr(), index.data_ptr(), _cabi.I64, 5, 3000, 100, 1, bad, base, 0, stream) == -1


def test_sorted_lse8_entry_point(cuda_device):
    """opsgnn_sorted_lse8 through ctypes: log-sum-exp per group of an [n, 8] matrix under sorted labels (both index
    dtypes, groups inside and across 128-row chunks, empty groups), against the float64 oracle; argument errors."""
    from ops_gnn import _cabi

    lib = _cabi.load()
    gen = torch.Generator().manual_seed(41)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    lengths = torch.cat([torch.randint(0, 60, (2000,), generator=gen), torch.tensor([5000, 0, 1])])
    labels = torch.repeat_interleave(torch.arange(lengths.numel()), lengths).contiguous()
    n, groups = labels.numel(), lengths.numel()
    values = torch.randn(n, 8, generator=gen) * 5
    want = oracle.grouped_logsumexp_oracle(values, labels, 0, groups).float()
    nbytes = ctypes.c_int64()
    _cabi.check(lib.opsgnn_sorted_lse8_workspace_bytes(n, ctypes.byref(nbytes)), "sorted_lse8_workspace_bytes")
    workspace = torch.empty(nbytes.value, dtype=torch.uint8, device=cuda_device)
    d_values = values.to(cuda_device)
    for index_dtype in (torch.int64, torch.int32):
        d_labels = labels.to(index_dtype).to(cuda_device)
        lse = torch.full((groups, 8), 7.0, device=cuda_device)
        _cabi.check(lib.opsgnn_sorted_lse8(d_labels.data_ptr(), _cabi.torch_dtype_id(index_dtype), d_values.data_ptr(),
                                           lse.data_ptr(), n, groups, workspace.data_ptr(), workspace.numel(), stream),
                    "sorted_lse8")
        assert_close(lse, want, what=f"sorted_lse8 {index_dtype}")
    assert lib.opsgnn_sorted_lse8(d_labels.data_ptr(), _cabi.I32, d_values.data_ptr(), lse.data_ptr(), n, groups,
                                  workspace.data_ptr(), 16, stream) == -3   # OPSGNN_ERR_WORKSPACE
    assert lib.opsgnn_sorted_lse8(d_labels.data_ptr(), 99, d_values.data_ptr(), lse.data_ptr(), n, groups,
                                  workspace.data_ptr(), workspace.numel(), stream) == -1
