"""Behavioural contract of the drop-in boundary on CUDA, ported from the reference's own contract tests: stream
ordering (test/conftest.py:217-230), `out=` identity and alias rejection (conftest.py:107-135), non-contiguous inputs
(test/unified_spmm/arch22/test_unified_spmm.py:687-706), reuse and invalidation of cached CSR facts after writes the
version counter does and does not see (:656-682, :757-768, :856-876), error precedence (:915-940), the COO front end
(test/torch_sparse_spmm/arch35/test_torch_sparse_spmm.py:609-640), the torch_sparse dispatcher registration
(python/ops_gnn/torch_sparse_spmm.py:406-431) and gradients against a float64 reference
(test_torch_sparse_spmm.py:164-181, 467-515).  Inputs are the reference's: a 3-row graph, 17 features."""
import math

import pytest
import torch

import oracle
from conftest import assert_close, assert_same, requires_gpu

pytestmark = requires_gpu

PATHS = ("fp16", "fp32", "batched_fp16", "copy_rhs")


def inputs(path, device, noncontiguous=False):
    ptr = torch.tensor([0, 2, 3, 3], dtype=torch.int64)
    idx = torch.tensor([0, 1, 0], dtype=torch.int64)
    dtype = torch.float16 if "fp16" in path else torch.float32
    shape = (3, 2, 17) if path == "batched_fp16" else (3, 17)
    x = (torch.arange(math.prod(shape)).reshape(shape) % 7 - 3).to(dtype)
    if noncontiguous:
        def strided(value):
            storage = torch.empty(value.shape[:-1] + (value.shape[-1] * 2,), device=device, dtype=value.dtype)
            view = storage[..., ::2]
            view.copy_(value)
            return view
        return tuple(strided(value) for value in (ptr, idx, x))
    return ptr.to(device), idx.to(device), x.to(device)


def invoke(path, ptr, idx, x, reduce, out=None):
    import ops_gnn

    operation = ops_gnn.bspmm if path == "batched_fp16" else ops_gnn.spmm
    return operation(ptr, idx, x, reduce=reduce, op="copy_rhs" if path == "copy_rhs" else "copy_lhs", out=out)


def assert_result(result, path, ptr, idx, x, reduce):
    expected = oracle.spmm_copy_oracle(ptr.cpu(), idx.cpu(), x.cpu(), reduce, "copy_rhs" if path == "copy_rhs" else "copy_lhs")
    assert_same(result, expected, f"{path} {reduce}")


# ---- streams, out=, special values --------------------------------------------------------------------------------------
@pytest.mark.parametrize("reduce", ["sum", "max", "min"])
def test_nondefault_stream_ordering(cuda_device, reduce):
    import ops_gnn

    stream = torch.cuda.Stream()
    ptr = torch.tensor([0, 1, 2], device=cuda_device)
    idx = torch.tensor([1, 0], device=cuda_device)
    x = torch.ones(2, 17, device=cuda_device, dtype=torch.float16)
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        x = x * -3                                   # produced on the side stream: the operator must run after it, there
        result = ops_gnn.spmm(ptr, idx, x, reduce=reduce) + 2
    torch.cuda.current_stream().wait_stream(stream)
    assert_same(result, torch.full((2, 17), -1, dtype=torch.float16), reduce)


def test_plan_built_on_one_stream_is_ordered_on_another(cuda_device):
    """A merge-path plan is cached per graph; the stream that reuses it must wait for the stream that built it."""
    from ops_gnn.torch_sparse_spmm import csr_spmm

    gen = torch.Generator().manual_seed(5)
    rows = 200000
    degree = torch.randint(0, 12, (rows,), generator=gen)
    ptr = torch.zeros(rows + 1, dtype=torch.int64)
    ptr[1:] = degree.cumsum(0)
    col = torch.randint(0, rows, (int(ptr[-1]),), generator=gen)
    mat = torch.randn(rows, 64, generator=gen)
    d_ptr, d_col, d_mat = ptr.to(cuda_device), col.to(cuda_device), mat.to(cuda_device)
    forward = __import__("ops_gnn")._pybind.torch_sparse_spmm.forward
    torch.cuda.synchronize()
    first, second = torch.cuda.Stream(), torch.cuda.Stream()
    with torch.cuda.stream(first):
        one = forward(d_ptr, d_col, None, d_mat, 0, 0)[0]           # builds and caches the plan on `first`
    with torch.cuda.stream(second):
        two = forward(d_ptr, d_col, None, d_mat, 0, 0)[0]           # back to back: reuses it on `second`
    torch.cuda.synchronize()
    assert torch.equal(one, two)
    want, _ = oracle.csr_spmm_oracle(ptr, col, None, mat, "sum")
    assert_close(one, want, what="sum", magnitude=oracle.csr_spmm_oracle(ptr, col, None, mat.abs(), "sum")[0])
    assert csr_spmm(d_ptr, d_col, None, d_mat, "sum").shape == one.shape


@pytest.mark.parametrize("reduce", ["sum", "max", "min"])
def test_special_values_and_supplied_out(cuda_device, reduce):
    import ops_gnn

    ptr, idx = torch.tensor([0, 2, 2]), torch.tensor([0, 1])
    x = torch.tensor([[float("inf"), float("nan")], [-float("inf"), 2]], dtype=torch.float16)
    out = torch.empty((2, 2), dtype=torch.float16, device=cuda_device)
    result = ops_gnn.spmm(ptr.to(cuda_device), idx.to(cuda_device), x.to(cuda_device), reduce=reduce, out=out)
    assert result.data_ptr() == out.data_ptr(), "the supplied out tensor is returned"
    assert_same(result, oracle.spmm_copy_oracle(ptr, idx, x, reduce), reduce)


def test_out_must_not_alias_inputs_and_bad_csr(cuda_device):
    import ops_gnn

    ptr, idx, x = inputs("fp16", cuda_device)
    with pytest.raises(RuntimeError, match="alias"):
        ops_gnn._pybind.spmm_sum_csr(ptr, idx, x, x)
    wide = x.float()
    shares_storage = torch.empty(0, device=cuda_device).set_(wide.untyped_storage(), 0, (3, 17), (17, 1))
    with pytest.raises(RuntimeError, match="alias"):
        ops_gnn._pybind.unified_spmm_csr(ptr, idx, wide, "copy_lhs", "sum", shares_storage)
    a, b = torch.randn(3, 17, device=cuda_device), torch.randn(3, 17, device=cuda_device)
    with pytest.raises(RuntimeError, match="sddmm_csr"):
        ops_gnn.sddmm_csr(ptr, idx, a, b, "mul", "u", "v", out=a[:3])
    for ptr_values, index_values in (([1, 2], [0]), ([0, 2], [0]), ([0, 2, 1, 2], [0, 1]), ([0, 1], [5])):
        with pytest.raises(RuntimeError, match="spmm"):
            ops_gnn.spmm(torch.tensor(ptr_values, device=cuda_device), torch.tensor(index_values, device=cuda_device),
                         torch.ones(2, 17, dtype=torch.float16, device=cuda_device))
    empty = ops_gnn.spmm(torch.zeros(4, dtype=torch.int64, device=cuda_device), torch.empty(0, dtype=torch.int64, device=cuda_device),
                         torch.empty(5, 17, dtype=torch.float16, device=cuda_device))
    assert_same(empty, torch.zeros(3, 17, dtype=torch.float16), "rows without edges")


@pytest.mark.parametrize("path", PATHS)
def test_noncontiguous_inputs_inference_and_out(cuda_device, path):
    for inference, noncontiguous, supplied_out in ((True, False, False), (False, True, False), (False, False, True)):
        with torch.inference_mode(inference):
            ptr, idx, x = inputs(path, cuda_device, noncontiguous)
            out = torch.empty((3,) + tuple(x.shape[1:]), device=cuda_device, dtype=x.dtype) if supplied_out else None
            for _ in range(3):
                result = invoke(path, ptr, idx, x, "max", out)
            if supplied_out:
                assert result.data_ptr() == out.data_ptr()
            x[0].fill_(float("nan"))
            assert_result(invoke(path, ptr, idx, x, "max", out), path, ptr, idx, x, "max")
            idx[0] = -1
            if path != "copy_rhs":
                with pytest.raises(RuntimeError, match="indices out of range"):
                    invoke(path, ptr, idx, x, "max", out)


# ---- cached CSR facts: reuse, and invalidation by writes of every kind ---------------------------------------------------
@pytest.mark.parametrize("path", PATHS)
def test_back_to_back_calls_reuse_cached_facts(cuda_device, path):
    import ops_gnn

    native = ops_gnn._pybind
    ptr, idx, x = inputs(path, cuda_device)
    native.clear_native_caches()
    invoke(path, ptr, idx, x, "sum")
    warm, clock = native.native_cache_sizes(), native.write_clock()
    assert warm[0] >= 1 and warm[1] >= 1, "the first call caches a plan and the validation facts"
    for _ in range(3):
        result = invoke(path, ptr, idx, x, "sum")
    assert native.native_cache_sizes() == warm and native.write_clock() == clock, "back-to-back calls derive nothing again"
    unrelated = torch.ones(1, device=cuda_device)             # any foreign operator may have written anything
    assert native.write_clock() != clock
    result = invoke(path, ptr, idx, x, "sum")
    after = native.native_cache_sizes()
    assert after[0] == warm[0] + 1 and after[1] == warm[1] + 1, "after foreign work the facts are derived again"
    assert unrelated.item() == 1
    assert_result(result, path, ptr, idx, x, "sum")


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("field,message", [
    ("endpoint", "indptr must start at zero and end at nnz"),
    ("range", "indptr values out of range"),
    ("order", "indptr must be non-decreasing"),
    ("index", "indices out of range"),
])
@pytest.mark.parametrize("alias", ["inplace", "data_alias", "storage_alias"])
def test_warm_csr_mutation(cuda_device, path, field, message, alias):
    if path == "copy_rhs" and field == "index":
        pytest.skip("copy_rhs does not dereference source index values")
    ptr, idx, x = inputs(path, cuda_device)
    for _ in range(3):
        invoke(path, ptr, idx, x, "sum")
    target = idx if field == "index" else ptr
    if alias == "data_alias":
        target = target.data                                   # shares storage, NOT the version counter
    elif alias == "storage_alias":
        target = torch.empty(0, device=cuda_device, dtype=target.dtype).set_(
            target.untyped_storage(), target.storage_offset(), target.size(), target.stride())
    if field == "endpoint":
        target[0] = 1
    elif field == "range":
        target[1] = 4
    elif field == "order":
        target[1], target[2] = 3, 2
    else:
        target[0] = -1
    for _ in range(2):
        with pytest.raises(RuntimeError, match=message):
            invoke(path, ptr, idx, x, "sum")


@pytest.mark.parametrize("path", ["fp16", "fp32", "batched_fp16"])
def test_native_out_write_invalidates_cached_facts(cuda_device, path):
    """A kernel of this library writes, through `out=`, into memory that an EARLIER call's index tensor aliases; no
    version counter moves.  The next call on the earlier graph must see the new contents."""
    import ops_gnn

    native = ops_gnn._pybind
    ptr, idx, x = inputs(path, cuda_device)
    writer = torch.tensor([[99], [98], [97]], device=cuda_device)                  # becomes idx = [99, 98, 97]
    restore = torch.tensor([[1], [0], [1]], device=cuda_device)
    writer_ptr = torch.arange(4, device=cuda_device)
    alias = idx.data.view(3, 1)                                                    # made before the facts are cached
    for _ in range(3):
        invoke(path, ptr, idx, x, "max")
    clock = native.write_clock()
    native.segment_csr_value(writer, writer_ptr, alias, "sum")                     # no ATen call in between: only the
    assert native.write_clock() != clock, "a planner that writes caller memory moves the write clock"   # planner's note
    with pytest.raises(RuntimeError, match="indices out of range"):
        invoke(path, ptr, idx, x, "max")
    native.segment_csr_value(restore, writer_ptr, alias, "sum")
    assert_result(invoke(path, ptr, idx, x, "max"), path, ptr, idx, x, "max")


@pytest.mark.parametrize("path", PATHS)
def test_error_priority_after_warm_facts(cuda_device, path):
    ptr, idx, x = inputs(path, cuda_device)
    for _ in range(3):
        invoke(path, ptr, idx, x, "sum")
    ptr.data.copy_(torch.tensor([1, 4, 2, 3], device=cuda_device))   # endpoint, range and order fail together
    idx.data.fill_(-1)                                               # and so do the indices
    for _ in range(2):
        with pytest.raises(RuntimeError, match="indptr must start at zero and end at nnz"):
            invoke(path, ptr, idx, x, "sum")
    for middle in (-1, 4):
        ptr.data.copy_(torch.tensor([0, middle, 2, 3], device=cuda_device))
        for _ in range(2):
            with pytest.raises(RuntimeError, match="indptr values out of range"):
                invoke(path, ptr, idx, x, "sum")


@pytest.mark.parametrize("path", ["fp16", "copy_rhs"])
def test_many_tensor_identities(cuda_device, path):
    cases = [inputs(path, cuda_device) for _ in range(70)]            # more identities than the caches hold
    for ptr, idx, x in cases:
        invoke(path, ptr, idx, x, "max")
    ptr, idx, x = cases[0]
    del cases
    x.data[0].fill_(float("nan"))
    assert_result(invoke(path, ptr, idx, x, "max"), path, ptr, idx, x, "max")


def test_sorted_index_fact_is_not_reused_after_an_unseen_write(cuda_device):
    """scatter_softmax caches "this label vector is sorted"; a write through `.data` must not leave it stale."""
    import ops_gnn

    gen = torch.Generator().manual_seed(3)
    labels = torch.arange(64).repeat_interleave(4)
    src = torch.randn(256, 8, generator=gen)
    d_labels, d_src = labels.to(cuda_device), src.to(cuda_device)
    for _ in range(2):
        got = ops_gnn.scatter_softmax(d_src, d_labels, 0, 64)
    assert_close(got, oracle.grouped_softmax_oracle(src, labels, 0, 64).float(), what="sorted")
    shuffled = labels[torch.randperm(256, generator=gen)]
    d_labels.data.copy_(shuffled.to(cuda_device))
    got = ops_gnn.scatter_softmax(d_src, d_labels, 0, 64)
    assert_close(got, oracle.grouped_softmax_oracle(src, shuffled, 0, 64).float(), what="after an unseen shuffle")


# ---- COO front end and support operators -----------------------------------------------------------------------------------
def _coo_inputs(device):
    index = torch.tensor([[2, 0, 0, 1], [1, 2, 0, 1]], dtype=torch.int64).to(device)
    value = torch.tensor([2.0, -1.0, 3.0, 4.0]).to(device)
    mat = torch.arange(12, dtype=torch.float32).reshape(3, 4).to(device)
    return index, value, mat


def _coo_expected(index, value, mat, rows=3):
    index, value, mat = index.cpu(), value.cpu(), mat.cpu()
    return torch.zeros((rows, mat.shape[1]), dtype=mat.dtype).index_add(0, index[0], value[:, None] * mat[index[1]])


def test_coo_front_end_observes_each_input_mutation(cuda_device):
    from ops_gnn import torch_sparse_spmm as front

    def check(index, value, mat):
        actual = front.coo_spmm(index, value, 3, 3, mat)
        assert_close(actual, _coo_expected(index, value, mat), what="coo_spmm")
        return actual

    front.clear_validation_cache()
    index, value, mat = _coo_inputs(cuda_device)
    saved = check(index, value, mat).clone()
    check(index, value, mat)
    assert front.validation_cache_info().coo_entries == 1, "the unsorted layout is cached once"
    value.add_(2)
    check(index, value, mat)
    mat.mul_(2)
    check(index, value, mat)
    index[1, 0] = 2
    check(index, value, mat)
    index[0, 0] = 0                                            # rows become sorted: no permutation any more
    check(index, value, mat)
    assert not torch.equal(saved, check(index, value, mat))
    with pytest.raises(ValueError, match="COO row out of range"):
        front.coo_spmm(torch.tensor([[3], [0]], device=cuda_device), None, 3, 3, mat)
    with pytest.raises(ValueError, match="int64"):
        front.coo_spmm(index.int(), value, 3, 3, mat)


def test_coo_to_csr_convert_and_permute_values(cuda_device):
    from ops_gnn import _pybind
    from ops_gnn import torch_sparse_spmm as front

    gen = torch.Generator().manual_seed(19)
    rows, cols, edges = 500, 300, 4000
    row = torch.randint(0, rows, (edges,), generator=gen)
    col = torch.randint(0, cols, (edges,), generator=gen)
    for dtype, width in ((torch.float32, ()), (torch.float16, (5,)), (torch.bfloat16, (3,)), (torch.int8, ())):
        value = (torch.randn((edges,) + width, generator=gen) * 4).to(dtype)
        index = torch.stack((row, col)).to(cuda_device)
        ptr, out_col, out_value = front.coo_to_csr(index, value.to(cuda_device), rows)
        order = torch.argsort(row, stable=True)
        assert_same(ptr, oracle.ind2ptr_oracle(row[order], rows), "coo_to_csr rowptr")
        assert_same(out_col, col[order], "coo_to_csr col")
        assert_same(out_value, value[order], f"coo_to_csr value {dtype}")
        assert_same(_pybind.torch_sparse_spmm.permute_values(value.to(cuda_device), order.to(cuda_device)), value[order],
                    f"permute_values {dtype}")
    sorted_row = row.sort().values.to(cuda_device)
    ptr = _pybind.torch_sparse_spmm.convert(sorted_row, rows + 1, True)
    assert_same(ptr, oracle.ind2ptr_oracle(sorted_row.cpu(), rows), "convert to pointers")
    assert_same(_pybind.torch_sparse_spmm.convert(ptr, edges, False), sorted_row.cpu(), "convert to rows")
    mat = torch.randn(cols, 33, generator=gen)
    weights = torch.randn(edges, generator=gen)
    got = front.coo_spmm(torch.stack((row, col)).to(cuda_device), weights.to(cuda_device), rows, cols, mat.to(cuda_device))
    terms = weights.double()[:, None] * mat.double()[col]
    want = torch.zeros(rows, 33, dtype=torch.float64).index_add_(0, row, terms)
    assert_close(got, want.float(), what="coo_spmm random", magnitude=torch.zeros(rows, 33, dtype=torch.float64).index_add_(0, row, terms.abs()))


# ---- torch_sparse dispatcher registration -------------------------------------------------------------------------------------
_SCHEMAS = (
    "spmm_sum(Tensor? row, Tensor rowptr, Tensor col, Tensor? value, Tensor? colptr, Tensor? csr2csc, Tensor mat) -> Tensor",
    "spmm_mean(Tensor? row, Tensor rowptr, Tensor col, Tensor? value, Tensor? rowcount, Tensor? colptr, Tensor? csr2csc, Tensor mat) -> Tensor",
    "spmm_min(Tensor rowptr, Tensor col, Tensor? value, Tensor mat) -> (Tensor, Tensor)",
    "spmm_max(Tensor rowptr, Tensor col, Tensor? value, Tensor mat) -> (Tensor, Tensor)",
    "ind2ptr(Tensor ind, int M) -> Tensor",
    "ptr2ind(Tensor ptr, int E) -> Tensor",
)
_DEFINED = []


@pytest.fixture(scope="module")
def torch_sparse_operators():
    """The six operator schemas of torch_sparse's SpMM path, defined here when the package is absent, then implemented
    for CUDA by the library's own registration code."""
    from ops_gnn import torch_sparse_spmm as front

    if front.torch_sparse is None and not _DEFINED:
        library = torch.library.Library("torch_sparse", "DEF")
        for schema in _SCHEMAS:
            library.define(schema)
        _DEFINED.append(library)
        registered = front.register_dispatcher_kernels()
        assert set(registered["CUDA"]) == {"spmm_sum", "spmm_mean", "spmm_min", "spmm_max", "ind2ptr", "ptr2ind"}
        assert set(registered["AutogradCUDA"]) == set(registered["CUDA"])
    return torch.ops.torch_sparse


def _small_graph(device, dtype=torch.float32):
    p = torch.tensor([0, 3, 3, 5])
    c = torch.tensor([1, 0, 1, 0, 1])
    r = torch.tensor([0, 0, 0, 2, 2])
    torch.manual_seed(617)
    v = (torch.rand(5) * 2 - 1).to(dtype)
    b = (torch.rand(2, 2, 7) * 2 - 1).to(dtype)
    return p, c, r, v, b


def test_registered_operators(cuda_device, torch_sparse_operators):
    ops = torch_sparse_operators
    p, c, r, v, b = _small_graph(cuda_device)
    pn, cn, rn, vn, bn = (t.to(cuda_device) for t in (p, c, r, v, b))
    counts = (p[1:] - p[:-1]).to(cuda_device)
    want, _ = oracle.csr_spmm_oracle(p, c, v, b, "sum")
    assert_close(ops.spmm_sum(rn, pn, cn, vn, None, None, bn), want, what="registered spmm_sum")
    want, _ = oracle.csr_spmm_oracle(p, c, v, b, "mean")
    assert_close(ops.spmm_mean(rn, pn, cn, vn, counts, None, None, bn), want, what="registered spmm_mean")
    for name in ("min", "max"):
        out, arg = getattr(ops, "spmm_" + name)(pn, cn, vn, bn)
        want, want_arg = oracle.csr_spmm_oracle(p, c, v, b, name)
        assert_same(out, want, "registered spmm_" + name)
        assert_same(arg, want_arg, "registered spmm_" + name + " arg")
    assert_same(ops.ind2ptr(rn, 3), p, "registered ind2ptr")
    assert_same(ops.ptr2ind(pn, 5), r, "registered ptr2ind")


# ---- gradients against a float64 reference ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("frontend,reduce", [("coo", "sum"), ("registered", "sum"), ("registered", "mean"), ("helper", "sum"),
                                             ("helper", "mean")])
def test_gradients_against_float64(cuda_device, torch_sparse_operators, dtype, frontend, reduce):
    from ops_gnn import torch_sparse_spmm as front

    p, c, r, v, b = _small_graph(cuda_device, dtype)
    vn, bn = v.to(cuda_device).requires_grad_(), b.to(cuda_device).requires_grad_()
    pn, cn, rn = p.to(cuda_device), c.to(cuda_device), r.to(cuda_device)
    perm = cn.argsort(stable=True)
    colptr = torch.tensor([0, 2, 5], device=cuda_device)
    counts = (p[1:] - p[:-1]).to(cuda_device)
    if frontend == "coo":
        out = front.coo_spmm(torch.stack((rn, cn)), vn, 3, 2, bn)
    elif frontend == "helper":
        out = front.csr_spmm(pn, cn, vn, bn, reduce)
    elif reduce == "sum":
        out = torch_sparse_operators.spmm_sum(rn, pn, cn, vn, colptr, perm, bn)
    else:
        out = torch_sparse_operators.spmm_mean(rn, pn, cn, vn, counts, colptr, perm, bn)
    upstream = (torch.rand(out.shape) * 2 - 1).to(dtype)
    out.backward(upstream.to(cuda_device))
    rv, rb = v.double().requires_grad_(), b.double().requires_grad_()
    reference, _ = oracle.csr_spmm_oracle(p, c, rv, rb, reduce, torch.float64)
    reference.backward(upstream.double())
    assert_close(vn.grad, rv.grad.to(dtype), what=f"d value {frontend} {reduce} {dtype}")
    assert_close(bn.grad, rb.grad.to(dtype), what=f"d mat {frontend} {reduce} {dtype}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("reduce", ["sum", "mean"])
@pytest.mark.parametrize("weighted,feature_values", [(False, False), (True, False), (True, True)])
def test_backward_batched_and_feature_weights(cuda_device, dtype, reduce, weighted, feature_values):
    from ops_gnn.torch_sparse_spmm import csr_spmm

    torch.manual_seed(41)
    ptr = torch.tensor([0, 3, 3, 4, 7])
    col = torch.tensor([2, 0, 2, 1, 3, 0, 1])
    mat = torch.randn(2, 3, 4, 17).to(dtype)
    v = torch.randn((7, 17) if feature_values else (7,)).to(dtype)
    vm = v.to(cuda_device).requires_grad_() if weighted else None
    mm = mat.to(cuda_device).requires_grad_()
    result = csr_spmm(ptr.to(cuda_device), col.to(cuda_device), vm, mm, reduce, output_dtype=torch.float32)
    weight = torch.randn(result.shape)
    (result * weight.to(cuda_device)).sum().backward()
    rv = v.double().requires_grad_() if weighted else None
    rm = mat.double().requires_grad_()
    reference, _ = oracle.csr_spmm_oracle(ptr, col, rv, rm, reduce, torch.float64)
    (reference * weight.double()).sum().backward()
    assert_close(mm.grad, rm.grad.to(dtype), what=f"d mat {dtype} {reduce}")
    if weighted:
        assert_close(vm.grad, rv.grad.to(dtype), what=f"d value {dtype} {reduce}")


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
@pytest.mark.parametrize("reduce", ["sum", "mean", "max", "min"])
def test_binary_message_gradients(cuda_device, op, reduce):
    """`bspmm` with a binary message is a differentiable composition: gradients against the same composition in float64."""
    import ops_gnn

    gen = torch.Generator().manual_seed(53)
    ptr = torch.tensor([0, 3, 3, 5, 9])
    col = torch.tensor([1, 0, 2, 0, 1, 3, 3, 0, 2])
    x = torch.randn(4, 3, 6, generator=gen)
    rhs = torch.randn(9, 3, 1, generator=gen) + 3.0                  # away from zero: `div` stays well conditioned
    xn, rn = x.to(cuda_device).requires_grad_(), rhs.to(cuda_device).requires_grad_()
    out = ops_gnn.bspmm(ptr.to(cuda_device), col.to(cuda_device), xn, op, reduce, rhs=rn)
    upstream = torch.randn(out.shape, generator=gen)
    out.backward(upstream.to(cuda_device))
    xr, rr = x.double().requires_grad_(), rhs.double().requires_grad_()
    lhs = xr[col]
    message = {"add": lhs + rr, "sub": lhs - rr, "mul": lhs * rr, "div": lhs / rr}[op]
    rows = torch.repeat_interleave(torch.arange(4), ptr[1:] - ptr[:-1])
    if reduce in ("sum", "mean"):
        want = torch.zeros(4, 3, 6, dtype=torch.float64).index_add(0, rows, message)
        if reduce == "mean":
            want = want / (ptr[1:] - ptr[:-1]).clamp(min=1).double().reshape(4, 1, 1)
    else:
        want = torch.zeros(4, 3, 6, dtype=torch.float64).scatter_reduce(
            0, rows.reshape(-1, 1, 1).expand_as(message), message, "amax" if reduce == "max" else "amin", include_self=False)
    assert_close(out, want.float(), what=f"{op} {reduce}")
    want.backward(upstream.double())
    assert_close(xn.grad, xr.grad.float(), what=f"d x {op} {reduce}")
    assert_close(rn.grad, rr.grad.float(), what=f"d rhs {op} {reduce}")
