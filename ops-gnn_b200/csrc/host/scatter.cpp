// Launch planner of scatter_forward (csrc/npu/scatter/op_host/scatter.cpp:242-267 of the reference).
// src is viewed as [before, dim_len, after]; the index is either one entry per position along `dim` or has src's
// full shape; `out` is pre-filled by the Python front-end (zeros, ones, dtype extremes, or the caller's tensor) and is
// reduced into in place.  float64 and int64, which the reference sends to a synchronous CPU fallback, run natively.
#include <pybind11/pybind11.h>

#include "ops.h"

namespace opsgnn {

namespace {

// Extrema without atomics: sort the labels once (a stable argsort, cached with the other facts of the label vector),
// then one launch of the CSR reduce engine whose "columns" are the permutation - a gather is what it does best.  A
// stable sort keeps the source order inside a group, so "the last edge among ties" of the engine's seeded rule is the
// largest source position, which is what scatter reports (csrc/npu/scatter/op_kernel/arch35/scatter_kernel_minmax.h:
// 116-147 of the reference does a second sweep for it).  Floating dtypes, a compact index along the leading dimension,
// no caller-seeded output; returns false (nothing launched) for anything else, and the atomic kernels take over.
// `out` is [groups, ...] contiguous, `arg` int64 of the same shape.
bool SortedExtremum(const at::Tensor& src, const at::Tensor& index, const at::Tensor& out, const at::Tensor& arg, int64_t dim_len,
                    int64_t after, bool is_min)
{
    const bool floating = src.scalar_type() == at::kFloat || src.scalar_type() == at::kHalf || src.scalar_type() == at::kBFloat16;
    if (!floating || dim_len <= 0 || after <= 0 || dim_len >= 2147483647LL || out.numel() == 0) {
        return false;
    }
    const int64_t groups = out.numel() / after;
    const LabelFacts facts = LabelFactsOf(index, true);
    if (facts.low < 0 || facts.high >= groups || !(facts.sorted || facts.perm.defined())) {
        return false;
    }
    at::Tensor ordered = facts.sorted ? index : index.index_select(0, facts.perm);
    at::Tensor ptr = at::empty({groups + 1}, index.options());
    CheckStatus(opsgnn_ind2ptr(ordered.const_data_ptr<int64_t>(), dim_len, ptr.data_ptr<int64_t>(), groups, CurrentStream(out)),
                "scatter");
    CsrReduceCall call;
    call.ptr = ptr;
    if (!facts.sorted) {
        call.col = facts.perm;
    }
    call.mat = src.view({dim_len, after});
    call.out = out.view({groups, after});
    call.arg = arg.view({groups, after});
    call.rows = groups;
    call.src_rows = dim_len;
    call.feat = after;
    call.nnz = dim_len;
    call.arg_none = dim_len;
    call.reduce = is_min ? OPSGNN_REDUCE_MIN : OPSGNN_REDUCE_MAX;
    call.extremum = OPSGNN_EXTREMUM_SEEDED_LAST;
    RunCsrReduce(call, "scatter");
    if (!facts.sorted) {
        // positions are places in the sorted order: map them back to source positions (dim_len stays dim_len)
        at::Tensor back = at::cat({facts.perm, at::full({1}, dim_len, facts.perm.options())});
        arg.copy_(back.index_select(0, arg.view({-1})).view(arg.sizes()));
    }
    return true;
}

}  // namespace

std::tuple<at::Tensor, at::Tensor> scatter_forward(at::Tensor src, at::Tensor index, int64_t dim, at::Tensor out,
                                                   int64_t reduce, bool has_out, int64_t /*hot_target*/)
{
    TORCH_CHECK(src.defined() && src.device().is_cuda(), "scatter: src must be a CUDA tensor");
    TORCH_CHECK(index.defined() && index.device() == src.device(), "scatter: index must be on src's device");
    TORCH_CHECK(out.defined() && out.device() == src.device(), "scatter: out must be on src's device");
    TORCH_CHECK(index.scalar_type() == at::kLong, "scatter: index must be int64");
    TORCH_CHECK(out.scalar_type() == src.scalar_type(), "scatter: out dtype must match src");
    TORCH_CHECK(src.dim() >= 1 && src.dim() <= 8, "scatter: src must have between 1 and 8 dimensions");
    TORCH_CHECK(dim >= 0 && dim < src.dim(), "scatter: dim out of range");
    TORCH_CHECK(reduce >= OPSGNN_SCATTER_SUM && reduce <= OPSGNN_SCATTER_MAX, "scatter: invalid reduce code");
    TORCH_CHECK(src.is_contiguous() && index.is_contiguous() && out.is_contiguous(),
                "scatter: src, index and out must be contiguous");
    TORCH_CHECK(out.dim() == src.dim(), "scatter: out and src must have the same rank");
    for (int64_t d = 0; d < src.dim(); ++d) {
        TORCH_CHECK(d == dim || out.size(d) == src.size(d), "scatter: out shape must match src outside the scatter dim");
    }
    if (has_out) {
        NoteCallerOutput(out);
    }
    const int64_t before = Product(src.sizes(), 0, dim);
    const int64_t dim_len = src.size(dim);
    const int64_t after = Product(src.sizes(), dim + 1, src.dim());
    const bool compact = index.dim() == 1 && index.numel() == dim_len;
    const bool full = !compact && index.numel() == src.numel();
    TORCH_CHECK(compact || full, "scatter: index must hold src.size(dim) or src.numel() entries");
    c10::cuda::CUDAGuard guard(src.device());
    const bool extremum = reduce == OPSGNN_SCATTER_MIN || reduce == OPSGNN_SCATTER_MAX;
    at::Tensor arg = extremum ? at::empty(out.sizes(), out.options().dtype(at::kLong))
                              : at::empty({0}, out.options().dtype(at::kLong));
    if (out.numel() == 0) {
        return {out, arg};
    }
    if (extremum && !has_out && compact && before == 1 &&
        SortedExtremum(src, index, out, arg, dim_len, after, reduce == OPSGNN_SCATTER_MIN)) {
        return {out, arg};
    }
    OpsgnnScatterDesc desc{};
    desc.before = before;
    desc.dim_len = dim_len;
    desc.after = after;
    desc.out_len = out.size(dim);
    desc.index_full = full ? 1 : 0;
    desc.reduce = static_cast<int32_t>(reduce);
    desc.dtype = DtypeId(src.scalar_type(), "scatter");
    desc.has_out = has_out ? 1 : 0;
    int64_t bytes = 0;
    CheckStatus(opsgnn_scatter_workspace_bytes(&desc, &bytes), "scatter");
    at::Tensor scratch = Scratch(bytes, out);
    CheckStatus(opsgnn_scatter(&desc, src.const_data_ptr(), index.data_ptr<int64_t>(), out.data_ptr(),
                               extremum ? arg.data_ptr<int64_t>() : nullptr, scratch.data_ptr(), scratch.numel(),
                               CurrentStream(out)),
                "scatter");
    return {out, arg};
}

// scatter min / max over a 1-D index along dimension 0 with no caller-provided output, outputs allocated HERE: the
// Python front-end calls it right after reading the index facts, with no tensor operation in between, so the cached
// permutation of an unsorted index is reused from call to call.  Returns nothing when the sorted path does not apply
// (the front-end then takes scatter_forward).  Not part of the reference binding.
std::optional<std::tuple<at::Tensor, at::Tensor>> scatter_extremum_sorted(const at::Tensor& src, const at::Tensor& index,
                                                                         int64_t length, bool is_min)
{
    TORCH_CHECK(src.defined() && src.device().is_cuda() && index.defined() && index.device() == src.device(),
                "scatter: src and index must be CUDA tensors on one GPU");
    if (index.scalar_type() != at::kLong || index.dim() != 1 || src.dim() < 1 || index.numel() != src.size(0) ||
        !src.is_contiguous() || !index.is_contiguous() || length <= 0) {
        return std::nullopt;
    }
    c10::cuda::CUDAGuard guard(src.device());
    auto shape = src.sizes().vec();
    shape[0] = length;
    at::Tensor out = at::empty(shape, src.options());
    at::Tensor arg = at::empty(shape, src.options().dtype(at::kLong));
    const int64_t after = Product(src.sizes(), 1, src.dim());
    if (!SortedExtremum(src, index, out, arg, src.size(0), after, is_min)) {
        return std::nullopt;
    }
    return std::make_tuple(out, arg);
}

}  // namespace opsgnn

namespace py = pybind11;

void BindScatter(py::module_& m)
{
    m.def("scatter_extremum_sorted", opsgnn::Scoped(&opsgnn::scatter_extremum_sorted), py::arg("src"), py::arg("index"),
          py::arg("length"), py::arg("is_min"),
          "scatter min / max along dim 0 through a cached stable argsort of the index (no atomics); None when it does not apply",
          py::call_guard<py::gil_scoped_release>());
    m.def("scatter_forward", opsgnn::Scoped(&opsgnn::scatter_forward), py::arg("src"), py::arg("index"), py::arg("dim"), py::arg("out"),
          py::arg("reduce"), py::arg("has_out"), py::arg("hot_target") = -1,
          "torch_scatter-compatible forward reduction (CUDA)", py::call_guard<py::gil_scoped_release>());
}
