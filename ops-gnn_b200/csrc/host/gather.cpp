// Launch planners of gather_csr and gather_coo, the row expansions that invert the segment reductions (they are the
// backward data movement of segment_csr / segment_coo sums).  Contracts follow the reference's host code: argument
// checks and messages of csrc/npu/gather_csr/op_host/gather_csr.cpp:95-160 and csrc/npu/gather_coo/op_host/
// gather_coo.cpp:107-183; `out` is returned as the same object when supplied, a non-contiguous or aliasing `out` is
// produced in a temporary and copied back, inputs that `out` aliases are read from a copy.  Unlike the reference,
// which validates the pointers on a host copy, the pointer checks run on the device (one pass, one 4-byte read).
#include <pybind11/pybind11.h>

#include "ops.h"

namespace opsgnn {
namespace {

bool ExpandDtype(at::ScalarType t)
{
    switch (t) {
        case at::kHalf:
        case at::kBFloat16:
        case at::kFloat:
        case at::kDouble:
        case at::kChar:
        case at::kByte:
        case at::kShort:
        case at::kInt:
        case at::kLong:
            return true;
        default:
            return false;
    }
}

void CheckGpu(const at::Tensor& t, const char* api, const char* name)
{
    TORCH_CHECK(t.defined(), api, ": ", name, " must be defined");
    TORCH_CHECK(t.device().is_cuda(), api, ": ", name, " must be a CUDA tensor, got device ", t.device());
}

// Runs the expansion into `out` when it can be written in place, else into a temporary that is copied back.
at::Tensor Expand(const at::Tensor& src, const at::Tensor& index, const std::optional<at::Tensor>& out,
                  const std::vector<int64_t>& shape, int64_t dim, int64_t out_rows, bool csr, const char* api)
{
    const bool has_out = out.has_value();
    at::Tensor source = src.contiguous();
    at::Tensor idx = index;
    bool direct = has_out && out->is_contiguous() && !out->requires_grad() && !out->is_inference();
    if (has_out && out->is_alias_of(src)) {
        direct = false;
    }
    if (has_out && out->is_alias_of(index)) {
        direct = false;
    }
    at::Tensor target = direct ? *out : at::empty(shape, src.options());
    const int64_t batches = Product(src.sizes(), 0, dim);
    const int64_t src_rows = src.size(dim);
    const int64_t row_bytes = Product(src.sizes(), dim + 1, src.dim()) * static_cast<int64_t>(src.element_size());
    if (target.numel() > 0) {
        if (has_out) {
            NoteCallerOutput(*out);
        }
        CheckStatus(opsgnn_gather_expand(source.const_data_ptr(), idx.const_data_ptr<int64_t>(), target.data_ptr(), batches,
                                         src_rows, out_rows, row_bytes, csr ? 1 : 0, CurrentStream(src)),
                    api);
    }
    if (has_out && !direct) {
        out->copy_(target);
    }
    return has_out ? *out : target;
}

}  // namespace

at::Tensor gather_csr(const at::Tensor& src, const at::Tensor& indptr, const std::optional<at::Tensor>& out)
{
    const char* api = "gather_csr";
    CheckGpu(src, api, "src");
    CheckGpu(indptr, api, "indptr");
    TORCH_CHECK(src.device() == indptr.device(), "gather_csr: src and indptr must be on the same GPU");
    TORCH_CHECK(ExpandDtype(src.scalar_type()), "gather_csr: unsupported src dtype ", src.scalar_type());
    TORCH_CHECK(indptr.scalar_type() == at::kLong, "gather_csr: indptr dtype must be int64");
    TORCH_CHECK(src.dim() >= 1 && src.dim() <= 8, "gather_csr: src rank must be in [1, 8], got ", src.dim());
    TORCH_CHECK(indptr.dim() >= 1 && indptr.dim() <= src.dim(), "gather_csr: indptr rank must be in [1, src.dim()], got ",
                indptr.dim());
    const int64_t dim = indptr.dim() - 1;
    if (out) {
        CheckGpu(*out, api, "out");
        TORCH_CHECK(out->device() == src.device(), "gather_csr: out and src must be on the same GPU");
        TORCH_CHECK(out->scalar_type() == src.scalar_type(), "gather_csr: out dtype must match src dtype");
        TORCH_CHECK(out->dim() == src.dim(), "gather_csr: out rank must match src rank");
        for (int64_t axis = 0; axis < src.dim(); ++axis) {
            TORCH_CHECK(axis == dim || out->size(axis) == src.size(axis), "gather_csr: out shape must match src outside dimension ",
                        dim);
        }
    }
    for (int64_t axis = 0; axis < dim; ++axis) {
        TORCH_CHECK(indptr.size(axis) == 1 || indptr.size(axis) == src.size(axis), "gather_csr: indptr dimension ", axis,
                    " with size ", indptr.size(axis), " cannot broadcast to src size ", src.size(axis));
    }
    const int64_t width = indptr.size(-1);
    if (width == 0) {
        TORCH_CHECK(src.size(dim) == 0, "gather_csr: an empty indptr requires src.size(", dim, ") to be 0, got ", src.size(dim));
    } else {
        TORCH_CHECK(src.size(dim) == width - 1, "gather_csr: src.size(", dim, ") must equal indptr.size(-1) - 1; got ",
                    src.size(dim), " and ", width - 1);
    }
    c10::cuda::CUDAGuard guard(src.device());
    auto shape = src.sizes().vec();
    auto expanded = indptr.sizes().vec();
    for (int64_t axis = 0; axis < dim; ++axis) {
        expanded[axis] = src.size(axis);
    }
    at::Tensor ptr = indptr.expand(expanded).contiguous();
    if (out && out->is_alias_of(indptr)) {
        ptr = ptr.clone();
    }
    const int64_t batches = Product(src.sizes(), 0, dim);
    int64_t endpoint = 0;
    if (width > 0 && batches > 0) {
        // One device pass per call: pointers within [0, endpoint], non-decreasing, one common endpoint for all batches.
        auto rows2d = ptr.view({batches, width});
        auto last = rows2d.select(1, width - 1);
        auto ok = ((rows2d >= 0).all() & (rows2d <= last.unsqueeze(1)).all() & (last == last[0]).all());
        if (width > 1) {
            ok = ok & (rows2d.slice(1, 1) >= rows2d.slice(1, 0, width - 1)).all();
        }
        auto facts = at::stack({ok.to(at::kLong), last[0]}).cpu();
        TORCH_CHECK(facts[0].item<int64_t>() == 1,
                    "gather_csr: indptr must be non-negative, non-decreasing, within [0, endpoint] and share one endpoint across "
                    "broadcast rows");
        endpoint = facts[1].item<int64_t>();
    }
    shape[dim] = endpoint;
    if (out) {
        TORCH_CHECK(out->size(dim) == endpoint, "gather_csr: out.size(", dim, ") must equal indptr endpoint ", endpoint, ", got ",
                    out->size(dim));
    }
    if (src.numel() == 0 || endpoint == 0) {
        if (out) {
            out->zero_();
            return *out;
        }
        return at::zeros(shape, src.options());
    }
    return Expand(src, ptr, out, shape, dim, endpoint, true, api);
}

at::Tensor gather_coo(const at::Tensor& src, const at::Tensor& index, const std::optional<at::Tensor>& out)
{
    const char* api = "gather_coo";
    CheckGpu(src, api, "src");
    CheckGpu(index, api, "index");
    TORCH_CHECK(src.device() == index.device(), "gather_coo: src and index must be on the same GPU");
    TORCH_CHECK(ExpandDtype(src.scalar_type()), "gather_coo does not support dtype ", src.scalar_type());
    TORCH_CHECK(index.scalar_type() == at::kLong, "gather_coo: index must have dtype torch.int64");
    TORCH_CHECK(src.dim() >= 1 && src.dim() <= 8, "gather_coo: src rank must be in [1, 8]");
    TORCH_CHECK(index.dim() >= 1 && index.dim() <= src.dim(), "gather_coo: index rank must be in [1, src.dim()]");
    const int64_t dim = index.dim() - 1;
    for (int64_t axis = 0; axis < dim; ++axis) {
        TORCH_CHECK(src.size(axis) == index.size(axis), "gather_coo: src and index prefix shapes must match at dim ", axis);
    }
    auto shape = src.sizes().vec();
    shape[dim] = index.size(dim);
    const int64_t batches = Product(src.sizes(), 0, dim);
    TORCH_CHECK(batches * index.size(dim) == 0 || src.size(dim) > 0,
                "gather_coo: index contains entries but src has zero rows along the gather dimension");
    if (out) {
        CheckGpu(*out, api, "out");
        TORCH_CHECK(out->device() == src.device(), "gather_coo: out must be on the same GPU as src");
        TORCH_CHECK(out->scalar_type() == src.scalar_type(), "gather_coo: out dtype must match src dtype");
        TORCH_CHECK(out->dim() == src.dim(), "gather_coo: out rank mismatch");
        for (int64_t axis = 0; axis < src.dim(); ++axis) {
            TORCH_CHECK(out->size(axis) == shape[axis], "gather_coo: out shape mismatch at dim ", axis);
        }
    }
    c10::cuda::CUDAGuard guard(src.device());
    at::Tensor idx = index.contiguous();
    if (out && out->is_alias_of(index)) {
        idx = idx.clone();
    }
    if (idx.numel() > 0) {
        // bounds on the device: min / max / sortedness in one pass, one 24-byte read
        auto stats = at::empty({3}, idx.options());
        CheckStatus(opsgnn_index_stats(idx.const_data_ptr(), OPSGNN_I64, idx.numel(), stats.data_ptr<int64_t>(), CurrentStream(src)),
                    api);
        auto host = stats.cpu();
        TORCH_CHECK(host[0].item<int64_t>() >= 0 && host[1].item<int64_t>() < src.size(dim),
                    "gather_coo: index values must lie in [0, ", src.size(dim), ")");
    }
    return Expand(src, idx, out, shape, dim, index.size(dim), false, api);
}

}  // namespace opsgnn

namespace py = pybind11;

void BindGather(py::module_& m)
{
    m.def("gather_csr", opsgnn::Scoped(&opsgnn::gather_csr), py::arg("src"), py::arg("indptr"), py::arg("out") = py::none(),
          "Expand segment rows by int64 CSR pointers on CUDA", py::call_guard<py::gil_scoped_release>());
    m.def("gather_coo", opsgnn::Scoped(&opsgnn::gather_coo), py::arg("src"), py::arg("index"), py::arg("out") = py::none(),
          "Gather rows by a sorted int64 COO index on CUDA", py::call_guard<py::gil_scoped_release>());
}
