// Launch planner of scatter_forward (csrc/npu/scatter/op_host/scatter.cpp:242-267 of the reference).
// src is viewed as [before, dim_len, after]; the index is either one entry per position along `dim` or has src's
// full shape; `out` is pre-filled by the Python front-end (zeros, ones, dtype extremes, or the caller's tensor) and is
// reduced into in place.  float64 and int64, which the reference sends to a synchronous CPU fallback, run natively.
#include <pybind11/pybind11.h>

#include "ops.h"

namespace opsgnn {

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

}  // namespace opsgnn

namespace py = pybind11;

void BindScatter(py::module_& m)
{
    m.def("scatter_forward", opsgnn::Scoped(&opsgnn::scatter_forward), py::arg("src"), py::arg("index"), py::arg("dim"), py::arg("out"),
          py::arg("reduce"), py::arg("has_out"), py::arg("hot_target") = -1,
          "torch_scatter-compatible forward reduction (CUDA)", py::call_guard<py::gil_scoped_release>());
}
