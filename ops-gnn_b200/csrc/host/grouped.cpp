// Launch planners of the grouped softmax family: scatter_softmax / scatter_log_softmax / scatter_logsumexp, forward
// and backward (csrc/npu/scatter_softmax/common/grouped_softmax_shared.h:178-248 and
// csrc/npu/scatter_logsumexp/common/grouped_logsumexp_shared.h:50-133 of the reference).  src is viewed as
// [batch, dim_len, after] around `dim`; the index is 1-D over dim_len (int32 as the reference binding passes it, or
// int64).  Sortedness of the index is read from one fused statistics pass, cached per tensor version; a sorted index
// takes the single-sweep path of the kernels.
#include <pybind11/pybind11.h>

#include <list>
#include <mutex>

#include "ops.h"

namespace opsgnn {
namespace {

struct SortedEntry {
    const c10::TensorImpl* impl;
    const void* data;
    int64_t version, numel;
    std::optional<c10::weak_intrusive_ptr<c10::TensorImpl>> alive;
    bool sorted;
};
std::mutex g_sorted_mutex;
std::list<SortedEntry> g_sorted;

// True when the index is non-decreasing.  One kernel and an 8-byte read on a miss; nothing on a hit.
bool IndexIsSorted(const at::Tensor& index)
{
    const bool cacheable = !index.is_inference();
    const c10::TensorImpl* impl = index.unsafeGetTensorImpl();
    const int64_t version = cacheable ? static_cast<int64_t>(index._version()) : -1;
    if (cacheable) {
        std::lock_guard<std::mutex> lock(g_sorted_mutex);
        for (auto it = g_sorted.begin(); it != g_sorted.end(); ++it) {
            if (it->impl == impl && it->data == index.const_data_ptr() && it->version == version &&
                it->numel == index.numel() && it->alive && !it->alive->expired()) {
                return it->sorted;
            }
        }
    }
    auto stats = at::empty({3}, index.options().dtype(at::kLong));
    CheckStatus(opsgnn_index_stats(index.const_data_ptr(), DtypeId(index.scalar_type(), "grouped"), index.numel(),
                                   stats.data_ptr<int64_t>(), CurrentStream(index)),
                "grouped");
    const bool sorted = stats[2].item<int64_t>() == 1;
    if (cacheable) {
        std::lock_guard<std::mutex> lock(g_sorted_mutex);
        g_sorted.push_front(SortedEntry{impl, index.const_data_ptr(), version, index.numel(),
                                        c10::weak_intrusive_ptr<c10::TensorImpl>(index.getIntrusivePtr()), sorted});
        if (g_sorted.size() > 32) {
            g_sorted.pop_back();
        }
    }
    return sorted;
}

struct View {
    int64_t batch, dim_len, after;
};

View CheckCommon(const at::Tensor& src, const at::Tensor& index, int64_t dim, int64_t dim_size, const char* api)
{
    TORCH_CHECK(src.defined() && src.device().is_cuda(), api, ": src must be a CUDA tensor");
    TORCH_CHECK(index.defined() && index.device() == src.device(), api, ": index must be on src's device");
    TORCH_CHECK(src.scalar_type() == at::kFloat || src.scalar_type() == at::kHalf || src.scalar_type() == at::kBFloat16,
                api, ": src must be float16, float32 or bfloat16");
    TORCH_CHECK(index.scalar_type() == at::kInt || index.scalar_type() == at::kLong, api, ": index must be int32 or int64");
    TORCH_CHECK(src.dim() >= 1 && dim >= 0 && dim < src.dim(), api, ": dim out of range");
    TORCH_CHECK(index.dim() == 1 && index.numel() == src.size(dim), api, ": index must be 1-D with src.size(dim) entries");
    TORCH_CHECK(dim_size >= 0, api, ": dim_size must be non-negative");
    TORCH_CHECK(src.is_contiguous() && index.is_contiguous(), api, ": src and index must be contiguous");
    return {Product(src.sizes(), 0, dim), src.size(dim), Product(src.sizes(), dim + 1, src.dim())};
}

OpsgnnGroupedDesc MakeDesc(const View& v, const at::Tensor& src, const at::Tensor& index, int64_t groups, int mode,
                           bool sorted)
{
    OpsgnnGroupedDesc d{};
    d.batch = v.batch;
    d.dim_len = v.dim_len;
    d.after = v.after;
    d.groups = groups;
    d.mode = mode;
    d.dtype = DtypeId(src.scalar_type(), "grouped");
    d.sorted = sorted ? 1 : 0;
    d.index_type = DtypeId(index.scalar_type(), "grouped");
    return d;
}

at::Tensor Forward(const at::Tensor& src, const at::Tensor& index, int64_t dim, int64_t dim_size, int mode,
                   const char* api)
{
    const View v = CheckCommon(src, index, dim, dim_size, api);
    c10::cuda::CUDAGuard guard(src.device());
    auto sizes = src.sizes().vec();
    if (mode == OPSGNN_GROUPED_LOGSUMEXP) {
        sizes[dim] = dim_size;
    }
    at::Tensor out = at::empty(sizes, src.options());
    if (out.numel() == 0) {
        return out;
    }
    const bool sorted = index.numel() > 0 && IndexIsSorted(index);
    OpsgnnGroupedDesc desc = MakeDesc(v, src, index, dim_size, mode, sorted);
    int64_t bytes = 0;
    CheckStatus(opsgnn_grouped_workspace_bytes(&desc, &bytes), api);
    at::Tensor scratch = Scratch(bytes, out);
    CheckStatus(opsgnn_grouped_forward(&desc, src.const_data_ptr(), index.const_data_ptr(), out.data_ptr(),
                                       scratch.data_ptr(), scratch.numel(), CurrentStream(out)),
                api);
    return out;
}

at::Tensor Backward(const at::Tensor* src, const at::Tensor& out, const at::Tensor& grad_out, const at::Tensor& index,
                    int64_t dim, int64_t dim_size, int mode, const char* api)
{
    const at::Tensor& shaped = src != nullptr ? *src : out;  // tensor with the source's shape
    const View v = CheckCommon(shaped, index, dim, dim_size, api);
    TORCH_CHECK(out.defined() && grad_out.defined() && out.device() == shaped.device() &&
                    grad_out.device() == shaped.device(),
                api, ": out and grad_out must be on the source's device");
    TORCH_CHECK(out.scalar_type() == shaped.scalar_type() && grad_out.scalar_type() == shaped.scalar_type(), api,
                ": out and grad_out must have the source's dtype");
    TORCH_CHECK(out.sizes() == grad_out.sizes(), api, ": grad_out must have the forward output's shape");
    TORCH_CHECK(out.is_contiguous() && grad_out.is_contiguous(), api, ": out and grad_out must be contiguous");
    if (mode == OPSGNN_GROUPED_LOGSUMEXP) {
        auto expected = shaped.sizes().vec();
        expected[dim] = dim_size;
        TORCH_CHECK(out.sizes().vec() == expected, api, ": out must have one row per group");
    } else {
        TORCH_CHECK(out.sizes() == shaped.sizes(), api, ": out must have the source's shape");
    }
    c10::cuda::CUDAGuard guard(shaped.device());
    at::Tensor grad_src = at::empty(shaped.sizes(), shaped.options());
    if (grad_src.numel() == 0) {
        return grad_src;
    }
    OpsgnnGroupedDesc desc = MakeDesc(v, shaped, index, dim_size, mode, false);
    int64_t bytes = 0;
    CheckStatus(opsgnn_grouped_workspace_bytes(&desc, &bytes), api);
    at::Tensor scratch = Scratch(bytes, grad_src);
    CheckStatus(opsgnn_grouped_backward(&desc, src != nullptr ? src->const_data_ptr() : nullptr, out.const_data_ptr(),
                                        grad_out.const_data_ptr(), index.const_data_ptr(), grad_src.data_ptr(),
                                        scratch.data_ptr(), scratch.numel(), CurrentStream(grad_src)),
                api);
    return grad_src;
}

}  // namespace

at::Tensor scatter_softmax_forward(const at::Tensor& src, const at::Tensor& index, int64_t dim, int64_t dim_size)
{
    return Forward(src, index, dim, dim_size, OPSGNN_GROUPED_SOFTMAX, "scatter_softmax");
}
at::Tensor scatter_softmax_backward(const at::Tensor& out, const at::Tensor& grad_out, const at::Tensor& index,
                                    int64_t dim, int64_t dim_size)
{
    return Backward(nullptr, out, grad_out, index, dim, dim_size, OPSGNN_GROUPED_SOFTMAX, "scatter_softmax");
}
at::Tensor scatter_log_softmax_forward(const at::Tensor& src, const at::Tensor& index, int64_t dim, int64_t dim_size)
{
    return Forward(src, index, dim, dim_size, OPSGNN_GROUPED_LOG_SOFTMAX, "scatter_log_softmax");
}
at::Tensor scatter_log_softmax_backward(const at::Tensor& out, const at::Tensor& grad_out, const at::Tensor& index,
                                        int64_t dim, int64_t dim_size)
{
    return Backward(nullptr, out, grad_out, index, dim, dim_size, OPSGNN_GROUPED_LOG_SOFTMAX, "scatter_log_softmax");
}
at::Tensor scatter_logsumexp_forward(const at::Tensor& src, const at::Tensor& index, int64_t dim, int64_t dim_size)
{
    return Forward(src, index, dim, dim_size, OPSGNN_GROUPED_LOGSUMEXP, "scatter_logsumexp");
}
at::Tensor scatter_logsumexp_backward(const at::Tensor& src, const at::Tensor& out, const at::Tensor& grad_out,
                                      const at::Tensor& index, int64_t dim, int64_t dim_size)
{
    TORCH_CHECK(src.defined() && src.is_contiguous(), "scatter_logsumexp: src must be contiguous");
    return Backward(&src, out, grad_out, index, dim, dim_size, OPSGNN_GROUPED_LOGSUMEXP, "scatter_logsumexp");
}

}  // namespace opsgnn

namespace py = pybind11;

void BindGrouped(py::module_& m)
{
    using namespace opsgnn;
    m.def("scatter_softmax_forward", &scatter_softmax_forward, py::arg("src"), py::arg("index"), py::arg("dim"),
          py::arg("dim_size"), "Grouped softmax forward on CUDA", py::call_guard<py::gil_scoped_release>());
    m.def("scatter_softmax_backward", &scatter_softmax_backward, py::arg("out"), py::arg("grad_out"), py::arg("index"),
          py::arg("dim"), py::arg("dim_size"), "Grouped softmax backward on CUDA",
          py::call_guard<py::gil_scoped_release>());
    m.def("scatter_log_softmax_forward", &scatter_log_softmax_forward, py::arg("src"), py::arg("index"), py::arg("dim"),
          py::arg("dim_size"), "Grouped log-softmax forward on CUDA", py::call_guard<py::gil_scoped_release>());
    m.def("scatter_log_softmax_backward", &scatter_log_softmax_backward, py::arg("out"), py::arg("grad_out"),
          py::arg("index"), py::arg("dim"), py::arg("dim_size"), "Grouped log-softmax backward on CUDA",
          py::call_guard<py::gil_scoped_release>());
    m.def("scatter_logsumexp_forward", &scatter_logsumexp_forward, py::arg("src"), py::arg("index"), py::arg("dim"),
          py::arg("dim_size"), "Grouped log-sum-exp forward on CUDA", py::call_guard<py::gil_scoped_release>());
    m.def("scatter_logsumexp_backward", &scatter_logsumexp_backward, py::arg("src"), py::arg("out"), py::arg("grad_out"),
          py::arg("index"), py::arg("dim"), py::arg("dim_size"), "Grouped log-sum-exp backward on CUDA",
          py::call_guard<py::gil_scoped_release>());
}
