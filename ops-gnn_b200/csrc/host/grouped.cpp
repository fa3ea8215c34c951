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
    TensorKey index;
    LabelFacts facts;
    // Sorted labels: their segment pointers and the CSR plan over them, built on the first sorted forward call for
    // `prepared_groups` groups and reused by later calls on the same stream (the tensors belong to that stream).
    int64_t prepared_groups = -1;
    void* prepared_stream = nullptr;
    at::Tensor ptr, plan;
};
std::mutex g_sorted_mutex;
std::list<SortedEntry> g_sorted;

// Miss: one statistics kernel and one run-length kernel, read back together (32 bytes, one synchronisation); an unsorted
// vector that should be sorted costs an argsort and a second run-length pass.  Hit: nothing.  The facts are reused under
// the rules of TensorKey (identity, version, layout and the write clock): a stale "sorted" would send an unsorted index
// down the sorted path.
}  // namespace

LabelFacts LabelFactsOf(const at::Tensor& index, bool want_permutation)
{
    auto key = TensorKey::Of(index);
    if (key) {
        std::lock_guard<std::mutex> lock(g_sorted_mutex);
        for (auto it = g_sorted.begin(); it != g_sorted.end(); ++it) {
            if (it->index.Matches(*key) && (it->facts.measured || !want_permutation)) {
                return it->facts;
            }
        }
    }
    LabelFacts facts;
    const int type = DtypeId(index.scalar_type(), "grouped");
    auto stats = at::empty({4}, index.options().dtype(at::kLong));
    CheckStatus(opsgnn_index_stats(index.const_data_ptr(), type, index.numel(), stats.data_ptr<int64_t>(), CurrentStream(index)),
                "grouped");
    CheckStatus(opsgnn_index_longest_run(index.const_data_ptr(), type, nullptr, index.numel(), stats.data_ptr<int64_t>() + 3,
                                         CurrentStream(index)),
                "grouped");
    auto host = stats.cpu();
    const int64_t* values = host.const_data_ptr<int64_t>();
    facts.low = values[0];
    facts.high = values[1];
    facts.sorted = values[2] == 1;
    if (facts.sorted) {
        facts.longest = values[3];
        facts.measured = true;
    } else if (want_permutation) {
        at::Tensor perm = at::argsort(index, /*stable=*/true, /*dim=*/0, /*descending=*/false);
        auto longest = at::empty({1}, index.options().dtype(at::kLong));
        CheckStatus(opsgnn_index_longest_run(index.const_data_ptr(), type, perm.const_data_ptr<int64_t>(), index.numel(),
                                             longest.data_ptr<int64_t>(), CurrentStream(index)),
                    "grouped");
        facts.longest = longest.item<int64_t>();
        facts.perm = perm;
        facts.measured = true;
    } else {
        facts.longest = index.numel();  // unknown: treat as long
    }
    if (key) {
        std::lock_guard<std::mutex> lock(g_sorted_mutex);
        g_sorted.remove_if([&](const SortedEntry& entry) { return entry.index.impl == key->impl; });
        g_sorted.push_front(SortedEntry{*key, facts});
        if (g_sorted.size() > 32) {
            g_sorted.pop_back();
        }
    }
    return facts;
}

namespace {

// Segment pointers + plan of a sorted label vector from the facts cache, building them on a miss.  False when the
// labels cannot be keyed (the caller then lets the kernel library scan them inside the call).
bool PreparedSegments(const at::Tensor& index, const OpsgnnGroupedDesc& desc, at::Tensor* ptr, at::Tensor* plan)
{
    auto key = TensorKey::Of(index);
    if (!key) {
        return false;
    }
    void* stream = CurrentStream(index);
    {
        std::lock_guard<std::mutex> lock(g_sorted_mutex);
        for (auto& entry : g_sorted) {
            if (entry.index.Matches(*key)) {
                if (entry.prepared_groups == desc.groups && entry.prepared_stream == stream && entry.ptr.defined()) {
                    *ptr = entry.ptr;
                    *plan = entry.plan;
                    return true;
                }
                break;
            }
        }
    }
    int64_t plan_bytes = 0;
    CheckStatus(opsgnn_csr_plan_bytes(desc.groups, desc.dim_len, &plan_bytes), "grouped");
    at::Tensor made_ptr = at::empty({desc.groups + 1}, index.options().dtype(at::kLong));
    at::Tensor made_plan = Scratch(plan_bytes, index);
    CheckStatus(opsgnn_grouped_prepare(&desc, index.const_data_ptr(), made_ptr.data_ptr<int64_t>(), made_plan.data_ptr(), stream),
                "grouped");
    std::lock_guard<std::mutex> lock(g_sorted_mutex);
    for (auto& entry : g_sorted) {
        if (entry.index.Matches(*key)) {
            entry.prepared_groups = desc.groups;
            entry.prepared_stream = stream;
            entry.ptr = made_ptr;
            entry.plan = made_plan;
            break;
        }
    }
    *ptr = made_ptr;
    *plan = made_plan;
    return true;
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
    // The single-read kernel takes one batch of rows made of whole 16-byte vectors; softmax and log-softmax only.
    const int64_t vec = 16 / static_cast<int64_t>(src.element_size());
    const bool short_shape = mode != OPSGNN_GROUPED_LOGSUMEXP && v.batch == 1 && v.after % vec == 0 &&
                             reinterpret_cast<uintptr_t>(src.const_data_ptr()) % 16 == 0 &&
                             reinterpret_cast<uintptr_t>(out.data_ptr()) % 16 == 0;
    LabelFacts facts;
    if (index.numel() > 0) {
        facts = LabelFactsOf(index, short_shape);
    }
    const bool short_groups = short_shape && facts.longest <= OPSGNN_GROUPED_SHORT_GROUP;
    OpsgnnGroupedDesc desc = MakeDesc(v, src, index, dim_size, mode, facts.sorted);
    // Sorted labels keep the two-sweep form (engine log-sum-exp + apply): its bulk-copy ring holds more bytes in flight
    // than one team of lanes per group can, and measured faster on 1,048,576 x 128 rows in groups of 8 (0.42 against
    // 0.61 ms per call).  The single-read kernel is the unsorted case's: 0.64 against 1.88 ms for the atomic phases.
    if (short_groups && !facts.sorted && facts.perm.defined()) {
        desc.sorted = OPSGNN_GROUPED_SORTED_SHORT;
    }
    int64_t bytes = 0;
    CheckStatus(opsgnn_grouped_workspace_bytes(&desc, &bytes), api);
    at::Tensor scratch = Scratch(bytes, out);
    if (short_groups && !facts.sorted && facts.perm.defined()) {
        CheckStatus(opsgnn_grouped_forward_permuted(&desc, src.const_data_ptr(), index.const_data_ptr(),
                                                    facts.perm.const_data_ptr<int64_t>(), out.data_ptr(), scratch.data_ptr(),
                                                    scratch.numel(), CurrentStream(out)),
                    api);
        return out;
    }
    // Sorted labels through the engine (every shape but the eight-column sweep): pointers and plan come from the cache.
    const bool sweep = v.batch == 1 && v.after == 8 && src.scalar_type() == at::kFloat;
    at::Tensor ptr, plan;
    if (facts.sorted && !sweep && index.numel() > 0 && PreparedSegments(index, desc, &ptr, &plan)) {
        CheckStatus(opsgnn_grouped_forward_prepared(&desc, src.const_data_ptr(), index.const_data_ptr(),
                                                    ptr.const_data_ptr<int64_t>(), plan.const_data_ptr(), out.data_ptr(),
                                                    scratch.data_ptr(), scratch.numel(), CurrentStream(out)),
                    api);
        return out;
    }
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

// (minimum, maximum, sorted, longest group) of a label vector for the Python front-ends: the same cached facts the
// forward planner reads a moment later, so validating the range costs no second pass.
std::tuple<int64_t, int64_t, bool, int64_t> index_facts(const at::Tensor& index, bool want_permutation)
{
    TORCH_CHECK(index.defined() && index.device().is_cuda() && index.dim() == 1 && index.is_contiguous() &&
                    (index.scalar_type() == at::kInt || index.scalar_type() == at::kLong),
                "index_facts: index must be a contiguous 1-D int32/int64 CUDA tensor");
    c10::cuda::CUDAGuard guard(index.device());
    if (index.numel() == 0) {
        return {0, -1, true, 0};
    }
    const LabelFacts facts = LabelFactsOf(index, want_permutation);
    return {facts.low, facts.high, facts.sorted, facts.longest};
}

void ClearSortedIndexCache()
{
    std::lock_guard<std::mutex> lock(g_sorted_mutex);
    g_sorted.clear();
}

int64_t SortedIndexCacheSize()
{
    std::lock_guard<std::mutex> lock(g_sorted_mutex);
    return static_cast<int64_t>(g_sorted.size());
}

}  // namespace opsgnn

namespace py = pybind11;

void BindGrouped(py::module_& m)
{
    using namespace opsgnn;
    m.def("index_facts", Scoped(&index_facts), py::arg("index"), py::arg("want_permutation") = true,
          "(minimum, maximum, sorted, rows of the largest group) of a contiguous label vector; cached per tensor like the "
          "other facts, and shared with the grouped-softmax planners",
          py::call_guard<py::gil_scoped_release>());
    m.def("scatter_softmax_forward", opsgnn::Scoped(&scatter_softmax_forward), py::arg("src"), py::arg("index"), py::arg("dim"),
          py::arg("dim_size"), "Grouped softmax forward on CUDA", py::call_guard<py::gil_scoped_release>());
    m.def("scatter_softmax_backward", opsgnn::Scoped(&scatter_softmax_backward), py::arg("out"), py::arg("grad_out"), py::arg("index"),
          py::arg("dim"), py::arg("dim_size"), "Grouped softmax backward on CUDA",
          py::call_guard<py::gil_scoped_release>());
    m.def("scatter_log_softmax_forward", opsgnn::Scoped(&scatter_log_softmax_forward), py::arg("src"), py::arg("index"), py::arg("dim"),
          py::arg("dim_size"), "Grouped log-softmax forward on CUDA", py::call_guard<py::gil_scoped_release>());
    m.def("scatter_log_softmax_backward", opsgnn::Scoped(&scatter_log_softmax_backward), py::arg("out"), py::arg("grad_out"),
          py::arg("index"), py::arg("dim"), py::arg("dim_size"), "Grouped log-softmax backward on CUDA",
          py::call_guard<py::gil_scoped_release>());
    m.def("scatter_logsumexp_forward", opsgnn::Scoped(&scatter_logsumexp_forward), py::arg("src"), py::arg("index"), py::arg("dim"),
          py::arg("dim_size"), "Grouped log-sum-exp forward on CUDA", py::call_guard<py::gil_scoped_release>());
    m.def("scatter_logsumexp_backward", opsgnn::Scoped(&scatter_logsumexp_backward), py::arg("src"), py::arg("out"), py::arg("grad_out"),
          py::arg("index"), py::arg("dim"), py::arg("dim_size"), "Grouped log-sum-exp backward on CUDA",
          py::call_guard<py::gil_scoped_release>());
}
