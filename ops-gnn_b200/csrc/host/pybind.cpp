// Python binding of the launch planners.  Function names, argument names and defaults are those of the reference's
// csrc/pybind.cpp:92-257 (both of its architecture branches, since one GPU build offers every operator); the module
// attribute `npu_arch` is kept for callers that read it and names this build "sm_100a".
#include <ATen/core/dispatch/Dispatcher.h>
#include <c10/core/DispatchKey.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "ops.h"

namespace py = pybind11;

namespace {

bool HasKernelForKey(const std::string& op_name, c10::DispatchKey key)
{
    const auto op = c10::Dispatcher::singleton().findOp(c10::OperatorName(op_name, ""));
    return op.has_value() && op->hasKernelForDispatchKey(key);
}

void BindSpmm(py::module_& m)
{
    using namespace opsgnn;
    m.def("spmm_max_csr", opsgnn::Scoped(&SpmmMaxCsr), py::arg("indptr"), py::arg("indices"), py::arg("x"), py::arg("out") = py::none(),
          "CSR SpMM max on CUDA", py::call_guard<py::gil_scoped_release>());
    m.def("spmm_min_csr", opsgnn::Scoped(&SpmmMinCsr), py::arg("indptr"), py::arg("indices"), py::arg("x"), py::arg("out") = py::none(),
          "CSR SpMM min on CUDA", py::call_guard<py::gil_scoped_release>());
    m.def("spmm_sum_csr", opsgnn::Scoped(&SpmmSumCsr), py::arg("indptr"), py::arg("indices"), py::arg("x"), py::arg("out") = py::none(),
          "CSR SpMM sum on CUDA", py::call_guard<py::gil_scoped_release>());
    m.def("unified_spmm_csr", opsgnn::Scoped(&UnifiedSpmmCsr), py::arg("indptr"), py::arg("indices"), py::arg("x"),
          py::arg("op") = "copy_lhs", py::arg("reduce") = "sum", py::arg("out") = py::none(),
          "Unified two-dimensional CSR SpMM on CUDA", py::call_guard<py::gil_scoped_release>());
    m.def("spmm_weighted_csr", opsgnn::Scoped(&SpmmWeightedCsr), py::arg("indptr"), py::arg("indices"), py::arg("x"), py::arg("weight"),
          py::arg("reduce") = "sum",
          "CSR SpMM with one edge weight per feature group (fused `mul` message); not part of the reference binding",
          py::call_guard<py::gil_scoped_release>());
    m.def("gather_rows", opsgnn::Scoped(&GatherRows), py::arg("x"), py::arg("index"), py::arg("unit_ptr"), py::arg("out"),
          "out[i] = x[index[i]] through the CSR engine (unit_ptr = 0..n); not part of the reference binding",
          py::call_guard<py::gil_scoped_release>());
    m.def("copy_rows_async", opsgnn::Scoped(&CopyRowsAsync), py::arg("src"), py::arg("dst"),
          "dst <- src with one cudaMemcpyAsync on the current stream (copy engine; dst may be a peer's symmetric-memory block)");
    m.def("gather_rows_into", opsgnn::Scoped(&GatherRowsInto), py::arg("x"), py::arg("index"), py::arg("outs"), py::arg("max_ctas") = 0,
          "outs[s][i] = x[index[start_s + i]] with a capped grid; the outputs may be views of a peer's mapped buffer; not "
          "part of the reference binding",
          py::call_guard<py::gil_scoped_release>());
    m.def("csr_spmm_into", opsgnn::Scoped(&CsrSpmmInto), py::arg("ptr"), py::arg("col"), py::arg("value"), py::arg("x"), py::arg("out"),
          "out[r] = sum_e value[e] * x[col[e]] into a caller-provided contiguous [rows, K] view; not part of the reference "
          "binding",
          py::call_guard<py::gil_scoped_release>());
    auto sub = m.def_submodule("torch_sparse_spmm", "torch_sparse SpMM on CUDA");
    sub.def("forward", opsgnn::Scoped(&TorchSparseSpmmForward), py::arg("ptr"), py::arg("col"), py::arg("value"), py::arg("mat"),
            py::arg("reduce"), py::arg("outtype"), py::call_guard<py::gil_scoped_release>());
    sub.def("validate", opsgnn::Scoped(&TorchSparseSpmmValidate), py::arg("ptr"), py::arg("col"), py::arg("n"),
            py::call_guard<py::gil_scoped_release>());
    sub.def("value_backward", opsgnn::Scoped(&TorchSparseSpmmValueGrad), py::arg("ptr"), py::arg("col"), py::arg("mat"), py::arg("grad"),
            py::arg("reduce"), py::arg("width"), py::call_guard<py::gil_scoped_release>());
    sub.def("convert", opsgnn::Scoped(&TorchSparseSpmmConvert), py::arg("src"), py::arg("output"), py::arg("to_ptr"),
            py::call_guard<py::gil_scoped_release>());
    sub.def("permute_values", opsgnn::Scoped(&TorchSparseSpmmPermuteValues), py::arg("value"), py::arg("perm"),
            py::call_guard<py::gil_scoped_release>());
    sub.def("tensor_version", opsgnn::Scoped(&TorchSparseSpmmTensorVersion), py::arg("tensor"));
}

void BindSegment(py::module_& m)
{
    using namespace opsgnn;
    m.def("segment_csr", opsgnn::Scoped(&segment_csr), py::arg("src"), py::arg("indptr"), py::arg("out") = py::none(),
          py::arg("reduce") = "sum", py::arg("return_arg") = true, py::call_guard<py::gil_scoped_release>());
    m.def(
        "segment_csr_value",
        [](at::Tensor src, at::Tensor indptr, std::optional<at::Tensor> out, const std::string& reduce) {
            PlannerScope scope;
            return segment_csr(std::move(src), std::move(indptr), std::move(out), reduce, false)[0];
        },
        py::arg("src"), py::arg("indptr"), py::arg("out") = py::none(), py::arg("reduce") = "sum",
        py::call_guard<py::gil_scoped_release>());
    m.attr("SEGMENT_COO_SUM") = static_cast<int32_t>(SEGMENT_COO_SUM);
    m.attr("SEGMENT_COO_MEAN") = static_cast<int32_t>(SEGMENT_COO_MEAN);
    m.attr("SEGMENT_COO_MIN") = static_cast<int32_t>(SEGMENT_COO_MIN);
    m.attr("SEGMENT_COO_MAX") = static_cast<int32_t>(SEGMENT_COO_MAX);
    m.def("segment_coo_forward", opsgnn::Scoped(&segment_coo_forward), py::arg("src"), py::arg("index"), py::arg("out"),
          py::arg("dim_size"), py::arg("reduce"), py::arg("return_arg") = true,
          py::call_guard<py::gil_scoped_release>());
    m.def(
        "segment_coo_value",
        [](at::Tensor src, at::Tensor index, std::optional<at::Tensor> out, std::optional<int64_t> dim_size,
           int64_t reduce) {
            PlannerScope scope;
            return std::get<0>(segment_coo_forward(std::move(src), std::move(index), std::move(out), dim_size, reduce,
                                                   false));
        },
        py::arg("src"), py::arg("index"), py::arg("out"), py::arg("dim_size"), py::arg("reduce"),
        py::call_guard<py::gil_scoped_release>());
    m.def("segment_logsumexp_forward", opsgnn::Scoped(&segment_logsumexp_forward), py::arg("src"), py::arg("indptr"),
          "CSR log-sum-exp forward on CUDA", py::call_guard<py::gil_scoped_release>());
}

void BindConvert(py::module_& m)
{
    using namespace opsgnn;
    m.def("ind2ptr", opsgnn::Scoped(&ind2ptr), py::arg("ind"), py::arg("M"),
          "Convert sorted row indices to CSR row pointer, same as torch_sparse.ind2ptr",
          py::call_guard<py::gil_scoped_release>());
    m.def("ptr2ind", opsgnn::Scoped(&ptr2ind), py::arg("ptr"), py::arg("E"),
          "Convert CSR row pointer to row indices, same as torch_sparse.ptr2ind",
          py::call_guard<py::gil_scoped_release>());
    m.def("csr_facts", opsgnn::Scoped(&csr_facts), py::arg("ptr"), py::arg("col"), py::arg("rows"), py::arg("cols"), py::arg("nnz"),
          "Validation bit mask of a CSR structure: 1 end points, 2 pointer range, 4 decreasing pointer, 8 column range",
          py::call_guard<py::gil_scoped_release>());
    m.def("index_stats", opsgnn::Scoped(&index_stats), py::arg("index"),
          "int64[3] on the device: minimum, maximum and 1 when the index is non-decreasing",
          py::call_guard<py::gil_scoped_release>());
}

}  // namespace

void BindSddmm(py::module_& m);
void BindScatter(py::module_& m);
void BindGrouped(py::module_& m);
void BindGather(py::module_& m);
void BindAttention(py::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
    m.doc() = "ops_gnn: CUDA (sm_100a) extension";
    m.attr("npu_arch") = "sm_100a";
    m.def(
        "has_private_use1_kernel",
        [](const std::string& op_name) { return HasKernelForKey(op_name, c10::DispatchKey::CUDA); },
        py::arg("op_name"),
        "True if the operator already has a kernel for this build's device key (CUDA), e.g. a pre-existing "
        "third-party registration");
    opsgnn::StartWriteObserver();
    m.def("clear_native_caches", []() {
        opsgnn::ClearCsrPlanCache();
        opsgnn::ClearCsrFactsCache();
        opsgnn::ClearSortedIndexCache();
    });
    m.def("write_clock", []() { return opsgnn::WriteClock(); },
          "Value of the process-wide write clock: it advances whenever an ATen operator runs outside this library's "
          "planners or a planner writes caller memory; cached plans and validation facts are reused only while it stands");
    m.def("native_cache_sizes", []() { return opsgnn::NativeCacheSizes(); },
          "(plans, validation facts, sorted-index facts) currently cached");
    m.def(
        "device_stall_count",
        [](int64_t device, bool synchronize) { return opsgnn::DeviceStallCount(static_cast<int>(device), synchronize); },
        py::arg("device"), py::arg("synchronize") = true,
        "Device-side waits that ran out on this device since the last look (reading clears the count); with "
        "synchronize the device is synchronised first so the count covers every launch enqueued so far",
        py::call_guard<py::gil_scoped_release>());
    m.def(
        "set_wait_polls", [](int64_t polls) { opsgnn::CheckStatus(opsgnn_set_wait_polls(polls), "set_wait_polls"); },
        py::arg("polls"),
        "Poll limit of one device-side bulk-copy wait for later launches; negative restores the default, zero makes "
        "every wait give up at once (the diagnostic that exercises the error path)");
    BindSegment(m);
    BindSpmm(m);
    BindConvert(m);
    BindSddmm(m);
    BindScatter(m);
    BindGrouped(m);
    BindGather(m);
    BindAttention(m);
}
