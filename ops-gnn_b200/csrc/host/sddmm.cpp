// Launch planner of sddmm_csr (csrc/npu/sddmm_csr/op_host/sddmm_csr.cpp:415-461 of the reference): same operand
// rules and messages; the int32 / uint32 offset limits and the unified-buffer capacity checks of the Ascend kernel do
// not apply because every offset here is 64-bit.  The CSR structure is validated on the device (cached per tensor
// version) instead of with one blocking reduction per call.
#include <pybind11/pybind11.h>

#include "ops.h"

namespace opsgnn {
namespace {

struct OpInfo {
    int code;
    bool use_lhs, use_rhs;
};

OpInfo ResolveOp(const std::string& op)
{
    if (op == "dot") return {OPSGNN_SDDMM_DOT, true, true};
    if (op == "add") return {OPSGNN_SDDMM_ADD, true, true};
    if (op == "sub") return {OPSGNN_SDDMM_SUB, true, true};
    if (op == "mul") return {OPSGNN_SDDMM_MUL, true, true};
    if (op == "div") return {OPSGNN_SDDMM_DIV, true, true};
    if (op == "copy_lhs") return {OPSGNN_SDDMM_COPY_LHS, true, false};
    if (op == "copy_rhs") return {OPSGNN_SDDMM_COPY_RHS, false, true};
    TORCH_CHECK(false, "sddmm_csr: op must be dot, add, sub, mul, div, copy_lhs or copy_rhs");
    return {OPSGNN_SDDMM_DOT, true, true};
}

void CheckTarget(int64_t target, const char* name)
{
    TORCH_CHECK(target >= 0 && target <= 2, "sddmm_csr: ", name, " must be 0 (src), 1 (edge) or 2 (dst)");
}

void CheckRows(const at::Tensor& feature, int64_t target, int64_t m, int64_t nnz, const char* name)
{
    if (target == OPSGNN_TARGET_ROW) {
        TORCH_CHECK(feature.size(0) >= m, "sddmm_csr: ", name, " has fewer rows than the CSR row count");
    } else if (target == OPSGNN_TARGET_EDGE) {
        TORCH_CHECK(feature.size(0) >= nnz, "sddmm_csr: ", name, " has fewer rows than the number of edges");
    }
}

}  // namespace

at::Tensor SddmmCsrForward(const at::Tensor& indptr, const at::Tensor& indices, const std::optional<at::Tensor>& lhs,
                           const std::optional<at::Tensor>& rhs, const std::string& op, int64_t lhs_target,
                           int64_t rhs_target, const std::optional<at::Tensor>& out)
{
    TORCH_CHECK(indptr.defined() && indices.defined(), "sddmm_csr: indptr and indices must be defined");
    TORCH_CHECK(indptr.device().is_cuda() && indices.device().is_cuda(),
                "sddmm_csr: indptr and indices must be CUDA tensors");
    const OpInfo info = ResolveOp(op);
    CheckTarget(lhs_target, "lhs_target");
    CheckTarget(rhs_target, "rhs_target");
    const auto device = indptr.device();
    TORCH_CHECK(indices.device() == device, "sddmm_csr: indices must be on the same GPU");
    const at::Tensor* lhs_ptr = nullptr;
    const at::Tensor* rhs_ptr = nullptr;
    if (info.use_lhs) {
        TORCH_CHECK(lhs.has_value(), "sddmm_csr: lhs is required for op ", op);
        TORCH_CHECK(lhs->defined(), "sddmm_csr: lhs must be defined");
        TORCH_CHECK(lhs->device() == device, "sddmm_csr: lhs must be on the same GPU");
        lhs_ptr = &*lhs;
    } else {
        TORCH_CHECK(!lhs.has_value(), "sddmm_csr: lhs is not used by op ", op);
    }
    if (info.use_rhs) {
        TORCH_CHECK(rhs.has_value(), "sddmm_csr: rhs is required for op ", op);
        TORCH_CHECK(rhs->defined(), "sddmm_csr: rhs must be defined");
        TORCH_CHECK(rhs->device() == device, "sddmm_csr: rhs must be on the same GPU");
        rhs_ptr = &*rhs;
    } else {
        TORCH_CHECK(!rhs.has_value(), "sddmm_csr: rhs is not used by op ", op);
    }
    const at::Tensor* primary = lhs_ptr ? lhs_ptr : rhs_ptr;
    TORCH_CHECK(primary != nullptr, "sddmm_csr: at least one feature tensor is required");
    const at::ScalarType dtype = primary->scalar_type();
    TORCH_CHECK(dtype == at::kHalf || dtype == at::kFloat || dtype == at::kBFloat16,
                "sddmm_csr: features must be float16 or float32");
    int64_t feat = 0;
    for (const at::Tensor* feature : {lhs_ptr, rhs_ptr}) {
        if (feature == nullptr) {
            continue;
        }
        TORCH_CHECK(feature->dim() == 2 && feature->size(1) > 0,
                    "sddmm_csr: features must be two-dimensional with a positive feature dim");
        TORCH_CHECK(feature->scalar_type() == dtype, "sddmm_csr: lhs and rhs must have the same dtype");
        TORCH_CHECK(!feature->requires_grad(), "sddmm_csr: autograd is not supported");
        if (feat == 0) {
            feat = feature->size(1);
        } else {
            TORCH_CHECK(feat == feature->size(1), "sddmm_csr: lhs and rhs must have the same feature dim");
        }
    }
    TORCH_CHECK(indptr.dim() == 1 && indices.dim() == 1 && indptr.numel() >= 1,
                "sddmm_csr: indptr and indices must be one-dimensional; indptr must be nonempty");
    TORCH_CHECK((indptr.scalar_type() == at::kInt || indptr.scalar_type() == at::kLong) &&
                    indices.scalar_type() == indptr.scalar_type(),
                "sddmm_csr: indptr and indices must have the same int32/int64 dtype");
    c10::cuda::CUDAGuard guard(device);
    const int64_t m = indptr.numel() - 1;
    const int64_t nnz = indices.numel();
    auto ptr = indptr.contiguous();
    auto idx = indices.contiguous();
    // Column range matters only for operands gathered by the column.
    int64_t dst_rows = -1;
    if (lhs_ptr && lhs_target == OPSGNN_TARGET_COL) {
        dst_rows = lhs_ptr->size(0);
    }
    if (rhs_ptr && rhs_target == OPSGNN_TARGET_COL) {
        dst_rows = dst_rows < 0 ? rhs_ptr->size(0) : std::min(dst_rows, rhs_ptr->size(0));
    }
    const int facts = CsrFacts(ptr, dst_rows >= 0 ? std::optional<at::Tensor>(idx) : std::nullopt, m,
                               dst_rows >= 0 ? dst_rows : 0, nnz);
    TORCH_CHECK(!(facts & 8), "sddmm_csr: CSR indices are out of range for dst features");
    TORCH_CHECK(!(facts & 7), "sddmm_csr: invalid CSR (indptr/indices)");
    if (lhs_ptr) {
        CheckRows(*lhs_ptr, lhs_target, m, nnz, "lhs");
    }
    if (rhs_ptr) {
        CheckRows(*rhs_ptr, rhs_target, m, nnz, "rhs");
    }
    std::vector<int64_t> shape = info.code == OPSGNN_SDDMM_DOT ? std::vector<int64_t>{nnz} : std::vector<int64_t>{nnz, feat};
    at::Tensor result;
    if (out.has_value()) {
        const at::Tensor& candidate = *out;
        TORCH_CHECK(candidate.defined(), "sddmm_csr: out must be defined");
        TORCH_CHECK(candidate.device() == device && candidate.scalar_type() == dtype,
                    "sddmm_csr: out must match the feature device and dtype");
        TORCH_CHECK(candidate.dim() == static_cast<int64_t>(shape.size()), "sddmm_csr: out has the wrong rank");
        for (size_t i = 0; i < shape.size(); ++i) {
            TORCH_CHECK(candidate.size(static_cast<int64_t>(i)) == shape[i], "sddmm_csr: out has the wrong shape");
        }
        TORCH_CHECK(candidate.is_contiguous(), "sddmm_csr: out must be contiguous");
        TORCH_CHECK(!candidate.requires_grad(), "sddmm_csr: out must not require gradients");
        TORCH_CHECK(!candidate.is_alias_of(indptr) && !candidate.is_alias_of(indices),
                    "sddmm_csr: out must not alias any input storage");
        for (const at::Tensor* feature : {lhs_ptr, rhs_ptr}) {
            if (feature != nullptr) {
                TORCH_CHECK(!candidate.is_alias_of(*feature), "sddmm_csr: out must not alias any input storage");
            }
        }
        result = candidate;
    } else {
        result = at::empty(shape, primary->options());
    }
    if (nnz == 0) {
        return result;
    }
    at::Tensor lhs_c = lhs_ptr ? lhs_ptr->contiguous() : at::Tensor();
    at::Tensor rhs_c = rhs_ptr ? rhs_ptr->contiguous() : at::Tensor();
    OpsgnnSddmmDesc desc{};
    desc.rows = m;
    desc.nnz = nnz;
    desc.feat = feat;
    desc.lhs_rows = lhs_ptr ? lhs_c.size(0) : 0;
    desc.rhs_rows = rhs_ptr ? rhs_c.size(0) : 0;
    desc.op = info.code;
    desc.lhs_target = static_cast<int32_t>(lhs_target);
    desc.rhs_target = static_cast<int32_t>(rhs_target);
    desc.index_type = DtypeId(ptr.scalar_type(), "sddmm_csr");
    desc.dtype = DtypeId(dtype, "sddmm_csr");
    int64_t bytes = 0;
    CheckStatus(opsgnn_sddmm_workspace_bytes(&desc, &bytes), "sddmm_csr");
    at::Tensor scratch = Scratch(bytes, result);
    CheckStatus(opsgnn_sddmm_csr(&desc, ptr.const_data_ptr(), idx.const_data_ptr(),
                                 lhs_ptr ? lhs_c.const_data_ptr() : nullptr, rhs_ptr ? rhs_c.const_data_ptr() : nullptr,
                                 result.data_ptr(), scratch.data_ptr(), scratch.numel(), CurrentStream(result)),
                "sddmm_csr");
    return result;
}

}  // namespace opsgnn

namespace py = pybind11;

void BindSddmm(py::module_& m)
{
    m.def("sddmm_csr", opsgnn::Scoped(&opsgnn::SddmmCsrForward), py::arg("indptr"), py::arg("indices"), py::arg("lhs"), py::arg("rhs"),
          py::arg("op") = "dot", py::arg("lhs_target") = 0, py::arg("rhs_target") = 2, py::arg("out") = py::none(),
          "CSR SDDMM on CUDA", py::call_guard<py::gil_scoped_release>());
}
