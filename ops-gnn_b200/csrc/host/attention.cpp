// Launch planner of the fused graph-attention aggregation (no counterpart in the reference, which composes the layer
// from sddmm_csr, leaky_relu, scatter_softmax and spmm: python/ops_gnn/spmm.py:148-208, 283-289).  Two native calls on the
// current stream: the edge logits and their per-row log-sum-exp, then the aggregation whose weights exp(logit - lse) are
// formed in the gather ring.  Returns (out, lse); lse is what a backward pass needs to rebuild the weights.
#include <pybind11/pybind11.h>

#include "ops.h"

namespace opsgnn {

std::tuple<at::Tensor, at::Tensor> GatAggregate(const at::Tensor& indptr, const at::Tensor& indices, const at::Tensor& edge_rows,
                                                const at::Tensor& x, const at::Tensor& left, const at::Tensor& right,
                                                double negative_slope)
{
    const char* api = "gat_aggregate";
    for (const auto& tensor : {indptr, indices, edge_rows, x, left, right}) {
        TORCH_CHECK(tensor.defined() && tensor.device().is_cuda(), api, ": inputs must be CUDA tensors");
        TORCH_CHECK(tensor.device() == x.device(), api, ": inputs must be on the same GPU");
    }
    TORCH_CHECK(x.dim() == 3 && left.dim() == 2 && right.dim() == 2, api, ": x must be [N, H, D], left [M, H] and right [N, H]");
    TORCH_CHECK(x.scalar_type() == at::kFloat && left.scalar_type() == at::kFloat && right.scalar_type() == at::kFloat, api,
                ": features and logit halves must be float32");
    TORCH_CHECK(indptr.dim() == 1 && indices.dim() == 1 && edge_rows.dim() == 1 && indptr.numel() >= 1 &&
                    (indptr.scalar_type() == at::kInt || indptr.scalar_type() == at::kLong) &&
                    indices.scalar_type() == indptr.scalar_type() && edge_rows.scalar_type() == indptr.scalar_type(),
                api, ": indptr, indices and edge_rows must be one-dimensional with one int32/int64 dtype");
    const int64_t rows = indptr.numel() - 1, sources = x.size(0), heads = x.size(1), width = x.size(2), edges = indices.numel();
    TORCH_CHECK(edge_rows.numel() == edges, api, ": edge_rows must hold one row id per edge");
    TORCH_CHECK(left.size(0) == rows && left.size(1) == heads && right.size(0) == sources && right.size(1) == heads, api,
                ": left must be [rows, H] and right [sources, H]");
    TORCH_CHECK(heads >= 1 && width >= 1, api, ": x must have at least one head and one feature");
    c10::cuda::CUDAGuard guard(x.device());
    auto ptr = indptr.contiguous();
    auto col = indices.contiguous();
    auto erow = edge_rows.contiguous();
    auto xc = x.contiguous();
    auto lc = left.contiguous();
    auto rc = right.contiguous();
    const int facts = CsrFacts(ptr, col, rows, sources, edges);
    TORCH_CHECK(!(facts & 1), api, ": indptr must start at zero and end at nnz");
    TORCH_CHECK(!(facts & 2), api, ": indptr values out of range");
    TORCH_CHECK(!(facts & 4), api, ": indptr must be non-decreasing");
    TORCH_CHECK(!(facts & 8), api, ": indices out of range");
    OpsgnnAttentionDesc desc{};
    desc.rows = rows;
    desc.src_rows = sources;
    desc.heads = heads;
    desc.width = width;
    desc.nnz = edges;
    desc.negative_slope = static_cast<float>(negative_slope);
    desc.index_type = DtypeId(ptr.scalar_type(), api);
    desc.dtype = OPSGNN_F32;
    auto lse = at::empty({rows, heads}, x.options());
    auto out = at::empty({rows, heads, width}, x.options());
    if (rows == 0) {
        return {out, lse};
    }
    RaiseIfDeviceStalled(out, api);
    int64_t bytes = 0;
    CheckStatus(opsgnn_attention_lse_workspace_bytes(&desc, &bytes), api);
    auto lse_scratch = Scratch(bytes, out);
    auto logits = at::empty({edges, heads}, x.options());  // written once, read once; never the softmax weights
    CheckStatus(opsgnn_attention_lse(&desc, erow.const_data_ptr(), col.const_data_ptr(), lc.const_data_ptr<float>(),
                                     rc.const_data_ptr<float>(), logits.data_ptr<float>(), lse.data_ptr<float>(),
                                     lse_scratch.data_ptr(), lse_scratch.numel(), CurrentStream(out)),
                api);
    OpsgnnCsrReduceDesc reduce{};
    reduce.rows = rows;
    reduce.src_rows = sources;
    reduce.feat = heads * width;
    reduce.nnz = edges;
    reduce.batches = 1;
    reduce.value_width = heads;
    reduce.reduce = OPSGNN_REDUCE_SUM;
    reduce.ptr_type = desc.index_type;
    reduce.col_type = desc.index_type;
    reduce.in_type = OPSGNN_F32;
    reduce.out_type = OPSGNN_F32;
    CheckStatus(opsgnn_csr_reduce_workspace_bytes(&reduce, &bytes), api);
    auto scratch = Scratch(bytes, out);
    at::Tensor plan = CsrPlan(ptr, rows, edges);
    const int status = opsgnn_attention_aggregate(&desc, ptr.const_data_ptr(), col.const_data_ptr(), logits.const_data_ptr<float>(),
                                                  lse.const_data_ptr<float>(), xc.const_data_ptr(), out.data_ptr(),
                                                  plan.const_data_ptr(), scratch.data_ptr(), scratch.numel(), CurrentStream(out));
    TORCH_CHECK(status != OPSGNN_ERR_UNSUPPORTED, api,
                ": unsupported shape for the fused kernel (needs heads * width a multiple of 256, heads a multiple of 4 and at "
                "most 21, width a multiple of 4); compose the layer from sddmm_csr, scatter_softmax and bspmm instead");
    CheckStatus(status, api);
    return {out, lse};
}

}  // namespace opsgnn

namespace py = pybind11;

void BindAttention(py::module_& m)
{
    m.def("gat_aggregate", opsgnn::Scoped(&opsgnn::GatAggregate), py::arg("indptr"), py::arg("indices"), py::arg("edge_rows"),
          py::arg("x"), py::arg("left"), py::arg("right"), py::arg("negative_slope") = 0.2,
          "Fused GAT aggregation: softmax over each row's edges of leaky_relu(left[row] + right[col]) per head, applied to "
          "x[col]; returns (out [M, H, D], lse [M, H]); not part of the reference binding",
          py::call_guard<py::gil_scoped_release>());
}
