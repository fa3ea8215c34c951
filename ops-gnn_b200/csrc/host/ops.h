// Declarations of the launch planners bound by pybind.cpp (same names and argument order as the functions the
// reference binds in csrc/pybind.cpp:92-257).
#pragma once

#include "common.h"

namespace opsgnn {

// torch_sparse SpMM family (spmm.cpp)
std::tuple<at::Tensor, at::Tensor> TorchSparseSpmmForward(at::Tensor ptr, at::Tensor col,
                                                          std::optional<at::Tensor> value, at::Tensor mat,
                                                          int64_t reduce, int64_t outType);
at::Tensor TorchSparseSpmmValidate(at::Tensor ptr, at::Tensor col, int64_t n);
at::Tensor TorchSparseSpmmValueGrad(at::Tensor ptr, at::Tensor col, at::Tensor mat, at::Tensor grad, int64_t reduce,
                                    int64_t width);
at::Tensor TorchSparseSpmmConvert(at::Tensor src, int64_t output, bool toPtr);
at::Tensor TorchSparseSpmmPermuteValues(at::Tensor value, at::Tensor perm);
std::optional<int64_t> TorchSparseSpmmTensorVersion(const at::Tensor& tensor);
at::Tensor SpmmSumCsr(const at::Tensor& indptr, const at::Tensor& indices, const at::Tensor& x,
                      const std::optional<at::Tensor>& out);
at::Tensor SpmmMaxCsr(const at::Tensor& indptr, const at::Tensor& indices, const at::Tensor& x,
                      const std::optional<at::Tensor>& out);
at::Tensor SpmmMinCsr(const at::Tensor& indptr, const at::Tensor& indices, const at::Tensor& x,
                      const std::optional<at::Tensor>& out);
at::Tensor UnifiedSpmmCsr(const at::Tensor& indptr, const at::Tensor& indices, const at::Tensor& x,
                          const std::string& op, const std::string& reduce, const std::optional<at::Tensor>& out);

at::Tensor GatherRows(const at::Tensor& x, const at::Tensor& index, const at::Tensor& unit_ptr, const at::Tensor& out);
void GatherRowsInto(const at::Tensor& x, const at::Tensor& index, const std::vector<at::Tensor>& outs, int64_t max_ctas);
void CopyRowsAsync(const at::Tensor& src, const at::Tensor& dst);
at::Tensor CsrSpmmInto(const at::Tensor& ptr, const at::Tensor& col, const std::optional<at::Tensor>& value,
                       const at::Tensor& x, const at::Tensor& out);
at::Tensor SpmmWeightedCsr(const at::Tensor& indptr, const at::Tensor& indices, const at::Tensor& x,
                           const at::Tensor& weight, const std::string& reduce);

// segment reductions (segment.cpp)
constexpr int64_t SEGMENT_COO_SUM = 0, SEGMENT_COO_MEAN = 1, SEGMENT_COO_MIN = 2, SEGMENT_COO_MAX = 3;
std::vector<at::Tensor> segment_csr(at::Tensor src, at::Tensor indptr, std::optional<at::Tensor> out,
                                    const std::string& reduce, bool return_arg);
std::tuple<at::Tensor, at::Tensor> segment_coo_forward(at::Tensor src, at::Tensor index,
                                                       std::optional<at::Tensor> out, std::optional<int64_t> dim_size,
                                                       int64_t reduce, bool return_arg);
at::Tensor segment_logsumexp_forward(const at::Tensor& src, const at::Tensor& indptr);

// index conversions (convert.cpp)
at::Tensor ind2ptr(at::Tensor ind, int64_t M);
at::Tensor ptr2ind(at::Tensor ptr, int64_t E);
at::Tensor index_stats(at::Tensor index);
int64_t csr_facts(at::Tensor ptr, std::optional<at::Tensor> col, int64_t rows, int64_t cols, int64_t nnz);

// fused graph attention (attention.cpp)
std::tuple<at::Tensor, at::Tensor> GatAggregate(const at::Tensor& indptr, const at::Tensor& indices, const at::Tensor& edge_rows,
                                                const at::Tensor& x, const at::Tensor& left, const at::Tensor& right,
                                                double negative_slope);

// row expansions (gather.cpp)
at::Tensor gather_csr(const at::Tensor& src, const at::Tensor& indptr, const std::optional<at::Tensor>& out);
at::Tensor gather_coo(const at::Tensor& src, const at::Tensor& index, const std::optional<at::Tensor>& out);

// SDDMM (sddmm.cpp)
at::Tensor SddmmCsrForward(const at::Tensor& indptr, const at::Tensor& indices, const std::optional<at::Tensor>& lhs,
                           const std::optional<at::Tensor>& rhs, const std::string& op, int64_t lhs_target,
                           int64_t rhs_target, const std::optional<at::Tensor>& out);

// scatter (scatter.cpp)
std::tuple<at::Tensor, at::Tensor> scatter_forward(at::Tensor src, at::Tensor index, int64_t dim, at::Tensor out,
                                                   int64_t reduce, bool has_out, int64_t hot_target);

std::optional<std::tuple<at::Tensor, at::Tensor>> scatter_extremum_sorted(const at::Tensor& src, const at::Tensor& index,
                                                                         int64_t length, bool is_min);

// grouped softmax family (grouped.cpp)
std::tuple<int64_t, int64_t, bool, int64_t> index_facts(const at::Tensor& index, bool want_permutation);
at::Tensor scatter_softmax_forward(const at::Tensor& src, const at::Tensor& index, int64_t dim, int64_t dim_size);
at::Tensor scatter_softmax_backward(const at::Tensor& out, const at::Tensor& grad_out, const at::Tensor& index,
                                    int64_t dim, int64_t dim_size);
at::Tensor scatter_log_softmax_forward(const at::Tensor& src, const at::Tensor& index, int64_t dim, int64_t dim_size);
at::Tensor scatter_log_softmax_backward(const at::Tensor& out, const at::Tensor& grad_out, const at::Tensor& index,
                                        int64_t dim, int64_t dim_size);
at::Tensor scatter_logsumexp_forward(const at::Tensor& src, const at::Tensor& index, int64_t dim, int64_t dim_size);
at::Tensor scatter_logsumexp_backward(const at::Tensor& src, const at::Tensor& out, const at::Tensor& grad_out,
                                      const at::Tensor& index, int64_t dim, int64_t dim_size);

}  // namespace opsgnn
