// Launch planners of the index conversions: ind2ptr (csrc/npu/ind2ptr/op_host/ind2ptr.cpp:20-42 of the reference),
// ptr2ind (csrc/npu/ptr2ind/op_host/ptr2ind.cpp:20-58) and the one-pass index statistics that replace the separate
// min / max / sortedness reductions of the Python front-ends.
#include "ops.h"

namespace opsgnn {

at::Tensor ind2ptr(at::Tensor ind, int64_t M)
{
    TORCH_CHECK(ind.dim() == 1, "ind2ptr: ind must be 1-D");
    TORCH_CHECK(ind.scalar_type() == at::kLong, "ind2ptr: ind must be int64 (torch.long)");
    TORCH_CHECK(M >= 0, "ind2ptr: M must be non-negative");
    CheckCuda(ind, "ind2ptr", "ind");
    c10::cuda::CUDAGuard guard(ind.device());
    auto out = at::empty({M + 1}, ind.options());
    if (ind.numel() == 0) {
        return out.zero_();
    }
    ind = ind.contiguous();
    CheckStatus(opsgnn_ind2ptr(ind.data_ptr<int64_t>(), ind.numel(), out.data_ptr<int64_t>(), M, CurrentStream(ind)),
                "ind2ptr");
    return out;
}

at::Tensor ptr2ind(at::Tensor ptr, int64_t E)
{
    TORCH_CHECK(ptr.dim() == 1, "ptr2ind: ptr must be 1-D");
    TORCH_CHECK(ptr.scalar_type() == at::kLong, "ptr2ind: ptr must be int64 (torch.long)");
    TORCH_CHECK(E >= 0, "ptr2ind: E must be non-negative");
    TORCH_CHECK(ptr.numel() >= 1, "ptr2ind: ptr must have at least one element");
    CheckCuda(ptr, "ptr2ind", "ptr");
    c10::cuda::CUDAGuard guard(ptr.device());
    ptr = ptr.contiguous();
    // The reference copies the whole pointer array to the host to validate it; here one kernel checks it on the device
    // and four bytes come back (cached per tensor version).
    const int facts = CsrFacts(ptr, std::nullopt, ptr.numel() - 1, 0, E);
    if (facts != 0) {
        // Reproduce the reference's order of complaints with a host check of the end points only.
        const int64_t first = ptr[0].item<int64_t>();
        const int64_t last = ptr[ptr.numel() - 1].item<int64_t>();
        TORCH_CHECK(first == 0, "ptr2ind: ptr must start with 0");
        TORCH_CHECK(last == E, "ptr2ind: ptr must end with num_edges");
        TORCH_CHECK(!(facts & 2), "ptr2ind: ptr contains an out-of-range value");
        TORCH_CHECK(!(facts & 4), "ptr2ind: ptr must be non-decreasing");
    }
    auto out = at::empty({E}, ptr.options());
    if (E == 0) {
        return out;
    }
    CheckStatus(opsgnn_ptr2ind(ptr.data_ptr<int64_t>(), ptr.numel() - 1, out.data_ptr<int64_t>(), E, CurrentStream(ptr)),
                "ptr2ind");
    return out;
}

at::Tensor index_stats(at::Tensor index)
{
    CheckCuda(index, "index_stats", "index");
    TORCH_CHECK(index.scalar_type() == at::kLong || index.scalar_type() == at::kInt,
                "index_stats: index must be int32 or int64");
    c10::cuda::CUDAGuard guard(index.device());
    index = index.contiguous();
    auto stats = at::empty({3}, index.options().dtype(at::kLong));
    CheckStatus(opsgnn_index_stats(index.const_data_ptr(), DtypeId(index.scalar_type(), "index_stats"), index.numel(),
                                   stats.data_ptr<int64_t>(), CurrentStream(index)),
                "index_stats");
    return stats;
}

}  // namespace opsgnn

namespace opsgnn {

// Bit mask of opsgnn_csr_validate for int32/int64 pointers (and columns when given); cached per tensor version.
int64_t csr_facts(at::Tensor ptr, std::optional<at::Tensor> col, int64_t rows, int64_t cols, int64_t nnz)
{
    CheckCuda(ptr, "csr_facts", "ptr");
    TORCH_CHECK(ptr.dim() == 1 && ptr.numel() == rows + 1 && rows >= 0 && nnz >= 0, "csr_facts: bad pointer shape");
    c10::cuda::CUDAGuard guard(ptr.device());
    ptr = ptr.contiguous();
    if (col) {
        CheckCuda(*col, "csr_facts", "col");
        TORCH_CHECK(col->scalar_type() == ptr.scalar_type() && col->numel() == nnz, "csr_facts: bad column tensor");
        col = col->contiguous();
    }
    return CsrFacts(ptr, col, rows, cols, nnz);
}

}  // namespace opsgnn
