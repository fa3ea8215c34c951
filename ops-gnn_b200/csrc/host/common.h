// Shared pieces of the C++ launch planners: dtype ids, current-stream lookup, status checks, scratch allocation and
// the per-graph cache of merge-path plans.  The planners validate and allocate with torch, then hand raw pointers to
// the C ABI of libopsgnn_b200.so; no planner computes on the host and none has a CPU path.
#pragma once

#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <optional>
#include <string>
#include <tuple>
#include <vector>

#include "opsgnn_b200.h"

namespace opsgnn {

inline int DtypeId(at::ScalarType t, const char* api)
{
    switch (t) {
        case at::kFloat:
            return OPSGNN_F32;
        case at::kHalf:
            return OPSGNN_F16;
        case at::kBFloat16:
            return OPSGNN_BF16;
        case at::kChar:
            return OPSGNN_I8;
        case at::kInt:
            return OPSGNN_I32;
        case at::kLong:
            return OPSGNN_I64;
        case at::kByte:
            return OPSGNN_U8;
        case at::kShort:
            return OPSGNN_I16;
        case at::kDouble:
            return OPSGNN_F64;
        default:
            TORCH_CHECK(false, api, ": unsupported dtype ", t);
    }
    return -1;
}

inline void CheckCuda(const at::Tensor& t, const char* api, const char* name)
{
    TORCH_CHECK(t.defined() && t.device().is_cuda(), api, ": ", name, " must be a CUDA tensor (there is no CPU path)");
}

inline void* CurrentStream(const at::Tensor& t)
{
    return reinterpret_cast<void*>(c10::cuda::getCurrentCUDAStream(t.device().index()).stream());
}

inline void CheckStatus(int status, const char* api)
{
    TORCH_CHECK(status == OPSGNN_OK, api, ": native launch failed: ", opsgnn_status_string(status), " (status ", status,
                ")");
}

// Byte scratch on the tensor's device; the caching allocator returns 512-byte aligned blocks.
inline at::Tensor Scratch(int64_t bytes, const at::Tensor& like)
{
    return at::empty({bytes > 0 ? bytes : 1}, like.options().dtype(at::kByte));
}

inline int64_t Product(c10::IntArrayRef sizes, int64_t from, int64_t to)
{
    int64_t p = 1;
    for (int64_t i = from; i < to; ++i) {
        p *= sizes[i];
    }
    return p;
}

// Merge-path plan of a pointer array, cached per tensor identity and version (a GNN calls the same graph every layer
// and every step).  Entries hold a weak reference, so a recycled address cannot revive a stale plan.
at::Tensor CsrPlan(const at::Tensor& ptr, int64_t rows, int64_t nnz_bound);
void ClearCsrPlanCache();

struct CsrReduceCall {
    at::Tensor ptr;                 // [rows + 1], int32/int64, contiguous
    std::optional<at::Tensor> col;  // [nnz] same dtype as ptr, or nullopt for consecutive source rows
    std::optional<at::Tensor> val;  // [nnz] or [nnz, feat], dtype of mat
    at::Tensor mat;                 // contiguous, viewed as [batches, src_rows, feat]
    at::Tensor out;                 // contiguous, viewed as [batches, rows, feat]
    std::optional<at::Tensor> arg;  // int64, shape of out (allocated internally when absent for min/max)
    int64_t rows = 0, src_rows = 0, feat = 0, nnz = 0, batches = 1, value_width = 0, arg_none = 0;
    int reduce = OPSGNN_REDUCE_SUM;
    int extremum = OPSGNN_EXTREMUM_IGNORE_NAN;
};

// Builds (or reuses) the plan, allocates carry scratch and launches the engine on the current stream.
void RunCsrReduce(CsrReduceCall& call, const char* api);

// Device-side waits that ran out (a bulk-copy wait of the reduce engine gave up; its launch left rows unwritten).  The
// kernels report into one word of mapped pinned host memory per device, registered with the C ABI on the device's first
// use, so the host can look without synchronising: every planner call looks first and raises for a stall of an EARLIER
// launch (the asynchronous-error convention of CUDA itself).  DeviceStallCount(sync = true) synchronises the device
// first, which makes the report cover everything enqueued so far.  Reading clears the word.
void RaiseIfDeviceStalled(const at::Tensor& on_device, const char* api);
int64_t DeviceStallCount(int device, bool synchronize);

// Validation facts of a CSR structure: bit mask of opsgnn_csr_validate, cached like the plans.  Costs one 4-byte
// device-to-host read on a miss.
int CsrFacts(const at::Tensor& ptr, const std::optional<at::Tensor>& col, int64_t rows, int64_t cols, int64_t nnz);
void ClearCsrFactsCache();

}  // namespace opsgnn
