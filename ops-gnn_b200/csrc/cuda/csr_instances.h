// Entry points of the translation units that instantiate the CSR reduce engine (one unit per value dtype so the
// build parallelises).
#pragma once

#include "csr_reduce.cuh"

namespace opsgnn {
namespace csr {

// Indexed gather (SpMM): ptr and col share one index width.
int RunSpmmF32(const Params& p, bool index64, int kind, cudaStream_t stream);
int RunSpmmF16(const Params& p, bool index64, int kind, bool out_f32, cudaStream_t stream);
int RunSpmmBF16(const Params& p, bool index64, int kind, bool out_f32, cudaStream_t stream);
int RunSpmmI8(const Params& p, bool index64, int kind, bool out_f32, cudaStream_t stream);
// Identity gather (segment reductions over consecutive rows).
int RunSegmentFloat(const Params& p, int dtype, bool ptr64, int kind, bool out_f32, cudaStream_t stream);
int RunSegmentOther(const Params& p, int dtype, bool ptr64, int kind, cudaStream_t stream);


// Weighted bulk instance in attention mode (csr_abi.cu): the weight of an edge is formed from per-node halves and the
// row's log-sum-exp instead of being read from memory.
int RunAttention(const OpsgnnCsrReduceDesc& desc, const void* ptr, const void* col, const float* logits, const float* lse,
                 const void* x, void* out, const void* plan, void* workspace, int64_t workspace_bytes, void* stream);

}  // namespace csr
}  // namespace opsgnn
