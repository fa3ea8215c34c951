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

}  // namespace csr
}  // namespace opsgnn
