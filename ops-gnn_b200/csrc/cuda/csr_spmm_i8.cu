// SpMM instances of the CSR reduce engine for int8 values (int32 accumulation, int32 or fp32 output).
#include "csr_instances.h"

namespace opsgnn {
namespace csr {

template <class O, class IndexT> static int RunI8(const Params& p, int kind, cudaStream_t stream)
{
    if (kind == kSum) {
        return Launch<int8_t, O, IndexT, IndexT, 1, 4, kSum>(p, stream);
    }
    if (kind == kExtremum) {
        return Launch<int8_t, O, IndexT, IndexT, 1, 4, kExtremum>(p, stream);
    }
    return OPSGNN_ERR_UNSUPPORTED;
}

int RunSpmmI8(const Params& p, bool index64, int kind, bool out_f32, cudaStream_t stream)
{
    if (out_f32) {
        return index64 ? RunI8<float, int64_t>(p, kind, stream) : RunI8<float, int32_t>(p, kind, stream);
    }
    return index64 ? RunI8<int32_t, int64_t>(p, kind, stream) : RunI8<int32_t, int32_t>(p, kind, stream);
}

}  // namespace csr
}  // namespace opsgnn
