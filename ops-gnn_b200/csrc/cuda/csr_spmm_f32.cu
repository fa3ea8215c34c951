// SpMM instances of the CSR reduce engine for fp32 values.
#include "csr_instances.h"

namespace opsgnn {
namespace csr {

template <class IndexT> static int RunF32(const Params& p, int kind, cudaStream_t stream)
{
    if (kind == kSum) {
        return LaunchShaped<float, float, IndexT, IndexT, kSum>(p, stream);
    }
    if (kind == kExtremum) {
        return LaunchShaped<float, float, IndexT, IndexT, kExtremum>(p, stream);
    }
    return OPSGNN_ERR_UNSUPPORTED;
}

int RunSpmmF32(const Params& p, bool index64, int kind, cudaStream_t stream)
{
    return index64 ? RunF32<int64_t>(p, kind, stream) : RunF32<int32_t>(p, kind, stream);
}

}  // namespace csr
}  // namespace opsgnn
