// Segment-reduction instances of the CSR reduce engine (col(e) = e) for fp32 / fp16 / bf16 sources.
#include "csr_instances.h"

namespace opsgnn {
namespace csr {

template <class T, class PtrT> static int RunFloat(const Params& p, int kind, cudaStream_t stream)
{
    switch (kind) {
        case kSum:
            return LaunchShaped<T, T, PtrT, Identity, kSum>(p, stream);
        case kExtremum:
            return LaunchShaped<T, T, PtrT, Identity, kExtremum>(p, stream);
        case kLogSumExp:
            return LaunchShaped<T, T, PtrT, Identity, kLogSumExp>(p, stream);
        default:
            return OPSGNN_ERR_UNSUPPORTED;
    }
}

int RunSegmentFloat(const Params& p, int dtype, bool ptr64, int kind, cudaStream_t stream)
{
    switch (dtype) {
        case OPSGNN_F32:
            return ptr64 ? RunFloat<float, int64_t>(p, kind, stream) : RunFloat<float, int32_t>(p, kind, stream);
        case OPSGNN_F16:
            return ptr64 ? RunFloat<__half, int64_t>(p, kind, stream) : RunFloat<__half, int32_t>(p, kind, stream);
        case OPSGNN_BF16:
            return ptr64 ? RunFloat<__nv_bfloat16, int64_t>(p, kind, stream)
                         : RunFloat<__nv_bfloat16, int32_t>(p, kind, stream);
        default:
            return OPSGNN_ERR_UNSUPPORTED;
    }
}

}  // namespace csr
}  // namespace opsgnn
