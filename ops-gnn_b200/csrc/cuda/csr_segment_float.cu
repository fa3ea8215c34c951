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

// fp32 log-sum-exp of a 16-bit source: the grouped softmax keeps its per-group statistics in fp32.
template <class T, class PtrT> static int RunWideLse(const Params& p, cudaStream_t stream)
{
    return LaunchShaped<T, float, PtrT, Identity, kLogSumExp>(p, stream);
}

int RunSegmentFloat(const Params& p, int dtype, bool ptr64, int kind, bool out_f32, cudaStream_t stream)
{
    if (out_f32 && dtype != OPSGNN_F32) {
        if (kind != kLogSumExp) {
            return OPSGNN_ERR_UNSUPPORTED;
        }
        if (dtype == OPSGNN_F16) {
            return ptr64 ? RunWideLse<__half, int64_t>(p, stream) : RunWideLse<__half, int32_t>(p, stream);
        }
        if (dtype == OPSGNN_BF16) {
            return ptr64 ? RunWideLse<__nv_bfloat16, int64_t>(p, stream) : RunWideLse<__nv_bfloat16, int32_t>(p, stream);
        }
        return OPSGNN_ERR_UNSUPPORTED;
    }
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
