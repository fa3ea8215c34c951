// SpMM instances of the CSR reduce engine for fp16 values (fp32 accumulation, fp16 or fp32 output).
#include "csr_instances.h"

namespace opsgnn {
namespace csr {

template <class O, class IndexT> static int RunF16(const Params& p, int kind, cudaStream_t stream)
{
    if (kind == kSum) {
        return LaunchShaped<__half, O, IndexT, IndexT, kSum>(p, stream);
    }
    if (kind == kExtremum) {
        return LaunchShaped<__half, O, IndexT, IndexT, kExtremum>(p, stream);
    }
    return OPSGNN_ERR_UNSUPPORTED;
}

int RunSpmmF16(const Params& p, bool index64, int kind, bool out_f32, cudaStream_t stream)
{
    if (out_f32) {
        return index64 ? RunF16<float, int64_t>(p, kind, stream) : RunF16<float, int32_t>(p, kind, stream);
    }
    return index64 ? RunF16<__half, int64_t>(p, kind, stream) : RunF16<__half, int32_t>(p, kind, stream);
}

}  // namespace csr
}  // namespace opsgnn
