// SpMM instances of the CSR reduce engine for bf16 values (fp32 accumulation, bf16 or fp32 output).
#include "csr_instances.h"

namespace opsgnn {
namespace csr {

template <class O, class IndexT> static int RunBF16(const Params& p, int kind, cudaStream_t stream)
{
    if (kind == kSum) {
        return LaunchShaped<__nv_bfloat16, O, IndexT, IndexT, kSum>(p, stream);
    }
    if (kind == kExtremum) {
        return LaunchShaped<__nv_bfloat16, O, IndexT, IndexT, kExtremum>(p, stream);
    }
    return OPSGNN_ERR_UNSUPPORTED;
}

int RunSpmmBF16(const Params& p, bool index64, int kind, bool out_f32, cudaStream_t stream)
{
    if (out_f32) {
        return index64 ? RunBF16<float, int64_t>(p, kind, stream) : RunBF16<float, int32_t>(p, kind, stream);
    }
    return index64 ? RunBF16<__nv_bfloat16, int64_t>(p, kind, stream) : RunBF16<__nv_bfloat16, int32_t>(p, kind, stream);
}

}  // namespace csr
}  // namespace opsgnn
