// Segment-reduction instances of the CSR reduce engine (col(e) = e) for float64 and the integer dtypes.
// Integer sums wrap in the accumulator exactly as two's-complement arithmetic in the value dtype does.
#include "csr_instances.h"

namespace opsgnn {
namespace csr {

template <class T> static int RunOther(const Params& p, bool ptr64, int kind, cudaStream_t stream)
{
    if (kind == kSum) {
        return ptr64 ? Launch<T, T, int64_t, Identity, 1, 4, kSum>(p, stream)
                     : Launch<T, T, int32_t, Identity, 1, 4, kSum>(p, stream);
    }
    if (kind == kExtremum) {
        return ptr64 ? Launch<T, T, int64_t, Identity, 1, 4, kExtremum>(p, stream)
                     : Launch<T, T, int32_t, Identity, 1, 4, kExtremum>(p, stream);
    }
    return OPSGNN_ERR_UNSUPPORTED;
}

int RunSegmentOther(const Params& p, int dtype, bool ptr64, int kind, cudaStream_t stream)
{
    switch (dtype) {
        case OPSGNN_F64:
            return RunOther<double>(p, ptr64, kind, stream);
        case OPSGNN_I8:
            return RunOther<int8_t>(p, ptr64, kind, stream);
        case OPSGNN_U8:
            return RunOther<uint8_t>(p, ptr64, kind, stream);
        case OPSGNN_I16:
            return RunOther<int16_t>(p, ptr64, kind, stream);
        case OPSGNN_I32:
            return RunOther<int32_t>(p, ptr64, kind, stream);
        case OPSGNN_I64:
            return RunOther<int64_t>(p, ptr64, kind, stream);
        default:
            return OPSGNN_ERR_UNSUPPORTED;
    }
}

}  // namespace csr
}  // namespace opsgnn
