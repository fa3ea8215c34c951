// C ABI of the CSR reduce engine: plan construction, scratch sizing and dtype dispatch.
#include <atomic>
#include <cstdio>

#include "csr_instances.h"

namespace opsgnn {
namespace csr {
namespace {

bool IsIndexType(int t) { return t == OPSGNN_I32 || t == OPSGNN_I64; }

int AccBytes(int in_type)
{
    switch (in_type) {
        case OPSGNN_F64:
        case OPSGNN_I64:
            return 8;
        default:
            return 4;
    }
}

int KindOf(int reduce)
{
    switch (reduce) {
        case OPSGNN_REDUCE_SUM:
        case OPSGNN_REDUCE_MEAN:
            return kSum;
        case OPSGNN_REDUCE_MIN:
        case OPSGNN_REDUCE_MAX:
            return kExtremum;
        case OPSGNN_REDUCE_LOGSUMEXP:
            return kLogSumExp;
        default:
            return -1;
    }
}

// Head of every reduce workspace: the launch's status word (stalled waits), padded to the alignment of what follows.
constexpr int64_t kStatusBytes = 256;

// Per device: an optional second place where a stalled wait is reported, and the poll limit of one wait.
constexpr int kMaxDevices = 64;
std::atomic<unsigned long long*> g_status_sink[kMaxDevices];
std::atomic<int64_t> g_wait_polls{-1};

// Upper bound of a carry row: every feature tile is padded to at most 256 features.
int64_t CarryWidth(const OpsgnnCsrReduceDesc& d) { return d.batches * AlignUp(d.feat > 0 ? d.feat : 1, 256); }

int CheckDesc(const OpsgnnCsrReduceDesc* d)
{
    if (d == nullptr || d->rows < 0 || d->src_rows < 0 || d->feat < 0 || d->nnz < 0 || d->batches < 1) {
        return OPSGNN_ERR_INVALID;
    }
    if (KindOf(d->reduce) < 0 || !IsIndexType(d->ptr_type)) {
        return OPSGNN_ERR_INVALID;
    }
    if (d->value_width < 0 || (d->value_width > 1 && (d->feat == 0 || d->feat % d->value_width != 0))) {
        return OPSGNN_ERR_INVALID;
    }
    if (d->nnz > 0 && d->src_rows == 0) {
        return OPSGNN_ERR_INVALID;
    }
    if (d->src_rows > 2147483647LL || d->feat > 2147483647LL) {
        return OPSGNN_ERR_LIMIT;  // staged column ids are 32-bit
    }
    if (d->extremum < OPSGNN_EXTREMUM_IGNORE_NAN || d->extremum > OPSGNN_EXTREMUM_SEEDED_LAST) {
        return OPSGNN_ERR_INVALID;
    }
    return OPSGNN_OK;
}

}  // namespace
}  // namespace csr
}  // namespace opsgnn

using namespace opsgnn;
using namespace opsgnn::csr;

extern "C" int opsgnn_csr_plan_bytes(int64_t rows, int64_t nnz, int64_t* bytes)
{
    if (bytes == nullptr || rows < 0 || nnz < 0) {
        return OPSGNN_ERR_INVALID;
    }
    *bytes = (NumCta(rows, nnz) + 1) * static_cast<int64_t>(sizeof(int64_t));
    return OPSGNN_OK;
}

extern "C" int opsgnn_csr_plan_build(const void* ptr, int ptr_type, int64_t rows, int64_t nnz, void* plan, void* stream)
{
    if (ptr == nullptr || plan == nullptr || rows < 0 || nnz < 0 || !IsIndexType(ptr_type)) {
        return OPSGNN_ERR_INVALID;
    }
    const int64_t num_cta = NumCta(rows, nnz);
    const int threads = 256;
    const unsigned grid = static_cast<unsigned>(CeilDiv(num_cta + 1, threads));
    if (ptr_type == OPSGNN_I64) {
        PlanKernel<int64_t><<<grid, threads, 0, AsStream(stream)>>>(static_cast<const int64_t*>(ptr), rows, nnz, num_cta,
                                                                      static_cast<int64_t*>(plan));
    } else {
        PlanKernel<int32_t><<<grid, threads, 0, AsStream(stream)>>>(static_cast<const int32_t*>(ptr), rows, nnz, num_cta,
                                                                      static_cast<int64_t*>(plan));
    }
    return LaunchStatus();
}

extern "C" int opsgnn_csr_reduce_workspace_bytes(const OpsgnnCsrReduceDesc* desc, int64_t* bytes)
{
    int status = CheckDesc(desc);
    if (status != OPSGNN_OK || bytes == nullptr) {
        return OPSGNN_ERR_INVALID;
    }
    const int64_t num_cta = NumCta(desc->rows, desc->nnz);
    const int64_t width = CarryWidth(*desc);
    int64_t total = kStatusBytes;                                      // status word
    total += AlignUp(num_cta * 8, 256);                                // carry_row
    total += AlignUp(num_cta * width * AccBytes(desc->in_type), 256);  // carry_val
    if (KindOf(desc->reduce) == kExtremum) {
        total += AlignUp(num_cta * width * 8, 256);  // carry_arg
    }
    *bytes = total;
    return OPSGNN_OK;
}

namespace opsgnn {
namespace csr {

// Argument checks and the launch parameters shared by opsgnn_csr_reduce and the attention aggregation.  Returns
// OPSGNN_OK with *launch = false when there is nothing to compute.
int PrepareReduce(const OpsgnnCsrReduceDesc* desc, const void* ptr, const void* col, const void* val, const void* mat,
                  void* out, int64_t* arg, const void* plan, void* workspace, int64_t workspace_bytes, Params* params,
                  bool* launch)
{
    *launch = false;
    int status = CheckDesc(desc);
    if (status != OPSGNN_OK) {
        return status;
    }
    const OpsgnnCsrReduceDesc& d = *desc;
    if (d.rows == 0 || d.feat == 0) {
        return OPSGNN_OK;
    }
    *launch = true;
    const int kind = KindOf(d.reduce);
    if (ptr == nullptr || out == nullptr || plan == nullptr || (d.nnz > 0 && mat == nullptr)) {
        return OPSGNN_ERR_INVALID;
    }
    if (kind == kExtremum && arg == nullptr) {
        return OPSGNN_ERR_INVALID;
    }
    if ((d.value_width != 0) != (val != nullptr)) {
        return OPSGNN_ERR_INVALID;
    }
    if (col != nullptr && (!IsIndexType(d.col_type) || d.col_type != d.ptr_type)) {
        return OPSGNN_ERR_UNSUPPORTED;
    }
    if (col == nullptr && d.nnz > d.src_rows) {
        return OPSGNN_ERR_INVALID;
    }
    int64_t needed = 0;
    opsgnn_csr_reduce_workspace_bytes(desc, &needed);
    if (workspace == nullptr || workspace_bytes < needed || !Aligned(workspace, 256)) {
        return OPSGNN_ERR_WORKSPACE;
    }

    Params& p = *params;
    p = Params{};
    p.ptr = ptr;
    p.col = col;
    p.val = val;
    p.mat = mat;
    p.out = out;
    p.arg = arg;
    p.plan = static_cast<const int64_t*>(plan);
    p.rows = d.rows;
    p.src_rows = d.src_rows;
    p.feat = d.feat;
    p.nnz = d.nnz;
    p.batches = d.batches;
    p.arg_none = d.arg_none;
    p.num_cta = NumCta(d.rows, d.nnz);
    p.mean = d.reduce == OPSGNN_REDUCE_MEAN;
    p.is_min = d.reduce == OPSGNN_REDUCE_MIN;
    p.extremum = d.extremum;
    p.has_val = val != nullptr;
    p.wide = (val == nullptr || d.value_width == 1) ? 0 : (d.value_width == d.feat ? 1 : 2);
    p.val_width = d.value_width;
    p.val_group = d.value_width > 0 ? d.feat / d.value_width : 1;
    char* cursor = static_cast<char*>(workspace);
    const int64_t width = CarryWidth(d);
    p.status = reinterpret_cast<unsigned long long*>(cursor);
    cursor += kStatusBytes;
    int device = 0;
    OPSGNN_CUDA_TRY(cudaGetDevice(&device));
    p.status_sink = (device >= 0 && device < kMaxDevices) ? g_status_sink[device].load(std::memory_order_relaxed) : nullptr;
    const int64_t polls = g_wait_polls.load(std::memory_order_relaxed);
    p.wait_polls = polls < 0 ? kBulkSpinLimit : static_cast<uint32_t>(polls > 0xffffffffLL ? 0xffffffffLL : polls);
    p.carry_row = reinterpret_cast<int64_t*>(cursor);
    cursor += AlignUp(p.num_cta * 8, 256);
    p.carry_val = cursor;
    cursor += AlignUp(p.num_cta * width * AccBytes(d.in_type), 256);
    p.carry_arg = reinterpret_cast<int64_t*>(cursor);

    return OPSGNN_OK;
}

int RunAttention(const OpsgnnCsrReduceDesc& desc, const void* ptr, const void* col, const float* logits, const float* lse,
                 const void* x, void* out, const void* plan, void* workspace, int64_t workspace_bytes, void* stream)
{
    Params p{};
    bool launch = false;
    // the logits take the place of the per-(edge, head) weights; the kernel turns them into exp(logit - lse[row])
    int status = PrepareReduce(&desc, ptr, col, logits, x, out, nullptr, plan, workspace, workspace_bytes, &p, &launch);
    if (status != OPSGNN_OK || !launch) {
        return status;
    }
    p.attention = 1;
    p.att_lse = lse;
    cudaStream_t s = AsStream(stream);
    OPSGNN_CUDA_TRY(cudaMemsetAsync(p.status, 0, sizeof(unsigned long long), s));
    return RunSpmmF32(p, desc.ptr_type == OPSGNN_I64, kSum, s);
}

}  // namespace csr
}  // namespace opsgnn

extern "C" int opsgnn_csr_reduce(const OpsgnnCsrReduceDesc* desc, const void* ptr, const void* col, const void* val,
                                 const void* mat, void* out, int64_t* arg, const void* plan, void* workspace,
                                 int64_t workspace_bytes, void* stream)
{
    Params p{};
    bool launch = false;
    int status = PrepareReduce(desc, ptr, col, val, mat, out, arg, plan, workspace, workspace_bytes, &p, &launch);
    if (status != OPSGNN_OK || !launch) {
        return status;
    }
    const OpsgnnCsrReduceDesc& d = *desc;
    const int kind = KindOf(d.reduce);
    const bool index64 = d.ptr_type == OPSGNN_I64;
    cudaStream_t s = AsStream(stream);
    OPSGNN_CUDA_TRY(cudaMemsetAsync(p.status, 0, sizeof(unsigned long long), s));
#ifdef OPSGNN_CHECKED
    // Diagnostic build only: run the launch synchronously and print the first out-of-range access it skipped.
    static unsigned long long* debug = nullptr;
    if (debug == nullptr) {
        OPSGNN_CUDA_TRY(cudaMalloc(&debug, 4 * sizeof(unsigned long long)));
    }
    OPSGNN_CUDA_TRY(cudaMemsetAsync(debug, 0, 4 * sizeof(unsigned long long), s));
    p.debug = debug;
    struct Report {
        cudaStream_t s;
        unsigned long long* debug;
        const OpsgnnCsrReduceDesc& d;
        ~Report()
        {
            unsigned long long host[4] = {0, 0, 0, 0};
            const cudaError_t sync = cudaStreamSynchronize(s);
            cudaMemcpy(host, debug, sizeof(host), cudaMemcpyDeviceToHost);
            if (host[0] != 0 || sync != cudaSuccess) {
                fprintf(stderr,
                        "[opsgnn checked] sync=%d violations=%llu site=%llu index=%lld limit=%lld rows=%lld src_rows=%lld "
                        "feat=%lld nnz=%lld batches=%lld reduce=%d in=%d out=%d\n",
                        static_cast<int>(sync), host[0], host[1], static_cast<long long>(host[2]),
                        static_cast<long long>(host[3]), static_cast<long long>(d.rows),
                        static_cast<long long>(d.src_rows), static_cast<long long>(d.feat),
                        static_cast<long long>(d.nnz), static_cast<long long>(d.batches), d.reduce, d.in_type,
                        d.out_type);
            }
        }
    } report{s, debug, d};
#endif
    if (col != nullptr) {
        switch (d.in_type) {
            case OPSGNN_F32:
                if (d.out_type != OPSGNN_F32) {
                    return OPSGNN_ERR_UNSUPPORTED;
                }
                return RunSpmmF32(p, index64, kind, s);
            case OPSGNN_F16:
                if (d.out_type != OPSGNN_F16 && d.out_type != OPSGNN_F32) {
                    return OPSGNN_ERR_UNSUPPORTED;
                }
                return RunSpmmF16(p, index64, kind, d.out_type == OPSGNN_F32, s);
            case OPSGNN_BF16:
                if (d.out_type != OPSGNN_BF16 && d.out_type != OPSGNN_F32) {
                    return OPSGNN_ERR_UNSUPPORTED;
                }
                return RunSpmmBF16(p, index64, kind, d.out_type == OPSGNN_F32, s);
            case OPSGNN_I8:
                if (d.out_type != OPSGNN_I32 && d.out_type != OPSGNN_F32) {
                    return OPSGNN_ERR_UNSUPPORTED;
                }
                return RunSpmmI8(p, index64, kind, d.out_type == OPSGNN_F32, s);
            default:
                return OPSGNN_ERR_UNSUPPORTED;
        }
    }
    const bool widened = d.out_type == OPSGNN_F32 && (d.in_type == OPSGNN_F16 || d.in_type == OPSGNN_BF16);
    if (val != nullptr || (d.out_type != d.in_type && !widened)) {
        return OPSGNN_ERR_UNSUPPORTED;
    }
    switch (d.in_type) {
        case OPSGNN_F32:
        case OPSGNN_F16:
        case OPSGNN_BF16:
            return RunSegmentFloat(p, d.in_type, index64, kind, widened, s);
        default:
            return RunSegmentOther(p, d.in_type, index64, kind, s);
    }
}

namespace opsgnn {
namespace csr {
template <class T, class PtrT>
__global__ void IntegerMeanKernel(T* out, const PtrT* ptr, int64_t rows, int64_t feat, int64_t batches)
{
    const int64_t total = batches * rows * feat;
    for (int64_t at = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; at < total;
         at += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t row = (at / feat) % rows;
        // The count is narrowed to the value dtype first (a 256-element uint8 segment has count 0 and mean 0).
        const T count = static_cast<T>(static_cast<int64_t>(ptr[row + 1]) - static_cast<int64_t>(ptr[row]));
        const T value = out[at];
        T mean = T(0);
        if (count != T(0)) {
            if (std::is_signed<T>::value && count == T(-1)) {
                mean = static_cast<T>(T(0) - value);  // avoids the INT_MIN / -1 trap, wraps like two's complement
            } else {
                mean = static_cast<T>(value / count);
            }
        }
        out[at] = mean;
    }
}

template <class T>
int IntegerMean(void* out, const void* ptr, int ptr_type, int64_t rows, int64_t feat, int64_t batches, cudaStream_t s)
{
    const int64_t total = batches * rows * feat;
    if (total == 0) {
        return OPSGNN_OK;
    }
    const int threads = 256;
    int64_t blocks = CeilDiv(total, threads);
    const int64_t cap = static_cast<int64_t>(SmCount()) * 16;
    blocks = blocks < cap ? blocks : cap;
    if (ptr_type == OPSGNN_I64) {
        IntegerMeanKernel<T, int64_t><<<static_cast<unsigned>(blocks), threads, 0, s>>>(
            static_cast<T*>(out), static_cast<const int64_t*>(ptr), rows, feat, batches);
    } else {
        IntegerMeanKernel<T, int32_t><<<static_cast<unsigned>(blocks), threads, 0, s>>>(
            static_cast<T*>(out), static_cast<const int32_t*>(ptr), rows, feat, batches);
    }
    return LaunchStatus();
}
}  // namespace csr
}  // namespace opsgnn

extern "C" int opsgnn_csr_integer_mean(void* out, int out_type, const void* ptr, int ptr_type, int64_t rows,
                                       int64_t feat, int64_t batches, void* stream)
{
    if (out == nullptr || ptr == nullptr || rows < 0 || feat < 0 || batches < 0 || !IsIndexType(ptr_type)) {
        return OPSGNN_ERR_INVALID;
    }
    cudaStream_t s = AsStream(stream);
    switch (out_type) {
        case OPSGNN_I8:
            return IntegerMean<int8_t>(out, ptr, ptr_type, rows, feat, batches, s);
        case OPSGNN_U8:
            return IntegerMean<uint8_t>(out, ptr, ptr_type, rows, feat, batches, s);
        case OPSGNN_I16:
            return IntegerMean<int16_t>(out, ptr, ptr_type, rows, feat, batches, s);
        case OPSGNN_I32:
            return IntegerMean<int32_t>(out, ptr, ptr_type, rows, feat, batches, s);
        case OPSGNN_I64:
            return IntegerMean<int64_t>(out, ptr, ptr_type, rows, feat, batches, s);
        default:
            return OPSGNN_ERR_UNSUPPORTED;
    }
}

extern "C" int opsgnn_csr_reduce_status(const void* workspace, void* stream, int64_t* stalled_waits)
{
    if (workspace == nullptr || stalled_waits == nullptr) {
        return OPSGNN_ERR_INVALID;
    }
    unsigned long long count = 0;
    cudaStream_t s = AsStream(stream);
    OPSGNN_CUDA_TRY(cudaMemcpyAsync(&count, workspace, sizeof(count), cudaMemcpyDeviceToHost, s));
    OPSGNN_CUDA_TRY(cudaStreamSynchronize(s));
    *stalled_waits = static_cast<int64_t>(count);
    return count == 0 ? OPSGNN_OK : OPSGNN_ERR_TIMEOUT;
}

extern "C" int opsgnn_set_status_sink(void* sink)
{
    int device = 0;
    OPSGNN_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) {
        return OPSGNN_ERR_LIMIT;
    }
    g_status_sink[device].store(static_cast<unsigned long long*>(sink), std::memory_order_relaxed);
    return OPSGNN_OK;
}

extern "C" int opsgnn_set_wait_polls(int64_t polls)
{
    g_wait_polls.store(polls, std::memory_order_relaxed);
    return OPSGNN_OK;
}

extern "C" const char* opsgnn_status_string(int status)
{
    switch (status) {
        case OPSGNN_OK:
            return "ok";
        case OPSGNN_ERR_INVALID:
            return "invalid argument";
        case OPSGNN_ERR_UNSUPPORTED:
            return "unsupported dtype or mode";
        case OPSGNN_ERR_WORKSPACE:
            return "workspace too small or misaligned";
        case OPSGNN_ERR_LIMIT:
            return "size beyond a fixed maximum";
        case OPSGNN_ERR_TIMEOUT:
            return "a bounded device-side wait ran out of polls";
        default:
            return status > 0 ? cudaGetErrorString(static_cast<cudaError_t>(status)) : "unknown status";
    }
}

extern "C" int opsgnn_sm_count(int* count)
{
    if (count == nullptr) {
        return OPSGNN_ERR_INVALID;
    }
    *count = SmCount();
    return OPSGNN_OK;
}
