// scatter(sum, mul, mean, min, max) with an unsorted index for sm_100a.
//
// src is viewed as [before, dim_len, after], out as [before, out_len, after]; element (b, p, a) is reduced into
// out[b, index(b, p, a), a] where the index is either one entry per position p ("compact") or one per element.
// Targets collide in arbitrary order, so the reduction runs on atomics:
//   sum / mean  red.global.add on the output itself (fp32 with after % 4 == 0 uses the 16-byte vector form, one
//               request per four features), or on a 32-bit shadow of it for the 8/16-bit dtypes, which have no atomic
//               add and would otherwise round every partial sum;
//   mul         compare-and-swap loop on the shadow;
//   min / max   atomic min / max on an order-preserving integer view of the value, then a second sweep that records,
//               for every element equal to the final extremum, the largest source position (the element the
//               reference's in-order `<=` / `>=` loop would have kept last), then a finalize sweep.
// NaN never wins an extremum; a target outside [0, out_len) is skipped (both as the reference's kernels do).
// Sums in floating point depend on the arrival order in their last bits; integers, extrema and positions do not.
//
// Algorithmic bytes per launch (sum): N*after*sizeof(T) + N*8 (index) + out_len*after*sizeof(T).
#include "common.cuh"

namespace opsgnn {
namespace scatter {

constexpr int kThreads = 256;

template <class T> struct ShadowOf { using type = T; };
template <> struct ShadowOf<__half> { using type = float; };
template <> struct ShadowOf<__nv_bfloat16> { using type = float; };
template <> struct ShadowOf<int8_t> { using type = int32_t; };
template <> struct ShadowOf<uint8_t> { using type = int32_t; };
template <> struct ShadowOf<int16_t> { using type = int32_t; };

struct Params {
    const void* src;
    const int64_t* index;
    void* out;
    int64_t* arg;
    void* shadow;         // accumulator array (== out when the dtype has native atomics)
    long long* count;     // mean: elements per target ([out_len] for a compact index, else [before, out_len, after])
    int64_t before, dim_len, after, out_len;
    int index_full;
    int reduce;
    int has_out;
};

inline unsigned Grid(int64_t items)
{
    int64_t blocks = CeilDiv(items, kThreads);
    const int64_t cap = static_cast<int64_t>(SmCount()) * 32;
    blocks = blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
    return static_cast<unsigned>(blocks);
}

// ---- atomics ------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void AtomicAdd(float* p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void AtomicAdd(double* p, double v) { atomicAdd(p, v); }
__device__ __forceinline__ void AtomicAdd(int32_t* p, int32_t v) { atomicAdd(p, v); }
__device__ __forceinline__ void AtomicAdd(int64_t* p, int64_t v)
{
    atomicAdd(reinterpret_cast<unsigned long long*>(p), static_cast<unsigned long long>(v));  // two's complement wrap
}

template <class S> __device__ __forceinline__ void AtomicMul(S* p, S v)
{
    if constexpr (sizeof(S) == 4) {
        unsigned* word = reinterpret_cast<unsigned*>(p);
        unsigned seen = *word, assumed;
        do {
            assumed = seen;
            S current;
            memcpy(&current, &assumed, 4);
            const S next = static_cast<S>(current * v);
            unsigned bits;
            memcpy(&bits, &next, 4);
            seen = atomicCAS(word, assumed, bits);
        } while (seen != assumed);
    } else {
        unsigned long long* word = reinterpret_cast<unsigned long long*>(p);
        unsigned long long seen = *word, assumed;
        do {
            assumed = seen;
            S current;
            memcpy(&current, &assumed, 8);
            const S next = static_cast<S>(current * v);
            unsigned long long bits;
            memcpy(&bits, &next, 8);
            seen = atomicCAS(word, assumed, bits);
        } while (seen != assumed);
    }
}

// Extremum on floats through the integer view: floats with a clear sign bit order like signed ints, floats with the sign
// bit set order in reverse like unsigned ints.  The branch is on the sign BIT, not on `v >= 0`: -0.0 compares equal to
// zero but its bits (0x80000000) are INT_MIN as a signed int, which would beat every stored negative in a signed min
// and lose to everything in a signed max.  On the unsigned path -0.0 sits just below +0.0, where it belongs.
__device__ __forceinline__ void AtomicExtremum(float* p, float v, bool is_min)
{
    const bool sign_clear = __float_as_int(v) >= 0;
    if (is_min) {
        if (sign_clear) {
            atomicMin(reinterpret_cast<int*>(p), __float_as_int(v));
        } else {
            atomicMax(reinterpret_cast<unsigned*>(p), __float_as_uint(v));
        }
    } else if (sign_clear) {
        atomicMax(reinterpret_cast<int*>(p), __float_as_int(v));
    } else {
        atomicMin(reinterpret_cast<unsigned*>(p), __float_as_uint(v));
    }
}
__device__ __forceinline__ void AtomicExtremum(double* p, double v, bool is_min)
{
    const bool sign_clear = __double_as_longlong(v) >= 0;
    if (is_min) {
        if (sign_clear) {
            atomicMin(reinterpret_cast<long long*>(p), __double_as_longlong(v));
        } else {
            atomicMax(reinterpret_cast<unsigned long long*>(p), static_cast<unsigned long long>(__double_as_longlong(v)));
        }
    } else if (sign_clear) {
        atomicMax(reinterpret_cast<long long*>(p), __double_as_longlong(v));
    } else {
        atomicMin(reinterpret_cast<unsigned long long*>(p), static_cast<unsigned long long>(__double_as_longlong(v)));
    }
}
__device__ __forceinline__ void AtomicExtremum(int32_t* p, int32_t v, bool is_min)
{
    if (is_min) {
        atomicMin(p, v);
    } else {
        atomicMax(p, v);
    }
}
__device__ __forceinline__ void AtomicExtremum(int64_t* p, int64_t v, bool is_min)
{
    if (is_min) {
        atomicMin(reinterpret_cast<long long*>(p), static_cast<long long>(v));
    } else {
        atomicMax(reinterpret_cast<long long*>(p), static_cast<long long>(v));
    }
}

// ---- kernels --------------------------------------------------------------------------------------------------------------
template <class T, class S> __global__ void WidenKernel(const T* __restrict__ out, S* __restrict__ shadow, int64_t n)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        shadow[i] = Widen<S, T>(out[i]);
    }
}

__device__ __forceinline__ int64_t TargetOf(const Params& p, int64_t b, int64_t pos, int64_t a)
{
    return p.index_full ? p.index[(b * p.dim_len + pos) * p.after + a] : p.index[pos];
}

template <class T, class S> __global__ void __launch_bounds__(kThreads) AccumulateKernel(const Params p)
{
    const T* __restrict__ src = static_cast<const T*>(p.src);
    S* __restrict__ shadow = static_cast<S*>(p.shadow);
    const int64_t total = p.before * p.dim_len * p.after;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const bool is_min = p.reduce == OPSGNN_SCATTER_MIN;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t a = i % p.after;
        const int64_t rest = i / p.after;
        const int64_t pos = rest % p.dim_len;
        const int64_t b = rest / p.dim_len;
        const int64_t target = TargetOf(p, b, pos, a);
        if (target < 0 || target >= p.out_len) {
            continue;
        }
        const int64_t at = (b * p.out_len + target) * p.after + a;
        const S value = Widen<S, T>(LoadStream(src + i));
        switch (p.reduce) {
            case OPSGNN_SCATTER_SUM:
                AtomicAdd(shadow + at, value);
                break;
            case OPSGNN_SCATTER_MEAN:
                AtomicAdd(shadow + at, value);
                if (p.index_full) {
                    atomicAdd(reinterpret_cast<unsigned long long*>(p.count + at), 1ULL);
                } else if (a == 0 && b == 0) {
                    atomicAdd(reinterpret_cast<unsigned long long*>(p.count + target), 1ULL);
                }
                break;
            case OPSGNN_SCATTER_MUL:
                AtomicMul<S>(shadow + at, value);
                break;
            default:
                if (value == value) {  // NaN never wins
                    AtomicExtremum(shadow + at, value, is_min);
                }
                break;
        }
    }
}

// fp32 sum with a compact index and after % 4 == 0: one 16-byte vector reduction per four features.
__global__ void __launch_bounds__(kThreads) AccumulateFloat4Kernel(const Params p)
{
    const float4* __restrict__ src = static_cast<const float4*>(p.src);
    float* __restrict__ out = static_cast<float*>(p.shadow);
    const int64_t quads = p.after >> 2;
    const int64_t total = p.before * p.dim_len * quads;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t q = i % quads;
        const int64_t rest = i / quads;
        const int64_t pos = rest % p.dim_len;
        const int64_t b = rest / p.dim_len;
        const int64_t target = p.index[pos];
        if (target < 0 || target >= p.out_len) {
            continue;
        }
        const float4 v = __ldcs(src + i);
        float* at = out + (b * p.out_len + target) * p.after + q * 4;
        atomicAdd(reinterpret_cast<float4*>(at), v);
        if (p.reduce == OPSGNN_SCATTER_MEAN && q == 0 && b == 0) {
            atomicAdd(reinterpret_cast<unsigned long long*>(p.count + target), 1ULL);
        }
    }
}

template <class T, class S> __global__ void __launch_bounds__(kThreads) ArgKernel(const Params p)
{
    const T* __restrict__ src = static_cast<const T*>(p.src);
    const S* __restrict__ shadow = static_cast<const S*>(p.shadow);
    const int64_t total = p.before * p.dim_len * p.after;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t a = i % p.after;
        const int64_t rest = i / p.after;
        const int64_t pos = rest % p.dim_len;
        const int64_t b = rest / p.dim_len;
        const int64_t target = TargetOf(p, b, pos, a);
        if (target < 0 || target >= p.out_len) {
            continue;
        }
        const int64_t at = (b * p.out_len + target) * p.after + a;
        const S value = Widen<S, T>(LoadStream(src + i));
        if (value == shadow[at]) {
            atomicMax(reinterpret_cast<long long*>(p.arg + at), static_cast<long long>(pos));
        }
    }
}

template <class T, class S> __global__ void __launch_bounds__(kThreads) FinalizeKernel(const Params p)
{
    T* __restrict__ out = static_cast<T*>(p.out);
    const S* __restrict__ shadow = static_cast<const S*>(p.shadow);
    const int64_t total = p.before * p.out_len * p.after;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const bool extremum = p.reduce == OPSGNN_SCATTER_MIN || p.reduce == OPSGNN_SCATTER_MAX;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        S value = shadow[i];
        if (p.reduce == OPSGNN_SCATTER_MEAN) {
            const int64_t target = (i / p.after) % p.out_len;
            const long long count = p.index_full ? p.count[i] : p.count[target];
            if (count > 0) {
                if constexpr (std::is_floating_point<S>::value) {
                    value = value / static_cast<S>(count);
                } else {
                    // Floor division; dtypes narrower than 32 bits wrap the count into their own range first and use
                    // at least 1, as the reference's finalize step does.  The numerator is the sum wrapped to T.
                    long long divisor = count;
                    if constexpr (sizeof(T) < 4) {
                        divisor = static_cast<long long>(static_cast<T>(count));
                        divisor = divisor < 1 ? 1 : divisor;
                    }
                    const long long numerator = static_cast<long long>(static_cast<T>(value));
                    long long quotient = numerator / divisor;
                    if ((numerator % divisor != 0) && ((numerator < 0) != (divisor < 0))) {
                        --quotient;
                    }
                    value = static_cast<S>(quotient);
                }
            }
        }
        if (extremum) {
            const int64_t where = p.arg[i];
            if (where < 0) {
                p.arg[i] = p.dim_len;
                if (!p.has_out) {
                    value = S(0);
                }
            }
        }
        out[i] = Narrow<T, S>(value);
    }
}

template <class T> int Run(Params p, cudaStream_t stream)
{
    using S = typename ShadowOf<T>::type;
    constexpr bool kShadowed = !std::is_same<T, S>::value;
    const int64_t out_elems = p.before * p.out_len * p.after;
    const int64_t src_elems = p.before * p.dim_len * p.after;
    const bool extremum = p.reduce == OPSGNN_SCATTER_MIN || p.reduce == OPSGNN_SCATTER_MAX;
    if (out_elems == 0) {
        return OPSGNN_OK;
    }
    if (kShadowed) {
        WidenKernel<T, S><<<Grid(out_elems), kThreads, 0, stream>>>(static_cast<const T*>(p.out), static_cast<S*>(p.shadow),
                                                                   out_elems);
    } else {
        p.shadow = p.out;
    }
    if (p.reduce == OPSGNN_SCATTER_MEAN) {
        const int64_t counters = p.index_full ? out_elems : p.out_len;
        OPSGNN_CUDA_TRY(cudaMemsetAsync(p.count, 0, counters * sizeof(long long), stream));
    }
    if (extremum) {
        OPSGNN_CUDA_TRY(cudaMemsetAsync(p.arg, 0xff, out_elems * sizeof(int64_t), stream));  // -1: nothing selected
    }
    if (src_elems > 0) {
        const bool vector_sum = std::is_same<T, float>::value && !p.index_full && p.after % 4 == 0 &&
                                (p.reduce == OPSGNN_SCATTER_SUM || p.reduce == OPSGNN_SCATTER_MEAN) &&
                                Aligned(p.src, 16) && Aligned(p.shadow, 16);
        if (vector_sum) {
            AccumulateFloat4Kernel<<<Grid(src_elems / 4), kThreads, 0, stream>>>(p);
        } else {
            AccumulateKernel<T, S><<<Grid(src_elems), kThreads, 0, stream>>>(p);
        }
        if (extremum) {
            ArgKernel<T, S><<<Grid(src_elems), kThreads, 0, stream>>>(p);
        }
    }
    if (kShadowed || extremum || p.reduce == OPSGNN_SCATTER_MEAN) {
        FinalizeKernel<T, S><<<Grid(out_elems), kThreads, 0, stream>>>(p);
    }
    return LaunchStatus();
}

inline int64_t ShadowBytes(int dtype)
{
    switch (dtype) {
        case OPSGNN_F16:
        case OPSGNN_BF16:
        case OPSGNN_I8:
        case OPSGNN_U8:
        case OPSGNN_I16:
            return 4;
        default:
            return 0;
    }
}

}  // namespace scatter
}  // namespace opsgnn

using namespace opsgnn;
using namespace opsgnn::scatter;

static int CheckScatterDesc(const OpsgnnScatterDesc* d)
{
    if (d == nullptr || d->before < 0 || d->dim_len < 0 || d->after < 0 || d->out_len < 0 ||
        d->reduce < OPSGNN_SCATTER_SUM || d->reduce > OPSGNN_SCATTER_MAX) {
        return OPSGNN_ERR_INVALID;
    }
    return DtypeBytes(d->dtype) == 0 ? OPSGNN_ERR_UNSUPPORTED : OPSGNN_OK;
}

extern "C" int opsgnn_scatter_workspace_bytes(const OpsgnnScatterDesc* desc, int64_t* bytes)
{
    const int status = CheckScatterDesc(desc);
    if (status != OPSGNN_OK || bytes == nullptr) {
        return status != OPSGNN_OK ? status : OPSGNN_ERR_INVALID;
    }
    const int64_t out_elems = desc->before * desc->out_len * desc->after;
    int64_t total = AlignUp(out_elems * ShadowBytes(desc->dtype), 256);
    if (desc->reduce == OPSGNN_SCATTER_MEAN) {
        total += AlignUp((desc->index_full ? out_elems : desc->out_len) * 8, 256);
    }
    *bytes = total;
    return OPSGNN_OK;
}

extern "C" int opsgnn_scatter(const OpsgnnScatterDesc* desc, const void* src, const int64_t* index, void* out,
                              int64_t* arg, void* workspace, int64_t workspace_bytes, void* stream)
{
    int status = CheckScatterDesc(desc);
    if (status != OPSGNN_OK) {
        return status;
    }
    const OpsgnnScatterDesc& d = *desc;
    const int64_t out_elems = d.before * d.out_len * d.after;
    const int64_t src_elems = d.before * d.dim_len * d.after;
    if (out_elems == 0) {
        return OPSGNN_OK;
    }
    const bool extremum = d.reduce == OPSGNN_SCATTER_MIN || d.reduce == OPSGNN_SCATTER_MAX;
    if (out == nullptr || (src_elems > 0 && (src == nullptr || index == nullptr)) || (extremum && arg == nullptr)) {
        return OPSGNN_ERR_INVALID;
    }
    int64_t needed = 0;
    opsgnn_scatter_workspace_bytes(desc, &needed);
    if (needed > 0 && (workspace == nullptr || workspace_bytes < needed || !Aligned(workspace, 256))) {
        return OPSGNN_ERR_WORKSPACE;
    }
    Params p{};
    p.src = src;
    p.index = index;
    p.out = out;
    p.arg = arg;
    char* cursor = static_cast<char*>(workspace);
    p.shadow = cursor;
    if (cursor != nullptr) {
        cursor += AlignUp(out_elems * ShadowBytes(d.dtype), 256);
    }
    p.count = reinterpret_cast<long long*>(cursor);
    p.before = d.before;
    p.dim_len = d.dim_len;
    p.after = d.after;
    p.out_len = d.out_len;
    p.index_full = d.index_full != 0;
    p.reduce = d.reduce;
    p.has_out = d.has_out;
    cudaStream_t s = AsStream(stream);
    switch (d.dtype) {
        case OPSGNN_F32:
            return Run<float>(p, s);
        case OPSGNN_F16:
            return Run<__half>(p, s);
        case OPSGNN_BF16:
            return Run<__nv_bfloat16>(p, s);
        case OPSGNN_F64:
            return Run<double>(p, s);
        case OPSGNN_I8:
            return Run<int8_t>(p, s);
        case OPSGNN_U8:
            return Run<uint8_t>(p, s);
        case OPSGNN_I16:
            return Run<int16_t>(p, s);
        case OPSGNN_I32:
            return Run<int32_t>(p, s);
        case OPSGNN_I64:
            return Run<int64_t>(p, s);
        default:
            return OPSGNN_ERR_UNSUPPORTED;
    }
}
