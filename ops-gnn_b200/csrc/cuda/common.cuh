// Shared device/host helpers of the sm_100a kernels: status plumbing, dtype traits,
// 16-byte vector load/store with fp32 widening, cache-hinted accesses.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <limits>
#include <type_traits>

#include "opsgnn_b200.h"

namespace opsgnn {

#define OPSGNN_CUDA_TRY(expr)                       \
    do {                                            \
        cudaError_t err__ = (expr);                 \
        if (err__ != cudaSuccess) {                 \
            return static_cast<int>(err__);         \
        }                                           \
    } while (0)

// Launch status without clearing a sticky error somebody else left behind.
inline int LaunchStatus()
{
    cudaError_t err = cudaPeekAtLastError();
    if (err != cudaSuccess) {
        (void)cudaGetLastError();
        return static_cast<int>(err);
    }
    return OPSGNN_OK;
}

inline cudaStream_t AsStream(void* stream) { return reinterpret_cast<cudaStream_t>(stream); }

inline int SmCount()
{
    static int cached[64] = {0};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
        return 148;
    }
    if (cached[device] == 0) {
        int count = 0;
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) {
            count = 148;
        }
        cached[device] = count;
    }
    return cached[device];
}

inline int64_t CeilDiv(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t AlignUp(int64_t a, int64_t b) { return CeilDiv(a, b) * b; }

inline int DtypeBytes(int dtype)
{
    switch (dtype) {
        case OPSGNN_F32:
        case OPSGNN_I32:
            return 4;
        case OPSGNN_F16:
        case OPSGNN_BF16:
        case OPSGNN_I16:
            return 2;
        case OPSGNN_I8:
        case OPSGNN_U8:
            return 1;
        case OPSGNN_I64:
        case OPSGNN_F64:
            return 8;
        default:
            return 0;
    }
}

// ---- accumulator type per storage type --------------------------------------
template <class T> struct AccOf { using type = T; };
template <> struct AccOf<__half> { using type = float; };
template <> struct AccOf<__nv_bfloat16> { using type = float; };
template <> struct AccOf<int8_t> { using type = int32_t; };
template <> struct AccOf<uint8_t> { using type = int32_t; };
template <> struct AccOf<int16_t> { using type = int32_t; };

template <class A, class T> __device__ __forceinline__ A Widen(T v) { return static_cast<A>(v); }
template <> __device__ __forceinline__ float Widen<float, __half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float Widen<float, __nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <class O, class A> __device__ __forceinline__ O Narrow(A v) { return static_cast<O>(v); }
template <> __device__ __forceinline__ __half Narrow<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 Narrow<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }

// ---- aligned vector of VEC elements of T ------------------------------------
template <class T, int VEC> struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };

// Widen a whole pack / narrow a whole array.  16-bit types go through their 32-bit words (two values per word) so
// the pack stays in registers; element-wise access to 2-byte members would push it to local memory.
template <class A, class T, int VEC> __device__ __forceinline__ void Unpack(const Pack<T, VEC>& p, A (&out)[VEC])
{
    if constexpr (sizeof(T) == 2 && VEC % 2 == 0 && std::is_same<A, float>::value &&
                  (std::is_same<T, __half>::value || std::is_same<T, __nv_bfloat16>::value)) {
        uint32_t words[VEC / 2];
        memcpy(words, &p, sizeof(words));
#pragma unroll
        for (int i = 0; i < VEC / 2; ++i) {
            if constexpr (std::is_same<T, __nv_bfloat16>::value) {
                out[2 * i] = __uint_as_float(words[i] << 16);
                out[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
            } else {
                __half2 pair;
                memcpy(&pair, &words[i], 4);
                const float2 f = __half22float2(pair);
                out[2 * i] = f.x;
                out[2 * i + 1] = f.y;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            out[i] = Widen<A, T>(p.v[i]);
        }
    }
}

template <class O, class A, int VEC> __device__ __forceinline__ Pack<O, VEC> Repack(const A (&in)[VEC])
{
    Pack<O, VEC> out;
    if constexpr (sizeof(O) == 2 && VEC % 2 == 0 && std::is_same<A, float>::value &&
                  (std::is_same<O, __half>::value || std::is_same<O, __nv_bfloat16>::value)) {
        uint32_t words[VEC / 2];
#pragma unroll
        for (int i = 0; i < VEC / 2; ++i) {
            if constexpr (std::is_same<O, __nv_bfloat16>::value) {
                const __nv_bfloat162 pair = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
                memcpy(&words[i], &pair, 4);
            } else {
                const __half2 pair = __floats2half2_rn(in[2 * i], in[2 * i + 1]);
                memcpy(&words[i], &pair, 4);
            }
        }
        memcpy(&out, words, sizeof(words));
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            out.v[i] = Narrow<O, A>(in[i]);
        }
    }
    return out;
}

// Scalar cache-hinted loads.  The toolkit's __ldg / __ldcs overloads for __half and __nv_bfloat16 are non-volatile
// inline asm, which the compiler may hoist above the branch that guards the pointer (a load through a null `val`
// pointer then faults even though the source never executes it).  16-bit values are therefore loaded through the
// unsigned short builtins, which are ordinary loads to the compiler, and bit-cast afterwards.
template <class T> __device__ __forceinline__ T LoadNc(const T* p)
{
    if constexpr (sizeof(T) == 2) {
        const unsigned short raw = __ldg(reinterpret_cast<const unsigned short*>(p));
        T out;
        memcpy(&out, &raw, 2);
        return out;
    } else {
        return __ldg(p);
    }
}

template <class T> __device__ __forceinline__ T LoadCs(const T* p)
{
    if constexpr (sizeof(T) == 2) {
        const unsigned short raw = __ldcs(reinterpret_cast<const unsigned short*>(p));
        T out;
        memcpy(&out, &raw, 2);
        return out;
    } else {
        return __ldcs(p);
    }
}

// Read-only gather through the non-coherent path (rows of the dense operand are never written by the kernel).
template <class T, int VEC> __device__ __forceinline__ Pack<T, VEC> LoadGather(const T* p)
{
    if constexpr (sizeof(T) * VEC == 16) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
        Pack<T, VEC> out;
        *reinterpret_cast<uint4*>(&out) = raw;
        return out;
    } else if constexpr (sizeof(T) * VEC == 8) {
        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
        Pack<T, VEC> out;
        *reinterpret_cast<uint2*>(&out) = raw;
        return out;
    } else {
        Pack<T, VEC> out;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            out.v[i] = LoadNc(p + i);
        }
        return out;
    }
}

// Streaming load: data read once (edge lists, sorted sources), evict-first in L2.
template <class T> __device__ __forceinline__ T LoadStream(const T* p) { return LoadCs(p); }

// Streaming store of an output row that is not read again by this kernel.
template <class T, int VEC> __device__ __forceinline__ void StoreStream(T* p, const Pack<T, VEC>& value)
{
    if constexpr (sizeof(T) * VEC == 16) {
        __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(&value));
    } else if constexpr (sizeof(T) * VEC == 8) {
        __stcs(reinterpret_cast<uint2*>(p), *reinterpret_cast<const uint2*>(&value));
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            p[i] = value.v[i];
        }
    }
}

template <class T, int VEC> __device__ __forceinline__ Pack<T, VEC> LoadPlain(const T* p)
{
    Pack<T, VEC> out;
    if constexpr (sizeof(T) * VEC == 16) {
        *reinterpret_cast<uint4*>(&out) = *reinterpret_cast<const uint4*>(p);
    } else if constexpr (sizeof(T) * VEC == 8) {
        *reinterpret_cast<uint2*>(&out) = *reinterpret_cast<const uint2*>(p);
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            out.v[i] = p[i];
        }
    }
    return out;
}

template <class T, int VEC> __device__ __forceinline__ void StorePlain(T* p, const Pack<T, VEC>& value)
{
    if constexpr (sizeof(T) * VEC == 16) {
        *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&value);
    } else if constexpr (sizeof(T) * VEC == 8) {
        *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(&value);
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            p[i] = value.v[i];
        }
    }
}

inline bool Aligned(const void* p, size_t bytes) { return (reinterpret_cast<uintptr_t>(p) % bytes) == 0; }

template <class T> struct Limits {
    __host__ __device__ static T Lowest() { return std::numeric_limits<T>::lowest(); }
    __host__ __device__ static T Max() { return std::numeric_limits<T>::max(); }
};
template <> struct Limits<float> {
    __host__ __device__ static float Lowest() { return -3.402823466e+38f; }
    __host__ __device__ static float Max() { return 3.402823466e+38f; }
};
template <> struct Limits<__half> {  // widest finite fp16, as fp32
    __host__ __device__ static float Lowest() { return -65504.0f; }
    __host__ __device__ static float Max() { return 65504.0f; }
};
template <> struct Limits<__nv_bfloat16> {  // widest finite bf16 (0x7f7f), as fp32
    __host__ __device__ static float Lowest() { return -3.3895313892515355e+38f; }
    __host__ __device__ static float Max() { return 3.3895313892515355e+38f; }
};
template <> struct Limits<double> {
    __host__ __device__ static double Lowest() { return -1.7976931348623157e+308; }
    __host__ __device__ static double Max() { return 1.7976931348623157e+308; }
};

}  // namespace opsgnn
