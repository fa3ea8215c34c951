// Grouped softmax / log-softmax / log-sum-exp over a 1-D index along one dimension, forward and backward, sm_100a.
//
// src is viewed as [batch, dim_len, after]; row p of every batch belongs to group index[p].  All arithmetic is fp32.
//
// Forward, sorted index (the common case: the index is the row id of a CSR graph): the index is turned into segment
// pointers by a boundary scan, the CSR reduce engine computes one fp32 log-sum-exp per (batch, group, feature) in a
// single sweep of src without atomics (online maximum + rescaled sum), and one more sweep writes
// exp(x - lse) or x - lse.  src is read twice and out written once.
// Forward, short groups (softmax / log-softmax, one batch, rows of whole 16-byte vectors, every group at most
// OPSGNN_GROUPED_SHORT_GROUP rows - the planner knows that from a cached fact about the index): SegmentSoftmaxKernel.
// A group of lanes owns a whole group of rows: it reads the rows, forms the log-sum-exp online, reads them again - from
// L1 / L2 now, the same lanes fetched them a moment ago - and writes exp(x - lse) or x - lse, so src crosses DRAM once
// and out once: the algorithmic bytes.  (Keeping the first rows in registers instead cost 158 registers and two thirds
// of the resident warps: 1.24 ms against 0.47 ms on the config-2 shape.)  With a permutation (a stable argsort of an UNSORTED index,
// made and cached by the planner) the same kernel reads and writes row perm[e] instead of row e: the unsorted case
// then needs no atomics and no fp32 scratch either.
// Forward, unsorted index without a permutation: the reference's three phases on fp32 scratch of shape [batch, groups, after]:
// atomic maximum, atomic sum of exp(x - max), then normalise (or max + log(sum) per group for log-sum-exp).
// Special values follow torch: a group holding +inf or only -inf gives NaN for softmax / log-softmax; log-sum-exp
// gives +inf / -inf for those groups and -inf for a group without members; NaN spreads over its group.
//
// Backward: softmax  grad = out * (g - sum_group(out * g)); log-softmax  grad = g - exp(out) * sum_group(g);
// log-sum-exp  grad = exp(src - out[group]) * g[group].  Group sums are fp32 atomic adds into scratch.
//
// Algorithmic bytes per forward launch (softmax): 2*N*after*sizeof(T) + N*sizeof(index).
#include "common.cuh"

namespace opsgnn {
namespace grouped {

constexpr int kThreads = 256;

struct Params {
    const void* src;
    const void* out_in;    // backward: forward output
    const void* grad_out;  // backward
    const void* index;
    void* out;             // forward result or grad_src
    float* top;            // [batch, groups, after] running maximum / fp32 log-sum-exp
    float* total;          // [batch, groups, after] sum of exponentials / backward group sums
    int64_t batch, dim_len, after, groups;
    int mode;
    int index64;
};

inline unsigned Grid(int64_t items)
{
    int64_t blocks = CeilDiv(items, kThreads);
    const int64_t cap = static_cast<int64_t>(SmCount()) * 32;
    blocks = blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
    return static_cast<unsigned>(blocks);
}

__device__ __forceinline__ int64_t GroupOf(const Params& p, int64_t pos)
{
    return p.index64 ? static_cast<const int64_t*>(p.index)[pos] : static_cast<const int32_t*>(p.index)[pos];
}

__device__ __forceinline__ void AtomicMaxFloat(float* address, float v)
{
    if (__float_as_int(v) >= 0) {  // the sign bit decides: -0.0 must take the unsigned path
        atomicMax(reinterpret_cast<int*>(address), __float_as_int(v));
    } else {
        atomicMin(reinterpret_cast<unsigned*>(address), __float_as_uint(v));
    }
}

__global__ void FillKernel(float* __restrict__ a, float va, float* __restrict__ b, float vb, int64_t n)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        if (a != nullptr) {
            a[i] = va;
        }
        if (b != nullptr) {
            b[i] = vb;
        }
    }
}

// Decode a flat element id into (batch, position, feature) and the flat id of its group statistic.
struct Where {
    int64_t stat;  // index into [batch, groups, after], or -1 when the group id is out of range
};
__device__ __forceinline__ Where Locate(const Params& p, int64_t i)
{
    const int64_t a = i % p.after;
    const int64_t rest = i / p.after;
    const int64_t pos = rest % p.dim_len;
    const int64_t b = rest / p.dim_len;
    const int64_t g = GroupOf(p, pos);
    if (g < 0 || g >= p.groups) {
        return {-1};
    }
    return {(b * p.groups + g) * p.after + a};
}

// ---- forward, unsorted -----------------------------------------------------------------------------------------------
template <class T> __global__ void __launch_bounds__(kThreads) MaxKernel(const Params p)
{
    const T* __restrict__ src = static_cast<const T*>(p.src);
    const int64_t n = p.batch * p.dim_len * p.after;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const Where w = Locate(p, i);
        const float x = Widen<float, T>(src[i]);
        if (w.stat >= 0 && x == x) {
            AtomicMaxFloat(p.top + w.stat, x);
        }
    }
}

__device__ __forceinline__ float Shift(const Params& p, float top)
{
    // log-sum-exp keeps infinite groups representable by clamping the shift to the finite range.
    if (p.mode == OPSGNN_GROUPED_LOGSUMEXP) {
        return fminf(fmaxf(top, -3.402823466e+38f), 3.402823466e+38f);
    }
    return top;
}

template <class T> __global__ void __launch_bounds__(kThreads) ExpSumKernel(const Params p)
{
    const T* __restrict__ src = static_cast<const T*>(p.src);
    const int64_t n = p.batch * p.dim_len * p.after;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const Where w = Locate(p, i);
        if (w.stat < 0) {
            continue;
        }
        const float x = Widen<float, T>(src[i]);
        atomicAdd(p.total + w.stat, __expf(x - Shift(p, p.top[w.stat])));
    }
}

template <class T> __global__ void __launch_bounds__(kThreads) NormalizeKernel(const Params p)
{
    const T* __restrict__ src = static_cast<const T*>(p.src);
    T* __restrict__ out = static_cast<T*>(p.out);
    const int64_t n = p.batch * p.dim_len * p.after;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const Where w = Locate(p, i);
        float result = 0.0f;
        if (w.stat >= 0) {
            const float shifted = Widen<float, T>(src[i]) - p.top[w.stat];
            const float sum = p.total[w.stat];
            result = p.mode == OPSGNN_GROUPED_SOFTMAX ? __expf(shifted) / sum : shifted - __logf(sum);
        }
        out[i] = Narrow<T, float>(result);
    }
}

template <class T> __global__ void __launch_bounds__(kThreads) FinishLogSumExpKernel(const Params p)
{
    T* __restrict__ out = static_cast<T*>(p.out);
    const int64_t n = p.batch * p.groups * p.after;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float sum = p.total[i];
        const float top = p.top[i];
        // No member: top is still -inf and the sum 0, which gives -inf as required.
        const float value = (sum == 0.0f && top == -INFINITY) ? -INFINITY : Shift(p, top) + __logf(sum);
        out[i] = Narrow<T, float>(value);
    }
}

// ---- forward, sorted -------------------------------------------------------------------------------------------------
// ptr[g] = number of index entries smaller than g (boundary scan of the sorted index).
template <class IndexT>
__global__ void BoundaryKernel(const IndexT* __restrict__ index, int64_t n, int64_t* __restrict__ ptr, int64_t groups,
                               const int64_t* __restrict__ perm = nullptr)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e <= n; e += stride) {
        // with a permutation the sorted sequence is index[perm[0]], index[perm[1]], ...
        int64_t prev = e == 0 ? -1 : static_cast<int64_t>(index[perm != nullptr ? perm[e - 1] : e - 1]);
        int64_t cur = e == n ? groups : static_cast<int64_t>(index[perm != nullptr ? perm[e] : e]);
        prev = prev < -1 ? -1 : (prev > groups ? groups : prev);
        cur = cur > groups ? groups : cur;
        for (int64_t g = prev + 1; g <= cur; ++g) {
            ptr[g] = e;
        }
    }
}

template <class T> __global__ void __launch_bounds__(kThreads) ApplyLseKernel(const Params p)
{
    const T* __restrict__ src = static_cast<const T*>(p.src);
    T* __restrict__ out = static_cast<T*>(p.out);
    const int64_t n = p.batch * p.dim_len * p.after;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const Where w = Locate(p, i);
        float result = 0.0f;
        if (w.stat >= 0) {
            const float lse = p.top[w.stat];
            const float x = Widen<float, T>(LoadStream(src + i));
            if (isfinite(lse)) {
                result = p.mode == OPSGNN_GROUPED_SOFTMAX ? __expf(x - lse) : x - lse;
            } else {
                result = NAN;  // +inf member, only -inf members, or NaN: torch.softmax gives NaN for the whole group
            }
        }
        out[i] = Narrow<T, float>(result);
    }
}

// Vector form for batch == 1 and `after` a multiple of the 16-byte vector width: one thread owns VEC consecutive
// features of one row, so the group id and the row decomposition are computed once per 16 bytes of src.
template <class T, int VEC> __global__ void __launch_bounds__(kThreads) ApplyLseVecKernel(const Params p)
{
    const T* __restrict__ src = static_cast<const T*>(p.src);
    T* __restrict__ out = static_cast<T*>(p.out);
    const int64_t per_row = p.after / VEC;
    const int64_t vectors = p.dim_len * per_row;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const bool small = vectors < (1LL << 32);
    for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < vectors; v += stride) {
        int64_t pos;
        if (small) {  // 32-bit division where it is exact
            pos = static_cast<unsigned>(v) / static_cast<unsigned>(per_row);
        } else {
            pos = v / per_row;
        }
        const int64_t a = (v - pos * per_row) * VEC;
        const int64_t g = GroupOf(p, pos);
        float result[VEC];
        if (g >= 0 && g < p.groups) {
            float x[VEC];
            Unpack<float, T, VEC>(LoadGather<T, VEC>(src + v * VEC), x);
            const float* __restrict__ lse_row = p.top + g * p.after + a;
#pragma unroll
            for (int c = 0; c < VEC; c += 4) {
                const float4 lse4 = __ldg(reinterpret_cast<const float4*>(lse_row + c));
                const float lse[4] = {lse4.x, lse4.y, lse4.z, lse4.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float shifted = x[c + q] - lse[q];
                    const float value = p.mode == OPSGNN_GROUPED_SOFTMAX ? __expf(shifted) : shifted;
                    result[c + q] = isfinite(lse[q]) ? value : NAN;  // same rule as the scalar kernel above
                }
            }
        } else {
#pragma unroll
            for (int c = 0; c < VEC; ++c) {
                result[c] = 0.0f;
            }
        }
        StoreStream<T, VEC>(out + v * VEC, Repack<T, float, VEC>(result));
    }
}


// ---- forward, short groups: one read of src, one write of out ---------------------------------------------------------
// `lanes` lanes (a power of two) own one group of rows at a time and `VEC` consecutive features each; a row wider than
// lanes * VEC features is walked tile by tile.  Row e of the (sorted) sequence is row perm[e] of src and out when a
// permutation is given.  Pseudo groups `groups` and `groups + 1` are the rows whose label lies below 0 or at / above
// `groups` (they come first / last in the sorted order): their output is 0, as in the other paths.
constexpr int kCachedRows = 4;

template <class T, int VEC> __global__ void __launch_bounds__(kThreads, 3) SegmentSoftmaxKernel(
    const Params p, const int64_t* __restrict__ ptr, const int64_t* __restrict__ perm, int lanes)
{
    const T* __restrict__ src = static_cast<const T*>(p.src);
    T* __restrict__ out = static_cast<T*>(p.out);
    const int lane = threadIdx.x & (lanes - 1);
    const int64_t team = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) / lanes;
    const int64_t teams = static_cast<int64_t>(gridDim.x) * kThreads / lanes;
    const int64_t vectors = p.after / VEC;
    for (int64_t g = team; g < p.groups + 2; g += teams) {
        const bool real = g < p.groups;
        const int64_t first = real ? ptr[g] : (g == p.groups ? 0 : ptr[p.groups]);
        const int64_t last = real ? ptr[g + 1] : (g == p.groups ? ptr[0] : p.dim_len);
        for (int64_t tile = lane; tile < vectors; tile += lanes) {
            const int64_t offset = tile * VEC;
            if (!real) {
                float zero[VEC];
#pragma unroll
                for (int c = 0; c < VEC; ++c) {
                    zero[c] = 0.0f;
                }
                for (int64_t e = first; e < last; ++e) {
                    const int64_t row = perm != nullptr ? perm[e] : e;
                    StoreStream<T, VEC>(out + row * p.after + offset, Repack<T, float, VEC>(zero));
                }
                continue;
            }
            float m[VEC], s[VEC];
#pragma unroll
            for (int c = 0; c < VEC; ++c) {
                m[c] = -INFINITY;
                s[c] = 0.0f;
            }
            // first sweep: online (maximum, scaled sum), kCachedRows rows per step with every load issued before the
            // first use, so a group costs as many round trips as it has steps, not as it has rows
            for (int64_t base = first; base < last; base += kCachedRows) {
                Pack<T, VEC> rows_in[kCachedRows];
#pragma unroll
                for (int k = 0; k < kCachedRows; ++k) {
                    if (base + k < last) {
                        const int64_t row = perm != nullptr ? perm[base + k] : base + k;
                        rows_in[k] = LoadGather<T, VEC>(src + row * p.after + offset);
                    }
                }
#pragma unroll
                for (int k = 0; k < kCachedRows; ++k) {
                    if (base + k < last) {
                        float x[VEC];
                        Unpack<float, T, VEC>(rows_in[k], x);
#pragma unroll
                        for (int c = 0; c < VEC; ++c) {
                            if (x[c] > m[c]) {
                                s[c] = s[c] * __expf(m[c] - x[c]) + 1.0f;
                                m[c] = x[c];
                            } else {
                                s[c] += __expf(x[c] == m[c] ? 0.0f : x[c] - m[c]);
                            }
                        }
                    }
                }
            }
            float lse[VEC];
#pragma unroll
            for (int c = 0; c < VEC; ++c) {
                lse[c] = s[c] == 0.0f ? m[c] : m[c] + __logf(s[c]);
            }
            // second sweep: the rows come back from L1 / L2 (the same lanes read them a moment ago), the result goes out
            // with streaming stores; a group with a +inf member, only -inf members or a NaN is NaN throughout
            for (int64_t base = first; base < last; base += kCachedRows) {
                Pack<T, VEC> rows_in[kCachedRows];
#pragma unroll
                for (int k = 0; k < kCachedRows; ++k) {
                    if (base + k < last) {
                        const int64_t row = perm != nullptr ? perm[base + k] : base + k;
                        rows_in[k] = LoadGather<T, VEC>(src + row * p.after + offset);
                    }
                }
#pragma unroll
                for (int k = 0; k < kCachedRows; ++k) {
                    if (base + k < last) {
                        const int64_t row = perm != nullptr ? perm[base + k] : base + k;
                        float x[VEC], y[VEC];
                        Unpack<float, T, VEC>(rows_in[k], x);
#pragma unroll
                        for (int c = 0; c < VEC; ++c) {
                            const float shifted = x[c] - lse[c];
                            const float value = p.mode == OPSGNN_GROUPED_SOFTMAX ? __expf(shifted) : shifted;
                            y[c] = isfinite(lse[c]) ? value : NAN;
                        }
                        StoreStream<T, VEC>(out + row * p.after + offset, Repack<T, float, VEC>(y));
                    }
                }
            }
        }
    }
}

template <class T> __global__ void CastKernel(const float* __restrict__ in, T* __restrict__ out, int64_t n)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        out[i] = Narrow<T, float>(in[i]);
    }
}

// ---- backward ---------------------------------------------------------------------------------------------------------
template <class T> __global__ void __launch_bounds__(kThreads) GradSumKernel(const Params p)
{
    const T* __restrict__ fwd = static_cast<const T*>(p.out_in);
    const T* __restrict__ grad = static_cast<const T*>(p.grad_out);
    const int64_t n = p.batch * p.dim_len * p.after;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const Where w = Locate(p, i);
        if (w.stat < 0) {
            continue;
        }
        const float g = Widen<float, T>(grad[i]);
        const float term = p.mode == OPSGNN_GROUPED_SOFTMAX ? g * Widen<float, T>(fwd[i]) : g;
        atomicAdd(p.total + w.stat, term);
    }
}

template <class T> __global__ void __launch_bounds__(kThreads) GradKernel(const Params p)
{
    const T* __restrict__ src = static_cast<const T*>(p.src);
    const T* __restrict__ fwd = static_cast<const T*>(p.out_in);
    const T* __restrict__ grad = static_cast<const T*>(p.grad_out);
    T* __restrict__ out = static_cast<T*>(p.out);
    const int64_t n = p.batch * p.dim_len * p.after;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const Where w = Locate(p, i);
        float result = 0.0f;
        if (w.stat >= 0) {
            if (p.mode == OPSGNN_GROUPED_SOFTMAX) {
                const float y = Widen<float, T>(fwd[i]);
                result = y * (Widen<float, T>(grad[i]) - p.total[w.stat]);
            } else if (p.mode == OPSGNN_GROUPED_LOG_SOFTMAX) {
                result = Widen<float, T>(grad[i]) - __expf(Widen<float, T>(fwd[i])) * p.total[w.stat];
            } else {
                // fwd and grad are per group here: [batch, groups, after]
                const float lse = Widen<float, T>(fwd[w.stat]);
                const float weight = __expf(Widen<float, T>(src[i]) - lse);
                const float g = Widen<float, T>(grad[w.stat]);
                result = weight * g;  // +inf member or all -inf group: inf - inf = NaN, as torch.logsumexp's gradient
            }
        }
        out[i] = Narrow<T, float>(result);
    }
}

struct Layout {
    int64_t stats;       // floats per statistic array
    int64_t top_off, total_off, ptr_off, plan_off, carry_off, carry_bytes, total_bytes;
    int64_t sweep_off, sweep_bytes;  // eight-column fp32 sources under sorted labels: the chunked sweep's boundary arrays
};

inline Layout MakeLayout(const OpsgnnGroupedDesc& d)
{
    Layout l{};
    l.stats = d.batch * d.groups * d.after;
    int64_t cursor = 0;
    l.top_off = cursor;
    cursor += AlignUp(l.stats * 4, 256);
    l.total_off = cursor;
    cursor += AlignUp(l.stats * 4, 256);
    if (d.sorted) {  // also the permuted form: the boundary scan runs over the sorted sequence
        l.ptr_off = cursor;
        cursor += AlignUp((d.groups + 1) * 8, 256);
        int64_t plan_bytes = 0;
        opsgnn_csr_plan_bytes(d.groups, d.dim_len, &plan_bytes);
        l.plan_off = cursor;
        cursor += AlignUp(plan_bytes, 256);
        OpsgnnCsrReduceDesc r{};
        r.rows = d.groups;
        r.src_rows = d.dim_len;
        r.feat = d.after;
        r.nnz = d.dim_len;
        r.batches = d.batch;
        r.reduce = OPSGNN_REDUCE_LOGSUMEXP;
        r.ptr_type = OPSGNN_I64;
        r.col_type = OPSGNN_I64;
        r.in_type = d.dtype;
        r.out_type = OPSGNN_F32;
        opsgnn_csr_reduce_workspace_bytes(&r, &l.carry_bytes);
        l.carry_off = cursor;
        cursor += AlignUp(l.carry_bytes, 256);
        if (d.batch == 1 && d.after == 8 && d.dtype == OPSGNN_F32) {
            opsgnn_sorted_lse8_workspace_bytes(d.dim_len, &l.sweep_bytes);
            l.sweep_off = cursor;
            cursor += AlignUp(l.sweep_bytes, 256);
        }
    }
    l.total_bytes = cursor;
    return l;
}

template <class T> bool ShortGroupShape(const OpsgnnGroupedDesc& d, const Params& p)
{
    constexpr int kVec = 16 / sizeof(T);
    return d.mode != OPSGNN_GROUPED_LOGSUMEXP && d.batch == 1 && d.after % kVec == 0 && Aligned(p.src, 16) && Aligned(p.out, 16);
}

template <class T>
int Forward(const OpsgnnGroupedDesc& d, Params p, char* workspace, const Layout& l, cudaStream_t s, const int64_t* perm = nullptr,
            const int64_t* ready_ptr = nullptr, const void* ready_plan = nullptr)
{
    const int64_t n = d.batch * d.dim_len * d.after;
    auto apply_lse = [&]() {  // second pass of the sorted forms: p.top holds the log-sum-exp of every group
        if (d.mode == OPSGNN_GROUPED_LOGSUMEXP) {
            CastKernel<T><<<Grid(l.stats), kThreads, 0, s>>>(p.top, static_cast<T*>(p.out), l.stats);
        } else {
            constexpr int kVec = 16 / sizeof(T);
            if (d.batch == 1 && d.after % kVec == 0 && Aligned(p.src, 16) && Aligned(p.out, 16) && Aligned(p.top, 16)) {
                ApplyLseVecKernel<T, kVec><<<Grid(n / kVec), kThreads, 0, s>>>(p);
            } else {
                ApplyLseKernel<T><<<Grid(n), kThreads, 0, s>>>(p);
            }
        }
        return LaunchStatus();
    };
    if constexpr (std::is_same<T, float>::value) {
        // Eight fp32 columns (per-head attention logits) under sorted labels: rows of 32 bytes are too narrow for the
        // engine's ring (2.15 ms for 34.5M rows), so the first pass is the attention layer's chunked sweep over the
        // values (no segment pointers, no plan).
        if (d.sorted == 1 && perm == nullptr && n > 0 && l.stats > 0 && l.sweep_bytes > 0 && Aligned(p.src, 16) &&
            Aligned(p.top, 16)) {
            const int status = opsgnn_sorted_lse8(p.index, p.index64 ? OPSGNN_I64 : OPSGNN_I32, static_cast<const float*>(p.src),
                                                  p.top, d.dim_len, d.groups, workspace + l.sweep_off, l.sweep_bytes, s);
            if (status != OPSGNN_OK) {
                return status;
            }
            return apply_lse();
        }
    }
    if (d.sorted && n > 0 && l.stats > 0) {
        int64_t* ptr = reinterpret_cast<int64_t*>(workspace + l.ptr_off);
        if (ready_ptr != nullptr) {  // prepared once for these labels: no boundary scan, no plan build
            ptr = const_cast<int64_t*>(ready_ptr);
        } else if (p.index64) {
            BoundaryKernel<int64_t><<<Grid(d.dim_len + 1), kThreads, 0, s>>>(static_cast<const int64_t*>(p.index), d.dim_len,
                                                                         ptr, d.groups, perm);
        } else {
            BoundaryKernel<int32_t><<<Grid(d.dim_len + 1), kThreads, 0, s>>>(static_cast<const int32_t*>(p.index), d.dim_len,
                                                                         ptr, d.groups, perm);
        }
        if (d.sorted == OPSGNN_GROUPED_SORTED_SHORT || perm != nullptr) {
            if (!ShortGroupShape<T>(d, p)) {
                return OPSGNN_ERR_UNSUPPORTED;
            }
            constexpr int kVec = 16 / sizeof(T);
            const int64_t vectors = d.after / kVec;
            int lanes = 1;
            while (lanes < 32 && lanes < vectors) {
                lanes <<= 1;
            }
            int64_t blocks = CeilDiv((d.groups + 2) * lanes, kThreads);
            const int64_t cap = static_cast<int64_t>(SmCount()) * 32;
            blocks = blocks < cap ? blocks : cap;
            SegmentSoftmaxKernel<T, kVec><<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(p, ptr, perm, lanes);
            return LaunchStatus();
        }
        int status = OPSGNN_OK;
        const void* plan = ready_plan;
        if (plan == nullptr || ready_ptr == nullptr) {
            status = opsgnn_csr_plan_build(ptr, OPSGNN_I64, d.groups, d.dim_len, workspace + l.plan_off, s);
            if (status != OPSGNN_OK) {
                return status;
            }
            plan = workspace + l.plan_off;
        }
        OpsgnnCsrReduceDesc r{};
        r.rows = d.groups;
        r.src_rows = d.dim_len;
        r.feat = d.after;
        r.nnz = d.dim_len;
        r.batches = d.batch;
        r.reduce = OPSGNN_REDUCE_LOGSUMEXP;
        r.ptr_type = OPSGNN_I64;
        r.col_type = OPSGNN_I64;
        r.in_type = d.dtype;
        r.out_type = OPSGNN_F32;
        status = opsgnn_csr_reduce(&r, ptr, nullptr, nullptr, p.src, p.top, nullptr, plan, workspace + l.carry_off,
                                   l.carry_bytes, s);
        if (status != OPSGNN_OK) {
            return status;
        }
        return apply_lse();
    }
    if (l.stats > 0) {
        FillKernel<<<Grid(l.stats), kThreads, 0, s>>>(p.top, -INFINITY, p.total, 0.0f, l.stats);
    }
    if (n > 0 && l.stats > 0) {
        MaxKernel<T><<<Grid(n), kThreads, 0, s>>>(p);
        ExpSumKernel<T><<<Grid(n), kThreads, 0, s>>>(p);
    }
    if (d.mode == OPSGNN_GROUPED_LOGSUMEXP) {
        if (l.stats > 0) {
            FinishLogSumExpKernel<T><<<Grid(l.stats), kThreads, 0, s>>>(p);
        }
    } else if (n > 0) {
        NormalizeKernel<T><<<Grid(n), kThreads, 0, s>>>(p);
    }
    return LaunchStatus();
}

template <class T> int Backward(const OpsgnnGroupedDesc& d, Params p, const Layout& l, cudaStream_t s)
{
    const int64_t n = d.batch * d.dim_len * d.after;
    if (n == 0) {
        return OPSGNN_OK;
    }
    if (d.mode != OPSGNN_GROUPED_LOGSUMEXP) {
        FillKernel<<<Grid(l.stats), kThreads, 0, s>>>(nullptr, 0.0f, p.total, 0.0f, l.stats);
        GradSumKernel<T><<<Grid(n), kThreads, 0, s>>>(p);
    }
    GradKernel<T><<<Grid(n), kThreads, 0, s>>>(p);
    return LaunchStatus();
}

inline int CheckDesc(const OpsgnnGroupedDesc* d)
{
    if (d == nullptr || d->batch < 0 || d->dim_len < 0 || d->after < 0 || d->groups < 0 ||
        d->mode < OPSGNN_GROUPED_SOFTMAX || d->mode > OPSGNN_GROUPED_LOGSUMEXP ||
        (d->index_type != OPSGNN_I32 && d->index_type != OPSGNN_I64)) {
        return OPSGNN_ERR_INVALID;
    }
    if (d->dtype != OPSGNN_F32 && d->dtype != OPSGNN_F16 && d->dtype != OPSGNN_BF16) {
        return OPSGNN_ERR_UNSUPPORTED;
    }
    return OPSGNN_OK;
}

}  // namespace grouped
}  // namespace opsgnn

using namespace opsgnn;
using namespace opsgnn::grouped;

extern "C" int opsgnn_grouped_workspace_bytes(const OpsgnnGroupedDesc* desc, int64_t* bytes)
{
    const int status = CheckDesc(desc);
    if (status != OPSGNN_OK || bytes == nullptr) {
        return status != OPSGNN_OK ? status : OPSGNN_ERR_INVALID;
    }
    *bytes = MakeLayout(*desc).total_bytes;
    return OPSGNN_OK;
}

static Params MakeParams(const OpsgnnGroupedDesc& d, char* workspace, const Layout& l)
{
    Params p{};
    p.top = reinterpret_cast<float*>(workspace + l.top_off);
    p.total = reinterpret_cast<float*>(workspace + l.total_off);
    p.batch = d.batch;
    p.dim_len = d.dim_len;
    p.after = d.after;
    p.groups = d.groups;
    p.mode = d.mode;
    p.index64 = d.index_type == OPSGNN_I64;
    return p;
}

extern "C" int opsgnn_grouped_forward(const OpsgnnGroupedDesc* desc, const void* src, const void* index, void* out,
                                      void* workspace, int64_t workspace_bytes, void* stream)
{
    int status = CheckDesc(desc);
    if (status != OPSGNN_OK) {
        return status;
    }
    const OpsgnnGroupedDesc& d = *desc;
    const Layout l = MakeLayout(d);
    const int64_t n = d.batch * d.dim_len * d.after;
    const int64_t out_elems = d.mode == OPSGNN_GROUPED_LOGSUMEXP ? l.stats : n;
    if (out_elems == 0) {
        return OPSGNN_OK;
    }
    if (out == nullptr || (n > 0 && (src == nullptr || index == nullptr))) {
        return OPSGNN_ERR_INVALID;
    }
    if (workspace == nullptr || workspace_bytes < l.total_bytes || !Aligned(workspace, 256)) {
        return OPSGNN_ERR_WORKSPACE;
    }
    Params p = MakeParams(d, static_cast<char*>(workspace), l);
    p.src = src;
    p.index = index;
    p.out = out;
    cudaStream_t s = AsStream(stream);
    switch (d.dtype) {
        case OPSGNN_F32:
            return Forward<float>(d, p, static_cast<char*>(workspace), l, s);
        case OPSGNN_F16:
            return Forward<__half>(d, p, static_cast<char*>(workspace), l, s);
        default:
            return Forward<__nv_bfloat16>(d, p, static_cast<char*>(workspace), l, s);
    }
}

extern "C" int opsgnn_grouped_prepare(const OpsgnnGroupedDesc* desc, const void* index, int64_t* ptr, void* plan, void* stream)
{
    int status = CheckDesc(desc);
    if (status != OPSGNN_OK) {
        return status;
    }
    const OpsgnnGroupedDesc& d = *desc;
    if (ptr == nullptr || plan == nullptr || (d.dim_len > 0 && index == nullptr) || !Aligned(plan, 256)) {
        return OPSGNN_ERR_INVALID;
    }
    cudaStream_t s = AsStream(stream);
    if (d.index_type == OPSGNN_I64) {
        BoundaryKernel<int64_t><<<Grid(d.dim_len + 1), kThreads, 0, s>>>(static_cast<const int64_t*>(index), d.dim_len, ptr,
                                                                     d.groups, nullptr);
    } else {
        BoundaryKernel<int32_t><<<Grid(d.dim_len + 1), kThreads, 0, s>>>(static_cast<const int32_t*>(index), d.dim_len, ptr,
                                                                     d.groups, nullptr);
    }
    status = LaunchStatus();
    if (status != OPSGNN_OK) {
        return status;
    }
    return opsgnn_csr_plan_build(ptr, OPSGNN_I64, d.groups, d.dim_len, plan, s);
}

extern "C" int opsgnn_grouped_forward_prepared(const OpsgnnGroupedDesc* desc, const void* src, const void* index,
                                               const int64_t* ptr, const void* plan, void* out, void* workspace,
                                               int64_t workspace_bytes, void* stream)
{
    int status = CheckDesc(desc);
    if (status != OPSGNN_OK) {
        return status;
    }
    const OpsgnnGroupedDesc& d = *desc;
    if (d.sorted != 1 || ptr == nullptr || plan == nullptr) {
        return OPSGNN_ERR_INVALID;
    }
    const Layout l = MakeLayout(d);
    const int64_t n = d.batch * d.dim_len * d.after;
    const int64_t out_elems = d.mode == OPSGNN_GROUPED_LOGSUMEXP ? l.stats : n;
    if (out_elems == 0) {
        return OPSGNN_OK;
    }
    if (out == nullptr || (n > 0 && (src == nullptr || index == nullptr))) {
        return OPSGNN_ERR_INVALID;
    }
    if (workspace == nullptr || workspace_bytes < l.total_bytes || !Aligned(workspace, 256)) {
        return OPSGNN_ERR_WORKSPACE;
    }
    Params p = MakeParams(d, static_cast<char*>(workspace), l);
    p.src = src;
    p.index = index;
    p.out = out;
    cudaStream_t s = AsStream(stream);
    switch (d.dtype) {
        case OPSGNN_F32:
            return Forward<float>(d, p, static_cast<char*>(workspace), l, s, nullptr, ptr, plan);
        case OPSGNN_F16:
            return Forward<__half>(d, p, static_cast<char*>(workspace), l, s, nullptr, ptr, plan);
        default:
            return Forward<__nv_bfloat16>(d, p, static_cast<char*>(workspace), l, s, nullptr, ptr, plan);
    }
}

extern "C" int opsgnn_grouped_forward_permuted(const OpsgnnGroupedDesc* desc, const void* src, const void* index,
                                               const int64_t* perm, void* out, void* workspace, int64_t workspace_bytes,
                                               void* stream)
{
    int status = CheckDesc(desc);
    if (status != OPSGNN_OK) {
        return status;
    }
    OpsgnnGroupedDesc d = *desc;
    if (d.mode == OPSGNN_GROUPED_LOGSUMEXP) {
        return OPSGNN_ERR_UNSUPPORTED;
    }
    d.sorted = OPSGNN_GROUPED_SORTED_SHORT;  // the sequence index[perm[.]] is sorted and its groups are short
    const Layout l = MakeLayout(d);
    const int64_t n = d.batch * d.dim_len * d.after;
    if (n == 0) {
        return OPSGNN_OK;
    }
    if (out == nullptr || src == nullptr || index == nullptr || perm == nullptr) {
        return OPSGNN_ERR_INVALID;
    }
    if (workspace == nullptr || workspace_bytes < l.total_bytes || !Aligned(workspace, 256)) {
        return OPSGNN_ERR_WORKSPACE;
    }
    Params p = MakeParams(d, static_cast<char*>(workspace), l);
    p.src = src;
    p.index = index;
    p.out = out;
    cudaStream_t s = AsStream(stream);
    switch (d.dtype) {
        case OPSGNN_F32:
            return Forward<float>(d, p, static_cast<char*>(workspace), l, s, perm);
        case OPSGNN_F16:
            return Forward<__half>(d, p, static_cast<char*>(workspace), l, s, perm);
        default:
            return Forward<__nv_bfloat16>(d, p, static_cast<char*>(workspace), l, s, perm);
    }
}

extern "C" int opsgnn_grouped_backward(const OpsgnnGroupedDesc* desc, const void* src, const void* out,
                                       const void* grad_out, const void* index, void* grad_src, void* workspace,
                                       int64_t workspace_bytes, void* stream)
{
    int status = CheckDesc(desc);
    if (status != OPSGNN_OK) {
        return status;
    }
    const OpsgnnGroupedDesc& d = *desc;
    const Layout l = MakeLayout(d);
    const int64_t n = d.batch * d.dim_len * d.after;
    if (n == 0) {
        return OPSGNN_OK;
    }
    if (out == nullptr || grad_out == nullptr || index == nullptr || grad_src == nullptr ||
        (d.mode == OPSGNN_GROUPED_LOGSUMEXP && src == nullptr)) {
        return OPSGNN_ERR_INVALID;
    }
    if (workspace == nullptr || workspace_bytes < l.total_bytes || !Aligned(workspace, 256)) {
        return OPSGNN_ERR_WORKSPACE;
    }
    Params p = MakeParams(d, static_cast<char*>(workspace), l);
    p.src = src;
    p.out_in = out;
    p.grad_out = grad_out;
    p.index = index;
    p.out = grad_src;
    cudaStream_t s = AsStream(stream);
    switch (d.dtype) {
        case OPSGNN_F32:
            return Backward<float>(d, p, l, s);
        case OPSGNN_F16:
            return Backward<__half>(d, p, l, s);
        default:
            return Backward<__nv_bfloat16>(d, p, l, s);
    }
}
