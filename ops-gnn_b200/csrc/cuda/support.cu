// Index conversions and CSR support kernels: ind2ptr, ptr2ind, CSR validation, value permutation, index statistics
// and the edge-value gradient of SpMM.  All of them are integer / streaming work bounded by HBM bandwidth.
#include "common.cuh"

namespace opsgnn {
namespace support {

constexpr int kThreads = 256;

inline unsigned StreamGrid(int64_t items, int per_thread = 1)
{
    int64_t blocks = CeilDiv(items, static_cast<int64_t>(kThreads) * per_thread);
    const int64_t cap = static_cast<int64_t>(SmCount()) * 32;
    blocks = blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
    return static_cast<unsigned>(blocks);
}

// ---- ind2ptr: boundaries of a sorted index ------------------------------------------------------------------------
// Thread e looks at the pair (ind[e-1], ind[e]) and fills ptr for every row that starts between them, so the sorted
// index is read once, coalesced; ptr[r] = number of entries smaller than r.
__global__ void Ind2PtrKernel(const int64_t* __restrict__ ind, int64_t nnz, int64_t* __restrict__ ptr, int64_t rows)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e <= nnz; e += stride) {
        int64_t prev = e == 0 ? -1 : LoadStream(ind + e - 1);
        int64_t cur = e == nnz ? rows : LoadStream(ind + e);
        prev = prev < -1 ? -1 : (prev > rows ? rows : prev);  // out-of-contract input must not write outside ptr
        cur = cur > rows ? rows : cur;
        for (int64_t r = prev + 1; r <= cur; ++r) {
            ptr[r] = e;
        }
    }
}

// ---- ptr2ind --------------------------------------------------------------------------------------------------------
// A block owns kEdgesPerBlock consecutive edges, finds the rows of its first and last edge with two binary searches,
// stages that slice of ptr in shared memory and lets every thread locate its edges there.
constexpr int kEdgesPerBlock = 2048;

__device__ __forceinline__ int64_t RowOfEdge(const int64_t* ptr, int64_t lo, int64_t hi, int64_t edge)
{
    // largest r in [lo, hi] with ptr[r] <= edge, given ptr[lo] <= edge
    while (lo < hi) {
        const int64_t mid = (lo + hi + 1) >> 1;
        if (ptr[mid] <= edge) {
            lo = mid;
        } else {
            hi = mid - 1;
        }
    }
    return lo;
}

__global__ void __launch_bounds__(kThreads) Ptr2IndKernel(const int64_t* __restrict__ ptr, int64_t rows,
                                                           int64_t* __restrict__ ind, int64_t nnz)
{
    __shared__ int64_t s_ptr[kEdgesPerBlock + 1];
    __shared__ int64_t s_first, s_last;
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kEdgesPerBlock;
    const int64_t end = base + kEdgesPerBlock < nnz ? base + kEdgesPerBlock : nnz;
    if (threadIdx.x == 0) {
        s_first = RowOfEdge(ptr, 0, rows > 0 ? rows - 1 : 0, base);
    } else if (threadIdx.x == 32) {
        s_last = RowOfEdge(ptr, 0, rows > 0 ? rows - 1 : 0, end - 1);
    }
    __syncthreads();
    const int64_t first = s_first;
    const int64_t span = s_last - first + 1;
    const bool staged = span <= kEdgesPerBlock;
    if (staged) {
        for (int64_t i = threadIdx.x; i < span; i += kThreads) {
            s_ptr[i] = ptr[first + i];
        }
    }
    __syncthreads();
    for (int64_t e = base + threadIdx.x; e < end; e += kThreads) {
        int64_t row;
        if (staged) {
            row = first + RowOfEdge(s_ptr, 0, span - 1, e);
        } else {
            row = RowOfEdge(ptr, first, s_last, e);
        }
        ind[e] = row;
    }
}

// ---- CSR validation ---------------------------------------------------------------------------------------------------
// Flags: 1 endpoints (ptr[0] != 0 or ptr[rows] != nnz), 2 pointer outside [0, nnz], 4 decreasing pointer,
// 8 column outside [0, cols).
template <class IndexT>
__global__ void ValidateKernel(const IndexT* __restrict__ ptr, const IndexT* __restrict__ col, int64_t rows,
                               int64_t cols, int64_t nnz, int32_t* __restrict__ status)
{
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    int32_t bad = 0;
    for (int64_t i = tid; i <= rows; i += stride) {
        const int64_t v = ptr[i];
        if ((i == 0 && v != 0) || (i == rows && v != nnz)) {
            bad |= 1;
        }
        if (v < 0 || v > nnz) {
            bad |= 2;
        }
        if (i < rows && v > static_cast<int64_t>(ptr[i + 1])) {
            bad |= 4;
        }
    }
    if (col != nullptr) {
        for (int64_t i = tid; i < nnz; i += stride) {
            const int64_t c = LoadStream(col + i);
            if (c < 0 || c >= cols) {
                bad |= 8;
            }
        }
    }
    bad = __reduce_or_sync(0xffffffffu, bad);
    if ((threadIdx.x & 31) == 0 && bad != 0) {
        atomicOr(status, bad);
    }
}

// ---- value permutation -------------------------------------------------------------------------------------------------
template <class T>
__global__ void PermuteKernel(const int64_t* __restrict__ perm, const T* __restrict__ value, T* __restrict__ out,
                              int64_t rows, int64_t width)
{
    const int64_t total = rows * width;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t r = i / width;
        int64_t from = perm[r];
        from = from < 0 ? 0 : (from >= rows ? rows - 1 : from);
        out[i] = value[from * width + (i - r * width)];
    }
}

// ---- index statistics --------------------------------------------------------------------------------------------------
__global__ void StatsInitKernel(int64_t* stats)
{
    stats[0] = 0x7fffffffffffffffLL;
    stats[1] = -0x7fffffffffffffffLL - 1;
    stats[2] = 1;
}

template <class IndexT>
__global__ void StatsKernel(const IndexT* __restrict__ index, int64_t n, int64_t* __restrict__ stats)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    long long lo = 0x7fffffffffffffffLL, hi = -0x7fffffffffffffffLL - 1;
    int unsorted = 0;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const long long v = index[i];
        lo = v < lo ? v : lo;
        hi = v > hi ? v : hi;
        if (i > 0 && static_cast<long long>(index[i - 1]) > v) {
            unsorted = 1;
        }
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
        const long long other_lo = __shfl_xor_sync(0xffffffffu, lo, offset);
        const long long other_hi = __shfl_xor_sync(0xffffffffu, hi, offset);
        lo = other_lo < lo ? other_lo : lo;
        hi = other_hi > hi ? other_hi : hi;
    }
    unsorted = __any_sync(0xffffffffu, unsorted);
    if ((threadIdx.x & 31) == 0) {
        atomicMin(reinterpret_cast<long long*>(stats), lo);
        atomicMax(reinterpret_cast<long long*>(stats + 1), hi);
        if (unsorted) {
            atomicExch(reinterpret_cast<unsigned long long*>(stats + 2), 0ULL);
        }
    }
}

// Longest run of equal consecutive values of a NON-DECREASING index (the largest group of a sorted label vector): every
// run start finds its end by a binary search for the first larger value.  On an index that is not sorted the result means
// nothing (the search still ends).
template <class IndexT>
__global__ void LongestRunKernel(const IndexT* __restrict__ index, const int64_t* __restrict__ perm, int64_t n,
                                 int64_t* __restrict__ longest)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    long long best = 0;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const long long v = index[perm != nullptr ? perm[i] : i];
        if (i > 0 && static_cast<long long>(index[perm != nullptr ? perm[i - 1] : i - 1]) == v) {
            continue;  // not a run start
        }
        int64_t lo = i + 1, hi = n;  // first position whose value exceeds v
        while (lo < hi) {
            const int64_t mid = (lo + hi) >> 1;
            if (static_cast<long long>(index[perm != nullptr ? perm[mid] : mid]) <= v) {
                lo = mid + 1;
            } else {
                hi = mid;
            }
        }
        best = (lo - i) > best ? (lo - i) : best;
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
        const long long other = __shfl_xor_sync(0xffffffffu, best, offset);
        best = other > best ? other : best;
    }
    if ((threadIdx.x & 31) == 0 && best > 0) {
        atomicMax(reinterpret_cast<long long*>(longest), best);
    }
}

// ---- SpMM edge-value gradient --------------------------------------------------------------------------------------------
// One warp per edge: lanes stride over the features (coalesced reads of the dense row and the gradient row), a shuffle
// tree finishes the dot product.  With one weight per feature the lanes write their products directly.
template <class T>
__global__ void __launch_bounds__(kThreads) ValueGradKernel(const int64_t* __restrict__ ptr, const int64_t* __restrict__ col,
                                                             const T* __restrict__ mat, const float* __restrict__ grad,
                                                             float* __restrict__ out, int64_t rows, int64_t src_rows,
                                                             int64_t feat, int64_t nnz, int64_t batches, int64_t width,
                                                             int mean)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (kThreads / 32);
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5); e < nnz; e += warps) {
        // row r with ptr[r] <= e < ptr[r+1]
        int64_t lo = 0, hi = rows;
        while (lo < hi) {
            const int64_t mid = (lo + hi) >> 1;
            if (ptr[mid + 1] <= e) {
                lo = mid + 1;
            } else {
                hi = mid;
            }
        }
        const int64_t row = lo < rows ? lo : rows - 1;
        int64_t c = col[e];
        c = c < 0 ? 0 : (c >= src_rows ? src_rows - 1 : c);
        float scale = 1.0f;
        if (mean) {
            const int64_t degree = ptr[row + 1] - ptr[row];
            if (degree > 0) {
                scale = static_cast<float>(degree);
            }
        }
        if (width == 1) {
            float acc = 0.0f;
            for (int64_t b = 0; b < batches; ++b) {
                const T* m = mat + (b * src_rows + c) * feat;
                const float* g = grad + (b * rows + row) * feat;
                for (int64_t k = lane; k < feat; k += 32) {
                    acc += Widen<float, T>(m[k]) * g[k];
                }
            }
            for (int offset = 16; offset > 0; offset >>= 1) {
                acc += __shfl_xor_sync(0xffffffffu, acc, offset);
            }
            if (lane == 0) {
                out[e] = mean ? acc / scale : acc;
            }
        } else {
            for (int64_t k = lane; k < feat; k += 32) {
                float acc = 0.0f;
                for (int64_t b = 0; b < batches; ++b) {
                    acc += Widen<float, T>(mat[(b * src_rows + c) * feat + k]) * grad[(b * rows + row) * feat + k];
                }
                out[e * feat + k] = mean ? acc / scale : acc;
            }
        }
    }
}

}  // namespace support
}  // namespace opsgnn

using namespace opsgnn;
using namespace opsgnn::support;

extern "C" int opsgnn_ind2ptr(const int64_t* ind, int64_t nnz, int64_t* ptr, int64_t rows, void* stream)
{
    if (ptr == nullptr || rows < 0 || nnz < 0 || (nnz > 0 && ind == nullptr)) {
        return OPSGNN_ERR_INVALID;
    }
    Ind2PtrKernel<<<StreamGrid(nnz + 1), kThreads, 0, AsStream(stream)>>>(ind, nnz, ptr, rows);
    return LaunchStatus();
}

extern "C" int opsgnn_ptr2ind(const int64_t* ptr, int64_t rows, int64_t* ind, int64_t nnz, void* stream)
{
    if (ptr == nullptr || rows < 0 || nnz < 0 || (nnz > 0 && (ind == nullptr || rows == 0))) {
        return OPSGNN_ERR_INVALID;
    }
    if (nnz == 0) {
        return OPSGNN_OK;
    }
    const int64_t blocks = CeilDiv(nnz, kEdgesPerBlock);
    if (blocks > 2147483647LL) {
        return OPSGNN_ERR_LIMIT;
    }
    Ptr2IndKernel<<<static_cast<unsigned>(blocks), kThreads, 0, AsStream(stream)>>>(ptr, rows, ind, nnz);
    return LaunchStatus();
}

extern "C" int opsgnn_csr_validate(const void* ptr, const void* col, int index_type, int64_t rows, int64_t cols,
                                   int64_t nnz, int32_t* status, void* stream)
{
    if (ptr == nullptr || status == nullptr || rows < 0 || nnz < 0 || cols < 0) {
        return OPSGNN_ERR_INVALID;
    }
    cudaStream_t s = AsStream(stream);
    OPSGNN_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int32_t), s));
    const unsigned grid = StreamGrid((rows + 1 > nnz ? rows + 1 : nnz), 4);
    if (index_type == OPSGNN_I64) {
        ValidateKernel<int64_t><<<grid, kThreads, 0, s>>>(static_cast<const int64_t*>(ptr),
                                                         static_cast<const int64_t*>(col), rows, cols, nnz, status);
    } else if (index_type == OPSGNN_I32) {
        ValidateKernel<int32_t><<<grid, kThreads, 0, s>>>(static_cast<const int32_t*>(ptr),
                                                         static_cast<const int32_t*>(col), rows, cols, nnz, status);
    } else {
        return OPSGNN_ERR_UNSUPPORTED;
    }
    return LaunchStatus();
}

extern "C" int opsgnn_permute_values(const int64_t* perm, const void* value, void* out, int64_t rows, int64_t width,
                                     int elem_bytes, void* stream)
{
    if (rows < 0 || width < 0) {
        return OPSGNN_ERR_INVALID;
    }
    if (rows == 0 || width == 0) {
        return OPSGNN_OK;
    }
    if (perm == nullptr || value == nullptr || out == nullptr) {
        return OPSGNN_ERR_INVALID;
    }
    const unsigned grid = StreamGrid(rows * width);
    cudaStream_t s = AsStream(stream);
    switch (elem_bytes) {
        case 1:
            PermuteKernel<uint8_t><<<grid, kThreads, 0, s>>>(perm, static_cast<const uint8_t*>(value),
                                                            static_cast<uint8_t*>(out), rows, width);
            break;
        case 2:
            PermuteKernel<uint16_t><<<grid, kThreads, 0, s>>>(perm, static_cast<const uint16_t*>(value),
                                                             static_cast<uint16_t*>(out), rows, width);
            break;
        case 4:
            PermuteKernel<uint32_t><<<grid, kThreads, 0, s>>>(perm, static_cast<const uint32_t*>(value),
                                                             static_cast<uint32_t*>(out), rows, width);
            break;
        case 8:
            PermuteKernel<uint64_t><<<grid, kThreads, 0, s>>>(perm, static_cast<const uint64_t*>(value),
                                                             static_cast<uint64_t*>(out), rows, width);
            break;
        default:
            return OPSGNN_ERR_UNSUPPORTED;
    }
    return LaunchStatus();
}

extern "C" int opsgnn_index_stats(const void* index, int index_type, int64_t n, int64_t* stats, void* stream)
{
    if (stats == nullptr || n < 0 || (n > 0 && index == nullptr)) {
        return OPSGNN_ERR_INVALID;
    }
    cudaStream_t s = AsStream(stream);
    StatsInitKernel<<<1, 1, 0, s>>>(stats);
    if (n > 0) {
        const unsigned grid = StreamGrid(n, 4);
        if (index_type == OPSGNN_I64) {
            StatsKernel<int64_t><<<grid, kThreads, 0, s>>>(static_cast<const int64_t*>(index), n, stats);
        } else if (index_type == OPSGNN_I32) {
            StatsKernel<int32_t><<<grid, kThreads, 0, s>>>(static_cast<const int32_t*>(index), n, stats);
        } else {
            return OPSGNN_ERR_UNSUPPORTED;
        }
    }
    return LaunchStatus();
}

extern "C" int opsgnn_index_longest_run(const void* index, int index_type, const int64_t* perm, int64_t n, int64_t* longest,
                                        void* stream)
{
    if (longest == nullptr || n < 0 || (n > 0 && index == nullptr)) {
        return OPSGNN_ERR_INVALID;
    }
    cudaStream_t s = AsStream(stream);
    OPSGNN_CUDA_TRY(cudaMemsetAsync(longest, 0, sizeof(int64_t), s));
    if (n > 0) {
        const unsigned grid = StreamGrid(n, 4);
        if (index_type == OPSGNN_I64) {
            LongestRunKernel<int64_t><<<grid, kThreads, 0, s>>>(static_cast<const int64_t*>(index), perm, n, longest);
        } else if (index_type == OPSGNN_I32) {
            LongestRunKernel<int32_t><<<grid, kThreads, 0, s>>>(static_cast<const int32_t*>(index), perm, n, longest);
        } else {
            return OPSGNN_ERR_UNSUPPORTED;
        }
    }
    return LaunchStatus();
}

extern "C" int opsgnn_spmm_value_grad(const int64_t* ptr, const int64_t* col, const void* mat, int mat_type,
                                      const float* grad, float* out, int64_t rows, int64_t src_rows, int64_t feat,
                                      int64_t nnz, int64_t batches, int64_t width, int mean, void* stream)
{
    if (rows < 0 || src_rows < 0 || feat < 0 || nnz < 0 || batches < 1 || (width != 1 && width != feat)) {
        return OPSGNN_ERR_INVALID;
    }
    if (nnz == 0) {
        return OPSGNN_OK;
    }
    if (ptr == nullptr || col == nullptr || mat == nullptr || grad == nullptr || out == nullptr || rows == 0 ||
        src_rows == 0) {
        return OPSGNN_ERR_INVALID;
    }
    const unsigned grid = StreamGrid(nnz * 32);
    cudaStream_t s = AsStream(stream);
    switch (mat_type) {
        case OPSGNN_F32:
            ValueGradKernel<float><<<grid, kThreads, 0, s>>>(ptr, col, static_cast<const float*>(mat), grad, out, rows,
                                                            src_rows, feat, nnz, batches, width, mean);
            break;
        case OPSGNN_F16:
            ValueGradKernel<__half><<<grid, kThreads, 0, s>>>(ptr, col, static_cast<const __half*>(mat), grad, out, rows,
                                                             src_rows, feat, nnz, batches, width, mean);
            break;
        case OPSGNN_BF16:
            ValueGradKernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(ptr, col, static_cast<const __nv_bfloat16*>(mat),
                                                                    grad, out, rows, src_rows, feat, nnz, batches, width,
                                                                    mean);
            break;
        default:
            return OPSGNN_ERR_UNSUPPORTED;
    }
    return LaunchStatus();
}
