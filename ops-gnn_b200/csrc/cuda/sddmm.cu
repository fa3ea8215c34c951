// SDDMM on CSR for sm_100a: out[e] = op(lhs[target_l(e)], rhs[target_r(e)]) for every edge e.
//
// Work is split by edges, never by rows: a thread block owns kEdgesPerCta consecutive edges, so power-law rows cost
// what their edges cost.  The row of an edge is found by a short binary search between the rows of the block's first
// and last edge (those two come from a per-call plan with one search per block).  Inside a warp, a group of G lanes
// (G = features / vector width, at most 32) owns one edge at a time and reads both operand rows with 16-byte loads:
// a 64-float row is one 256-byte request of 16 lanes, and two edges are in flight per warp instruction.  `dot`
// finishes with a shuffle tree inside the group and the warp writes its 64 results as two coalesced stores; the
// elementwise ops stream their [nnz, F] result rows with 16-byte stores.  Operand rows selected by the CSR row are
// re-read from L1 across the row's edges; rows selected by the column are the HBM-bound gather.
//
// Algorithmic bytes per launch (dot): nnz*(sizeof(index) + F*sizeof(T) + sizeof(T)) + rows*(sizeof(index) + F*sizeof(T)).
#include <utility>

#include <atomic>

#include "common.cuh"

namespace opsgnn {
namespace sddmm {

constexpr int kThreads = 256;
#ifndef OPSGNN_SDDMM_DOT_MAX_VECTORS
#define OPSGNN_SDDMM_DOT_MAX_VECTORS 4  // 16-byte vectors of each operand row a lane may own in the dot kernel
#endif
constexpr int kWarps = kThreads / 32;
constexpr int kEdgesPerWarp = 64;
constexpr int kEdgesPerCta = kWarps * kEdgesPerWarp;

struct Params {
    const void* indptr;
    const void* indices;
    const void* lhs;
    const void* rhs;
    void* out;
    int64_t* plan;  // row of the first edge of every block, num_cta + 1 entries
    int64_t rows;
    int64_t nnz;
    int64_t feat;
    int64_t lhs_rows;  // clamp bound of the lhs gather
    int64_t rhs_rows;
    int64_t num_cta;
    int op;
    int lhs_target;
    int rhs_target;
    int group;  // lanes per edge
};

// Row r with ptr[r] <= edge < ptr[r+1], searched in [lo, hi].
template <class IndexT>
__device__ __forceinline__ int64_t RowOf(const IndexT* __restrict__ ptr, int64_t lo, int64_t hi, int64_t edge)
{
    while (lo < hi) {
        const int64_t mid = (lo + hi + 1) >> 1;
        if (static_cast<int64_t>(ptr[mid]) <= edge) {
            lo = mid;
        } else {
            hi = mid - 1;
        }
    }
    return lo;
}

template <class IndexT>
__global__ void PlanKernel(const IndexT* __restrict__ ptr, int64_t rows, int64_t nnz, int64_t num_cta,
                           int64_t* __restrict__ plan)
{
    const int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (c > num_cta) {
        return;
    }
    int64_t edge = c * kEdgesPerCta;
    edge = edge < nnz ? edge : (nnz > 0 ? nnz - 1 : 0);
    plan[c] = rows > 0 ? RowOf(ptr, 0, rows - 1, edge) : 0;
}

__device__ __forceinline__ float Combine(int op, float a, float b)
{
    switch (op) {
        case OPSGNN_SDDMM_ADD:
            return a + b;
        case OPSGNN_SDDMM_SUB:
            return a - b;
        case OPSGNN_SDDMM_MUL:
            return a * b;
        case OPSGNN_SDDMM_DIV:
            return a / b;
        case OPSGNN_SDDMM_COPY_LHS:
            return a;
        default:
            return b;
    }
}

template <class T, class IndexT, int VEC, bool DOT>
__global__ void __launch_bounds__(kThreads) SddmmKernel(const Params p)
{
    constexpr int kUnroll = 4;
    __shared__ int64_t s_lhs[kEdgesPerCta];  // operand row offsets (row index * feat)
    __shared__ int64_t s_rhs[kEdgesPerCta];
    __shared__ float s_dot[DOT ? kEdgesPerCta : 1];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int64_t cta = blockIdx.x;
    const int64_t e0 = cta * kEdgesPerCta;
    const int count = static_cast<int>((p.nnz - e0 < kEdgesPerCta) ? p.nnz - e0 : kEdgesPerCta);
    const IndexT* __restrict__ ptr = static_cast<const IndexT*>(p.indptr);
    const IndexT* __restrict__ col = static_cast<const IndexT*>(p.indices);
    const T* __restrict__ lhs = static_cast<const T*>(p.lhs);
    const T* __restrict__ rhs = static_cast<const T*>(p.rhs);
    const int64_t F = p.feat;
    const bool use_lhs = p.op != OPSGNN_SDDMM_COPY_RHS;
    const bool use_rhs = p.op != OPSGNN_SDDMM_COPY_LHS;
    const bool need_row = (use_lhs && p.lhs_target == OPSGNN_TARGET_ROW) || (use_rhs && p.rhs_target == OPSGNN_TARGET_ROW);
    const bool need_col = (use_lhs && p.lhs_target == OPSGNN_TARGET_COL) || (use_rhs && p.rhs_target == OPSGNN_TARGET_COL);

    // ---- operand row of every edge of the block ------------------------------------------------------------------
    const int64_t row_lo = need_row ? p.plan[cta] : 0;
    const int64_t row_hi = need_row ? p.plan[cta + 1] : 0;
    for (int j = tid; j < count; j += kThreads) {
        const int64_t e = e0 + j;
        const int64_t r = need_row ? RowOf(ptr, row_lo, row_hi, e) : 0;
        const int64_t c = need_col ? static_cast<int64_t>(LoadStream(col + e)) : 0;
        auto pick = [&](int target, int64_t bound) {
            int64_t v = target == OPSGNN_TARGET_ROW ? r : (target == OPSGNN_TARGET_EDGE ? e : c);
            v = v < 0 ? 0 : (v >= bound ? bound - 1 : v);  // validated upstream; never fault on a bad index
            return v * F;
        };
        s_lhs[j] = use_lhs ? pick(p.lhs_target, p.lhs_rows) : 0;
        s_rhs[j] = use_rhs ? pick(p.rhs_target, p.rhs_rows) : 0;
    }
    __syncthreads();

    // ---- groups of G lanes walk the warp's edges ---------------------------------------------------------------------
    const int G = p.group;
    const int groups = 32 / G;
    const int g = lane / G;
    const int gl = lane - g * G;
    const int w0 = warp * kEdgesPerWarp;
    const int per_group = kEdgesPerWarp / groups;  // consecutive edges per group keep the row operand hot in L1
    T* __restrict__ out = static_cast<T*>(p.out);

    for (int t0 = 0; t0 < per_group; t0 += kUnroll) {
        float partial[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            partial[u] = 0.0f;
        }
        for (int64_t f = static_cast<int64_t>(gl) * VEC; f < F; f += static_cast<int64_t>(G) * VEC) {
            Pack<T, VEC> a[kUnroll], b[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int j = w0 + g * per_group + t0 + u;
                if (t0 + u < per_group && j < count) {
                    if (use_lhs) {
                        a[u] = LoadGather<T, VEC>(lhs + s_lhs[j] + f);
                    }
                    if (use_rhs) {
                        b[u] = LoadGather<T, VEC>(rhs + s_rhs[j] + f);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int j = w0 + g * per_group + t0 + u;
                if (t0 + u < per_group && j < count) {
                    float fa[VEC], fb[VEC];
                    if (use_lhs) {
                        Unpack<float, T, VEC>(a[u], fa);
                    }
                    if (use_rhs) {
                        Unpack<float, T, VEC>(b[u], fb);
                    }
                    if constexpr (DOT) {
#pragma unroll
                        for (int i = 0; i < VEC; ++i) {
                            partial[u] += fa[i] * fb[i];
                        }
                    } else {
                        float combined[VEC];
#pragma unroll
                        for (int i = 0; i < VEC; ++i) {
                            combined[i] = Combine(p.op, use_lhs ? fa[i] : 0.0f, use_rhs ? fb[i] : 0.0f);
                        }
                        StoreStream<T, VEC>(out + (e0 + j) * F + f, Repack<T, float, VEC>(combined));
                    }
                }
            }
        }
        if constexpr (DOT) {
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                float v = partial[u];
                for (int offset = G >> 1; offset > 0; offset >>= 1) {
                    v += __shfl_xor_sync(0xffffffffu, v, offset, 32);  // offsets below G stay inside the group
                }
                const int j = w0 + g * per_group + t0 + u;
                if (gl == 0 && t0 + u < per_group && j < count) {
                    s_dot[j] = v;
                }
            }
        }
    }
    if constexpr (DOT) {
        __syncwarp();
        for (int j = w0 + lane; j < w0 + kEdgesPerWarp && j < count; j += 32) {
            out[e0 + j] = Narrow<T, float>(s_dot[j]);
        }
    }
}

// ---- dot product, the hot SDDMM form ---------------------------------------------------------------------------------
// `lpe` lanes share an edge and every lane owns NVL 16-byte vectors of both operand rows, so a 64-float row is four
// lanes x four vectors: eight edges per warp instruction and two shuffle steps per dot instead of four.  Each lane
// group walks consecutive edges, and the operand selected by `lhs` is kept in registers until its row id changes:
// with lhs gathered by the CSR row (the caller swaps the operands when only rhs is) it is loaded once per row, not
// once per edge.  Row ids are staged as 32-bit numbers; addresses are one 32 x 32 -> 64 multiply-add.
template <class T, class IndexT, int VEC, int NVL>
__global__ void __launch_bounds__(kThreads, NVL == 4 ? 4 : 6) SddmmDotKernel(const Params p)
{
    __shared__ int s_a[kEdgesPerCta];
    __shared__ int s_b[kEdgesPerCta];
    __shared__ float s_dot[kEdgesPerCta];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int64_t cta = blockIdx.x;
    const int64_t e0 = cta * kEdgesPerCta;
    const int count = static_cast<int>((p.nnz - e0 < kEdgesPerCta) ? p.nnz - e0 : kEdgesPerCta);
    const IndexT* __restrict__ ptr = static_cast<const IndexT*>(p.indptr);
    const IndexT* __restrict__ col = static_cast<const IndexT*>(p.indices);
    const int F32 = static_cast<int>(p.feat);
    const bool need_row = p.lhs_target == OPSGNN_TARGET_ROW || p.rhs_target == OPSGNN_TARGET_ROW;
    const bool need_col = p.lhs_target == OPSGNN_TARGET_COL || p.rhs_target == OPSGNN_TARGET_COL;

    const int64_t row_lo = need_row ? p.plan[cta] : 0;
    const int64_t row_hi = need_row ? p.plan[cta + 1] : 0;
    for (int j = tid; j < count; j += kThreads) {
        const int64_t e = e0 + j;
        const int64_t r = need_row ? RowOf(ptr, row_lo, row_hi, e) : 0;
        const int64_t c = need_col ? static_cast<int64_t>(LoadStream(col + e)) : 0;
        auto pick = [&](int target, int64_t bound) {
            int64_t v = target == OPSGNN_TARGET_ROW ? r : (target == OPSGNN_TARGET_EDGE ? e : c);
            v = v < 0 ? 0 : (v >= bound ? bound - 1 : v);  // validated upstream; never fault on a bad index
            return static_cast<int>(v);                   // operand rows stay below 2^31 (checked by the launcher)
        };
        s_a[j] = pick(p.lhs_target, p.lhs_rows);
        s_b[j] = pick(p.rhs_target, p.rhs_rows);
    }
    __syncthreads();

    const int lpe = p.group;
    const int groups = 32 / lpe;
    const int g = lane / lpe;
    const int gl = lane - g * lpe;
    const int per_group = kEdgesPerWarp / groups;
    const int first = warp * kEdgesPerWarp + g * per_group;
    const T* __restrict__ a_base = static_cast<const T*>(p.lhs) + gl * VEC;
    const T* __restrict__ b_base = static_cast<const T*>(p.rhs) + gl * VEC;
    const int step = lpe * VEC;  // elements between a lane's consecutive vectors

    float fa[NVL][VEC];
    int held = -1;  // row id whose lhs fragment sits in fa
    auto hold = [&](int id) {
        if (id != held) {
            const T* row = a_base + static_cast<int64_t>(id) * F32;
#pragma unroll
            for (int k = 0; k < NVL; ++k) {
                Unpack<float, T, VEC>(LoadGather<T, VEC>(row + k * step), fa[k]);
            }
            held = id;
        }
    };
    auto dot = [&](const Pack<T, VEC> (&b)[NVL]) {
        float sum = 0.0f;
#pragma unroll
        for (int k = 0; k < NVL; ++k) {
            float fb[VEC];
            Unpack<float, T, VEC>(b[k], fb);
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                sum += fa[k][i] * fb[i];
            }
        }
        return sum;
    };

    for (int t = 0; t < per_group; t += 2) {
        const int j0 = first + t;
        const int j1 = j0 + 1;
        const bool live0 = j0 < count;
        const bool live1 = t + 1 < per_group && j1 < count;
        Pack<T, VEC> b0[NVL], b1[NVL];
        if (live0) {
            const T* row = b_base + static_cast<int64_t>(s_b[j0]) * F32;
#pragma unroll
            for (int k = 0; k < NVL; ++k) {
                b0[k] = LoadGather<T, VEC>(row + k * step);
            }
        }
        if (live1) {
            const T* row = b_base + static_cast<int64_t>(s_b[j1]) * F32;
#pragma unroll
            for (int k = 0; k < NVL; ++k) {
                b1[k] = LoadGather<T, VEC>(row + k * step);
            }
        }
        float d0 = 0.0f, d1 = 0.0f;
        if (live0) {
            hold(s_a[j0]);
            d0 = dot(b0);
        }
        if (live1) {
            hold(s_a[j1]);
            d1 = dot(b1);
        }
        for (int offset = lpe >> 1; offset > 0; offset >>= 1) {  // offsets below lpe stay inside the lane group
            d0 += __shfl_xor_sync(0xffffffffu, d0, offset, 32);
            d1 += __shfl_xor_sync(0xffffffffu, d1, offset, 32);
        }
        if (gl == 0) {
            if (live0) {
                s_dot[j0] = d0;
            }
            if (live1) {
                s_dot[j1] = d1;
            }
        }
    }
    __syncwarp();
    T* __restrict__ out = static_cast<T*>(p.out);
    const int w0 = warp * kEdgesPerWarp;
    for (int j = w0 + lane; j < w0 + kEdgesPerWarp && j < count; j += 32) {
        out[e0 + j] = Narrow<T, float>(s_dot[j]);
    }
}

// Vectors per lane for the dot kernel: the widest of 4 / 2 / 1 (at most 16 elements of fp32, 16 of a 16-bit type per
// operand) that leaves a power-of-two number of lanes per edge, at most 32; 0 when the width does not fit.
template <class T> inline int DotVectorsPerLane(int64_t feat)
{
    constexpr int kVec = 16 / sizeof(T);
    if (feat % kVec != 0) {
        return 0;
    }
    const int64_t vectors = feat / kVec;
    for (int nvl = (sizeof(T) == 4 && OPSGNN_SDDMM_DOT_MAX_VECTORS >= 4) ? 4 : 2; nvl >= 1; nvl >>= 1) {
        if (vectors % nvl == 0) {
            const int64_t lanes = vectors / nvl;
            if (lanes <= 32 && (lanes & (lanes - 1)) == 0) {
                return nvl;
            }
        }
    }
    return 0;
}

template <class T, class IndexT, int VEC> int LaunchTyped(const Params& p, cudaStream_t stream)
{
    const unsigned grid = static_cast<unsigned>(p.num_cta);
    if (p.op == OPSGNN_SDDMM_DOT) {
        SddmmKernel<T, IndexT, VEC, true><<<grid, kThreads, 0, stream>>>(p);
    } else {
        SddmmKernel<T, IndexT, VEC, false><<<grid, kThreads, 0, stream>>>(p);
    }
    return LaunchStatus();
}

template <class T, class IndexT> int LaunchVec(Params p, cudaStream_t stream)
{
    constexpr int kVec = 16 / sizeof(T);
    const bool vector_ok = p.feat % kVec == 0 && (p.lhs == nullptr || Aligned(p.lhs, 16)) &&
                           (p.rhs == nullptr || Aligned(p.rhs, 16)) && (p.op == OPSGNN_SDDMM_DOT || Aligned(p.out, 16));
    if (vector_ok && p.op == OPSGNN_SDDMM_DOT && p.lhs_rows <= 2147483647LL && p.rhs_rows <= 2147483647LL &&
        p.feat <= 2147483647LL) {
        const int nvl = DotVectorsPerLane<T>(p.feat);
        if (nvl > 0) {
            if (p.lhs_target != OPSGNN_TARGET_ROW && p.rhs_target == OPSGNN_TARGET_ROW) {
                // a dot product commutes: keep the operand gathered by the CSR row in the cached position
                std::swap(p.lhs, p.rhs);
                std::swap(p.lhs_rows, p.rhs_rows);
                std::swap(p.lhs_target, p.rhs_target);
            }
            p.group = static_cast<int>(p.feat / kVec / nvl);
            const unsigned grid = static_cast<unsigned>(p.num_cta);
            if (nvl == 4) {
                SddmmDotKernel<T, IndexT, kVec, 4><<<grid, kThreads, 0, stream>>>(p);
            } else if (nvl == 2) {
                SddmmDotKernel<T, IndexT, kVec, 2><<<grid, kThreads, 0, stream>>>(p);
            } else {
                SddmmDotKernel<T, IndexT, kVec, 1><<<grid, kThreads, 0, stream>>>(p);
            }
            return LaunchStatus();
        }
    }
    const int vec = vector_ok ? kVec : 1;
    int group = 1;
    while (group < 32 && static_cast<int64_t>(group) * vec < p.feat) {
        group <<= 1;
    }
    p.group = group;
    if (vector_ok) {
        return LaunchTyped<T, IndexT, kVec>(p, stream);
    }
    return LaunchTyped<T, IndexT, 1>(p, stream);
}

template <class IndexT> int LaunchIndexed(const Params& p, int dtype, cudaStream_t stream)
{
    switch (dtype) {
        case OPSGNN_F32:
            return LaunchVec<float, IndexT>(p, stream);
        case OPSGNN_F16:
            return LaunchVec<__half, IndexT>(p, stream);
        case OPSGNN_BF16:
            return LaunchVec<__nv_bfloat16, IndexT>(p, stream);
        default:
            return OPSGNN_ERR_UNSUPPORTED;
    }
}

}  // namespace sddmm
}  // namespace opsgnn

using namespace opsgnn;
using namespace opsgnn::sddmm;

extern "C" int opsgnn_sddmm_workspace_bytes(const OpsgnnSddmmDesc* desc, int64_t* bytes)
{
    if (desc == nullptr || bytes == nullptr || desc->nnz < 0) {
        return OPSGNN_ERR_INVALID;
    }
    *bytes = (CeilDiv(desc->nnz, kEdgesPerCta) + 1) * static_cast<int64_t>(sizeof(int64_t));
    return OPSGNN_OK;
}

extern "C" int opsgnn_sddmm_csr(const OpsgnnSddmmDesc* desc, const void* indptr, const void* indices, const void* lhs,
                                const void* rhs, void* out, void* workspace, int64_t workspace_bytes, void* stream)
{
    if (desc == nullptr || desc->rows < 0 || desc->nnz < 0 || desc->feat < 1) {
        return OPSGNN_ERR_INVALID;
    }
    const OpsgnnSddmmDesc& d = *desc;
    if (d.op < OPSGNN_SDDMM_DOT || d.op > OPSGNN_SDDMM_COPY_RHS || d.lhs_target < 0 || d.lhs_target > 2 ||
        d.rhs_target < 0 || d.rhs_target > 2 || (d.index_type != OPSGNN_I32 && d.index_type != OPSGNN_I64)) {
        return OPSGNN_ERR_INVALID;
    }
    if (d.nnz == 0) {
        return OPSGNN_OK;
    }
    const bool use_lhs = d.op != OPSGNN_SDDMM_COPY_RHS;
    const bool use_rhs = d.op != OPSGNN_SDDMM_COPY_LHS;
    if (indptr == nullptr || indices == nullptr || out == nullptr || (use_lhs && lhs == nullptr) ||
        (use_rhs && rhs == nullptr) || (use_lhs && d.lhs_rows < 1) || (use_rhs && d.rhs_rows < 1) || d.rows < 1) {
        return OPSGNN_ERR_INVALID;
    }
    int64_t needed = 0;
    opsgnn_sddmm_workspace_bytes(desc, &needed);
    if (workspace == nullptr || workspace_bytes < needed || !Aligned(workspace, 8)) {
        return OPSGNN_ERR_WORKSPACE;
    }
    Params p{};
    p.indptr = indptr;
    p.indices = indices;
    p.lhs = use_lhs ? lhs : nullptr;
    p.rhs = use_rhs ? rhs : nullptr;
    p.out = out;
    p.plan = static_cast<int64_t*>(workspace);
    p.rows = d.rows;
    p.nnz = d.nnz;
    p.feat = d.feat;
    p.lhs_rows = d.lhs_rows;
    p.rhs_rows = d.rhs_rows;
    p.num_cta = CeilDiv(d.nnz, kEdgesPerCta);
    p.op = d.op;
    p.lhs_target = d.lhs_target;
    p.rhs_target = d.rhs_target;
    if (p.num_cta > 2147483647LL) {
        return OPSGNN_ERR_LIMIT;
    }
    cudaStream_t s = AsStream(stream);
    const unsigned plan_grid = static_cast<unsigned>(CeilDiv(p.num_cta + 1, 256));
    if (d.index_type == OPSGNN_I64) {
        PlanKernel<int64_t><<<plan_grid, 256, 0, s>>>(static_cast<const int64_t*>(indptr), d.rows, d.nnz, p.num_cta, p.plan);
    } else {
        PlanKernel<int32_t><<<plan_grid, 256, 0, s>>>(static_cast<const int32_t*>(indptr), d.rows, d.nnz, p.num_cta, p.plan);
    }
    int status = LaunchStatus();
    if (status != OPSGNN_OK) {
        return status;
    }
    return d.index_type == OPSGNN_I64 ? LaunchIndexed<int64_t>(p, d.dtype, s) : LaunchIndexed<int32_t>(p, d.dtype, s);
}

// ---- variant for callers that cannot allocate ---------------------------------------------------------------------------
// The per-block row plan lives in a fixed array inside this library instead of caller-provided scratch.  Every GPU
// that loads the library keeps these 256 KiB until the process exits.
#define OPSGNN_SDDMM_STATIC_MAX_EDGES (1LL << 24)
namespace {
constexpr int64_t kStaticPlanEntries = OPSGNN_SDDMM_STATIC_MAX_EDGES / opsgnn::sddmm::kEdgesPerCta + 1;
static __device__ __align__(256) int64_t g_static_plan[kStaticPlanEntries];
constexpr int kMaxDevices = 64;
// device address of g_static_plan, per device ordinal; atomic because first calls on one device may come from several host threads
std::atomic<void*> g_static_plan_address[kMaxDevices];
}  // namespace

extern "C" int opsgnn_sddmm_csr_static(const OpsgnnSddmmDesc* desc, const void* indptr, const void* indices,
                                       const void* lhs, const void* rhs, void* out, void* stream)
{
    if (desc == nullptr) {
        return OPSGNN_ERR_INVALID;
    }
    if (desc->nnz > OPSGNN_SDDMM_STATIC_MAX_EDGES) {
        return OPSGNN_ERR_LIMIT;  // more edges than the built-in plan array can describe
    }
    int device = -1;
    OPSGNN_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) {
        return OPSGNN_ERR_LIMIT;
    }
    void* plan_address = g_static_plan_address[device].load(std::memory_order_acquire);
    if (plan_address == nullptr) {
        // In host code `g_static_plan` names a host-side stand-in, not device memory: the address a kernel may use
        // has to be looked up, with the owning device current (it is: cudaGetDevice above).
        void* address = nullptr;
        OPSGNN_CUDA_TRY(cudaGetSymbolAddress(&address, g_static_plan));
        g_static_plan_address[device].store(address, std::memory_order_release);
        plan_address = address;
    }
    return opsgnn_sddmm_csr(desc, indptr, indices, lhs, rhs, out, plan_address,
                            kStaticPlanEntries * static_cast<int64_t>(sizeof(int64_t)), stream);
}
