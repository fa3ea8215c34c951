// Fused graph-attention aggregation (GAT layer) in two launches, with no [E, H] tensor ever written:
//
//   logit[e, h] = leaky_relu(left[row(e), h] + right[col(e), h])
//   lse[r, h]   = log sum_{e in row r} exp(logit[e, h])                                   (EdgeLogitLse + MergeBoundary)
//   out[r, h, :] = sum_{e in row r} exp(logit[e, h] - lse[r, h]) * x[col(e), h, :]        (weighted bulk instance of the
//                                                                                          CSR reduce engine, attention mode)
//
// The logits are written once by the first launch (E * H floats) and read once by the second, where they ride in the
// gather ring beside the rows they scale (one contiguous bulk copy per stage); the LeakyReLU output and the softmax
// weights are never in memory.  Gathering the column-side halves again inside the aggregation instead (one more bulk
// copy per EDGE) was measured: 10.7 ms against 9.1 ms for the aggregation alone on the 34.5M-edge graph.
//
// The reference composes this layer from four operators and materialises the logits, the softmax weights and, in its
// `spmm` fallback, the [E, H, D] messages (python/ops_gnn/spmm.py:148-208, 283-289 of the reference).  Here the first launch
// reads only the edge list and the [N, H] halves (40 bytes per edge against 2 KiB per edge for the aggregation), the second
// forms each weight from values that ride in the gather ring beside the row they scale.  Knowing the log-sum-exp before the
// aggregation keeps every partial sum a plain sum: rows that span warps and thread blocks go through the engine's ordinary
// carry path and the result is bitwise reproducible.
//
// EdgeLogitLse: the edge list is cut into chunks of kChunk consecutive edges; `heads` threads own a chunk (one head each)
// and walk it in order with an online (maximum, scaled sum) state.  Rows that begin and end inside a chunk are finished
// on the spot; the first and the last row of every chunk may continue in a neighbour, so their partial states go to a
// boundary array that MergeBoundary folds in chunk order (one thread per head and run of equal rows: deterministic).
// Algorithmic bytes: nnz * (row id + column id + H * 4) + rows * H * 8.
#include "csr_instances.h"

namespace opsgnn {
namespace attention {

constexpr int kThreads = 256;
constexpr int kChunk = 128;
constexpr int kStep = 8;  // edges whose loads are in flight together in one thread

struct LseParams {
    const void* edge_rows;
    const void* col;
    const float* left;
    const float* right;
    float* logits;        // [nnz, heads]: leaky_relu(left[row] + right[col]), written once for the aggregation to read
    float* lse;           // [rows, heads], pre-filled with -inf
    int64_t* long_runs;   // [0] = number of long runs, [1 + k] = boundary slot that opens the k-th one
    int64_t* bound_row;   // [chunks, 2]: row of the chunk's first / last partial, -1 when absent
    float* bound_state;   // [chunks, 2, heads, 2]: (maximum, sum)
    int64_t nnz, rows, src_rows, chunks;
    int heads, lanes;     // lanes = heads rounded up to a power of two
    float slope;
};

__device__ __forceinline__ void Offer(float& m, float& s, float x)
{
    if (x > m) {
        s = s * __expf(m - x) + 1.0f;  // m = -inf initially: 0 * 0 + 1
        m = x;
    } else {
        s += __expf(x == m ? 0.0f : x - m);
    }
}

template <class IndexT> __global__ void __launch_bounds__(kThreads, 4) EdgeLogitLseKernel(const LseParams p)
{
    const int64_t thread = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int64_t chunk = thread / p.lanes;
    const int head = static_cast<int>(thread - chunk * p.lanes);
    if (chunk >= p.chunks || head >= p.heads) {
        return;
    }
    const IndexT* __restrict__ edge_rows = static_cast<const IndexT*>(p.edge_rows);
    const IndexT* __restrict__ col = static_cast<const IndexT*>(p.col);
    const int64_t e0 = chunk * kChunk;
    const int64_t e1 = (e0 + kChunk < p.nnz) ? e0 + kChunk : p.nnz;
    const int64_t first_row = static_cast<int64_t>(__ldg(edge_rows + e0));
    int64_t row = first_row;
    float bias = (row >= 0 && row < p.rows) ? __ldg(p.left + row * p.heads + head) : 0.0f;
    float m = -INFINITY, s = 0.0f;
    bool first_done = false;
    float* state = p.bound_state + (chunk * 2) * p.heads * 2 + head * 2;
    for (int64_t base = e0; base < e1; base += kStep) {
        int r[kStep], c[kStep];  // rows and columns fit 31 bits (checked by the entry point)
        float v[kStep];
#pragma unroll
        for (int u = 0; u < kStep; ++u) {
            const int64_t e = base + u < e1 ? base + u : e1 - 1;
            const int64_t row_id = static_cast<int64_t>(__ldg(edge_rows + e));
            int64_t column = static_cast<int64_t>(__ldg(col + e));
            column = column < 0 ? 0 : (column >= p.src_rows ? p.src_rows - 1 : column);  // validated upstream; never fault
            r[u] = static_cast<int>(row_id < 0 ? -1 : (row_id >= p.rows ? p.rows : row_id));
            c[u] = static_cast<int>(column);
        }
#pragma unroll
        for (int u = 0; u < kStep; ++u) {
            v[u] = __ldg(p.right + static_cast<int64_t>(c[u]) * p.heads + head);
        }
#pragma unroll
        for (int u = 0; u < kStep; ++u) {
            if (base + u >= e1) {
                break;
            }
            if (r[u] != row) {  // the current row ends here
                if (!first_done) {
                    state[0] = m;  // first row of the chunk: may have begun in an earlier chunk
                    state[1] = s;
                    first_done = true;
                } else if (row >= 0 && row < p.rows) {
                    p.lse[row * p.heads + head] = s == 0.0f ? m : m + __logf(s);  // began and ended inside this chunk
                }
                row = r[u];
                bias = (row >= 0 && row < p.rows) ? __ldg(p.left + row * p.heads + head) : 0.0f;
                m = -INFINITY;
                s = 0.0f;
            }
            float logit = bias + v[u];
            logit = logit > 0.0f ? logit : logit * p.slope;
            p.logits[(base + u) * p.heads + head] = logit;  // the heads of an edge are adjacent: one 32-byte sector
            Offer(m, s, logit);
        }
    }
    // the last row of the chunk may continue in the next one; a chunk with a single row has only a first partial
    float* tail = state + p.heads * 2;
    if (!first_done) {
        state[0] = m;
        state[1] = s;
        tail[0] = -INFINITY;
        tail[1] = 0.0f;
    } else {
        tail[0] = m;
        tail[1] = s;
    }
    if (head == 0) {
        p.bound_row[chunk * 2] = first_row;
        p.bound_row[chunk * 2 + 1] = first_done ? row : -1;
    }
}

// The same sweep for 3 to 8 heads (LANES = 4 or 8 threads per chunk): the row and column ids of a trip of eight edges
// are loaded once per chunk - lane g of the chunk's group loads edge g - and handed round with group-wide shuffles
// instead of every head loading all of them, and the ids of the next trip are in flight while this one is processed.
// Lanes beyond the head count and groups beyond the last chunk run along (shuffles name the whole group) and write
// nothing.  The order in which a head sees its edges, and therefore every result, is that of the kernel above.
template <class IndexT, int LANES> __global__ void __launch_bounds__(kThreads, 4) EdgeLogitLseTeamKernel(const LseParams p)
{
    static_assert(LANES == 4 || LANES == 8, "a trip of eight edges is split over the group");
    constexpr int kTrip = 8;
    constexpr int kPer = kTrip / LANES;  // ids a lane loads per trip
    const int64_t thread = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int64_t chunk_of_thread = thread / LANES;
    const int head = static_cast<int>(thread - chunk_of_thread * LANES);
    const bool live = chunk_of_thread < p.chunks;
    const int64_t chunk = live ? chunk_of_thread : p.chunks - 1;  // an idle group shadows the last chunk
    const bool writes = live && head < p.heads;
    const int h = head < p.heads ? head : p.heads - 1;
    const int group_lane = (threadIdx.x & 31) & ~(LANES - 1);
    const unsigned group = ((LANES == 32 ? 0u : (1u << LANES)) - 1u) << group_lane;
    const IndexT* __restrict__ edge_rows = static_cast<const IndexT*>(p.edge_rows);
    const IndexT* __restrict__ col = static_cast<const IndexT*>(p.col);
    const int64_t e0 = chunk * kChunk;
    const int64_t e1 = (e0 + kChunk < p.nnz) ? e0 + kChunk : p.nnz;
    auto load_ids = [&](int64_t base, int (&rows_of)[kPer], int (&cols_of)[kPer]) {
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            int64_t e = base + head + k * LANES;
            e = e < e1 ? e : e1 - 1;
            const int64_t row_id = static_cast<int64_t>(__ldg(edge_rows + e));
            int64_t column = static_cast<int64_t>(__ldg(col + e));
            column = column < 0 ? 0 : (column >= p.src_rows ? p.src_rows - 1 : column);  // validated upstream; never fault
            rows_of[k] = static_cast<int>(row_id < 0 ? -1 : (row_id >= p.rows ? p.rows : row_id));
            cols_of[k] = static_cast<int>(column);
        }
    };
    int next_rows[kPer], next_cols[kPer];
    load_ids(e0, next_rows, next_cols);
    const int64_t first_id = static_cast<int64_t>(__ldg(edge_rows + e0));
    const int first_row = static_cast<int>(first_id < 0 ? -1 : (first_id >= p.rows ? p.rows : first_id));
    int row = first_row;
    float bias = (row >= 0 && row < p.rows) ? __ldg(p.left + static_cast<int64_t>(row) * p.heads + h) : 0.0f;
    float m = -INFINITY, s = 0.0f;
    bool first_done = false;
    float* state = p.bound_state + (chunk * 2) * p.heads * 2 + h * 2;
    for (int64_t base = e0; base < e1; base += kTrip) {
        int my_rows[kPer], my_cols[kPer];
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            my_rows[k] = next_rows[k];
            my_cols[k] = next_cols[k];
        }
        if (base + kTrip < e1) {
            load_ids(base + kTrip, next_rows, next_cols);
        }
        float v[kTrip];
#pragma unroll
        for (int u = 0; u < kTrip; ++u) {
            const int column = __shfl_sync(group, my_cols[u / LANES], group_lane + (u % LANES));
            v[u] = __ldg(p.right + static_cast<int64_t>(column) * p.heads + h);
        }
#pragma unroll
        for (int u = 0; u < kTrip; ++u) {
            const int r = __shfl_sync(group, my_rows[u / LANES], group_lane + (u % LANES));  // by every lane of the group
            if (base + u < e1) {
                if (r != row) {  // the current row ends here
                    if (!first_done) {
                        if (writes) {
                            state[0] = m;  // first row of the chunk: may have begun in an earlier chunk
                            state[1] = s;
                        }
                        first_done = true;
                    } else if (writes && row >= 0 && row < p.rows) {
                        p.lse[static_cast<int64_t>(row) * p.heads + h] = s == 0.0f ? m : m + __logf(s);
                    }
                    row = r;
                    bias = (row >= 0 && row < p.rows) ? __ldg(p.left + static_cast<int64_t>(row) * p.heads + h) : 0.0f;
                    m = -INFINITY;
                    s = 0.0f;
                }
                float logit = bias + v[u];
                logit = logit > 0.0f ? logit : logit * p.slope;
                if (writes) {
                    p.logits[(base + u) * p.heads + h] = logit;
                }
                Offer(m, s, logit);
            }
        }
    }
    if (!writes) {
        return;
    }
    float* tail = state + p.heads * 2;
    if (!first_done) {
        state[0] = m;
        state[1] = s;
        tail[0] = -INFINITY;
        tail[1] = 0.0f;
    } else {
        tail[0] = m;
        tail[1] = s;
    }
    if (head == 0) {
        p.bound_row[chunk * 2] = first_id;
        p.bound_row[chunk * 2 + 1] = first_done ? row : -1;
    }
}

// Eight heads, 16-byte aligned operands: two threads per chunk, four heads each, so that every gather, store and bias
// load moves 16 bytes per lane (a warp instruction covers 16 chunks x 32 bytes instead of 4) - the sweep is bound by
// the bytes it keeps in flight, and this quadruples them per instruction.  Ids are shared and prefetched as in the
// team kernel; the order in which a head sees its edges is unchanged.
// FROM_VALUES = true is the same sweep over given values instead of logits to be formed: `right` is then a [nnz, 8]
// matrix read in edge order (no columns, no bias, no activation, nothing written per edge) - the log-sum-exp per group
// of narrow rows under sorted labels.
template <class IndexT, bool FROM_VALUES = false>
__global__ void __launch_bounds__(kThreads, 3) EdgeLogitLseQuadKernel(const LseParams p)
{
    constexpr int kTrip = 8;
    constexpr int kGroup = 2;            // lanes per chunk
    constexpr int kPer = kTrip / kGroup;  // ids a lane loads per trip
    const int64_t thread = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int64_t chunk_of_thread = thread / kGroup;
    const int half = static_cast<int>(thread - chunk_of_thread * kGroup);
    const bool writes = chunk_of_thread < p.chunks;
    const int64_t chunk = writes ? chunk_of_thread : p.chunks - 1;  // an idle pair shadows the last chunk
    const int group_lane = (threadIdx.x & 31) & ~(kGroup - 1);
    const unsigned group = 3u << group_lane;
    const IndexT* __restrict__ edge_rows = static_cast<const IndexT*>(p.edge_rows);
    const IndexT* __restrict__ col = static_cast<const IndexT*>(p.col);
    const float4* __restrict__ left = reinterpret_cast<const float4*>(p.left);
    const float4* __restrict__ right = reinterpret_cast<const float4*>(p.right);
    float4* __restrict__ logits = reinterpret_cast<float4*>(p.logits);
    const int64_t e0 = chunk * kChunk;
    const int64_t e1 = (e0 + kChunk < p.nnz) ? e0 + kChunk : p.nnz;
    auto load_ids = [&](int64_t base, int (&rows_of)[kPer], int (&cols_of)[kPer]) {
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            int64_t e = base + half + k * kGroup;
            e = e < e1 ? e : e1 - 1;
            const int64_t row_id = static_cast<int64_t>(__ldg(edge_rows + e));
            int64_t column = 0;
            if constexpr (!FROM_VALUES) {
                column = static_cast<int64_t>(__ldg(col + e));
                column = column < 0 ? 0 : (column >= p.src_rows ? p.src_rows - 1 : column);  // validated upstream; never fault
            }
            rows_of[k] = static_cast<int>(row_id < 0 ? -1 : (row_id >= p.rows ? p.rows : row_id));
            cols_of[k] = static_cast<int>(column);
        }
    };
    auto finish = [](float m, float s) { return s == 0.0f ? m : m + __logf(s); };
    int next_rows[kPer], next_cols[kPer];
    load_ids(e0, next_rows, next_cols);
    const int64_t first_id = static_cast<int64_t>(__ldg(edge_rows + e0));
    int row = static_cast<int>(first_id < 0 ? -1 : (first_id >= p.rows ? p.rows : first_id));
    const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 bias = zero;
    if constexpr (!FROM_VALUES) {
        bias = (row >= 0 && row < p.rows) ? __ldg(left + static_cast<int64_t>(row) * 2 + half) : zero;
    }
    float m[4], s[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        m[q] = -INFINITY;
        s[q] = 0.0f;
    }
    bool first_done = false;
    float4* state = reinterpret_cast<float4*>(p.bound_state + (chunk * 2) * 16 + half * 8);  // [chunk][first/last][8 heads][2]
    for (int64_t base = e0; base < e1; base += kTrip) {
        int my_rows[kPer], my_cols[kPer];
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            my_rows[k] = next_rows[k];
            my_cols[k] = next_cols[k];
        }
        if (base + kTrip < e1) {
            load_ids(base + kTrip, next_rows, next_cols);
        }
        float4 v[kTrip];
#pragma unroll
        for (int u = 0; u < kTrip; ++u) {
            if constexpr (FROM_VALUES) {
                const int64_t e = base + u < e1 ? base + u : e1 - 1;
                v[u] = __ldg(right + e * 2 + half);
            } else {
                const int column = __shfl_sync(group, my_cols[u / kGroup], group_lane + (u % kGroup));
                v[u] = __ldg(right + static_cast<int64_t>(column) * 2 + half);
            }
        }
#pragma unroll
        for (int u = 0; u < kTrip; ++u) {
            const int r = __shfl_sync(group, my_rows[u / kGroup], group_lane + (u % kGroup));  // by both lanes of the pair
            if (base + u < e1) {
                if (r != row) {  // the current row ends here
                    if (!first_done) {
                        if (writes) {  // first row of the chunk: may have begun in an earlier chunk
                            state[0] = make_float4(m[0], s[0], m[1], s[1]);
                            state[1] = make_float4(m[2], s[2], m[3], s[3]);
                        }
                        first_done = true;
                    } else if (writes && row >= 0 && row < p.rows) {
                        reinterpret_cast<float4*>(p.lse)[static_cast<int64_t>(row) * 2 + half] =
                            make_float4(finish(m[0], s[0]), finish(m[1], s[1]), finish(m[2], s[2]), finish(m[3], s[3]));
                    }
                    row = r;
                    if constexpr (!FROM_VALUES) {
                        bias = (row >= 0 && row < p.rows) ? __ldg(left + static_cast<int64_t>(row) * 2 + half) : zero;
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        m[q] = -INFINITY;
                        s[q] = 0.0f;
                    }
                }
                float4 logit = v[u];
                if constexpr (!FROM_VALUES) {
                    logit = make_float4(bias.x + v[u].x, bias.y + v[u].y, bias.z + v[u].z, bias.w + v[u].w);
                    logit.x = logit.x > 0.0f ? logit.x : logit.x * p.slope;
                    logit.y = logit.y > 0.0f ? logit.y : logit.y * p.slope;
                    logit.z = logit.z > 0.0f ? logit.z : logit.z * p.slope;
                    logit.w = logit.w > 0.0f ? logit.w : logit.w * p.slope;
                    if (writes) {
                        logits[(base + u) * 2 + half] = logit;
                    }
                }
                Offer(m[0], s[0], logit.x);
                Offer(m[1], s[1], logit.y);
                Offer(m[2], s[2], logit.z);
                Offer(m[3], s[3], logit.w);
            }
        }
    }
    if (!writes) {
        return;
    }
    // the last row of the chunk may continue in the next one; a chunk with a single row has only a first partial
    float4* tail = state + 4;  // 8 heads x 2 floats further on
    if (!first_done) {
        state[0] = make_float4(m[0], s[0], m[1], s[1]);
        state[1] = make_float4(m[2], s[2], m[3], s[3]);
        tail[0] = make_float4(-INFINITY, 0.0f, -INFINITY, 0.0f);
        tail[1] = make_float4(-INFINITY, 0.0f, -INFINITY, 0.0f);
    } else {
        tail[0] = make_float4(m[0], s[0], m[1], s[1]);
        tail[1] = make_float4(m[2], s[2], m[3], s[3]);
    }
    if (half == 0) {
        p.bound_row[chunk * 2] = first_id;
        p.bound_row[chunk * 2 + 1] = first_done ? row : -1;
    }
}

// One thread per boundary slot: the slot that opens a run of equal rows folds the run in slot order, head by head.  A run
// longer than kShortRun slots (a hub row that spans hundreds of chunks) would make that one thread a serial chain of
// dependent loads, so its opener only records the slot; LongRunKernel folds those runs with a warp each.
constexpr int kShortRun = 4;
constexpr int kMaxLongRuns = 1 << 16;

__global__ void __launch_bounds__(kThreads) MergeBoundaryKernel(const LseParams p)
{
    const int64_t slot = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int64_t slots = p.chunks * 2;
    if (slot >= slots) {
        return;
    }
    const int64_t row = p.bound_row[slot];
    if (row < 0 || row >= p.rows) {
        return;
    }
    int64_t before = slot - 1;  // nearest earlier slot that holds a partial (at most two steps back)
    while (before >= 0 && p.bound_row[before] < 0) {
        --before;
    }
    if (before >= 0 && p.bound_row[before] == row) {
        return;  // not the opener of its run
    }
    // Rows are sorted, so the run is long when a slot that far ahead still carries the row.  Inside a run that spans whole
    // chunks only the chunks' first slots carry it (their last slots are absent), so both parities are looked at: an
    // opener in a last slot would otherwise walk a hub row's hundreds of chunks alone (measured: 0.29 ms for this kernel).
    const bool far = (slot + kShortRun < slots && p.bound_row[slot + kShortRun] == row) ||
                     (slot + kShortRun + 1 < slots && p.bound_row[slot + kShortRun + 1] == row);
    if (far) {
        const unsigned long long at = atomicAdd(reinterpret_cast<unsigned long long*>(p.long_runs), 1ULL);
        if (at < kMaxLongRuns) {
            p.long_runs[1 + at] = slot;
        }
        return;
    }
    int64_t last = slot;  // the run is [slot, last]; short, so its end is found first and the heads walk it afterwards
    for (int64_t next = slot + 1; next < slots; ++next) {
        const int64_t other = p.bound_row[next];
        if (other < 0) {
            continue;
        }
        if (other != row) {
            break;
        }
        last = next;
    }
    if (p.heads % 2 == 0) {  // two heads per 16-byte load: (max, sum, max, sum); the workspace is 256-byte aligned
        for (int head = 0; head < p.heads; head += 2) {
            float4 state = *reinterpret_cast<const float4*>(p.bound_state + (slot * p.heads + head) * 2);
            for (int64_t next = slot + 1; next <= last; ++next) {
                if (p.bound_row[next] == row) {
                    const float4 other = *reinterpret_cast<const float4*>(p.bound_state + (next * p.heads + head) * 2);
                    csr::LseMerge(state.x, state.y, other.x, other.y);
                    csr::LseMerge(state.z, state.w, other.z, other.w);
                }
            }
            p.lse[row * p.heads + head] = state.y == 0.0f ? state.x : state.x + __logf(state.y);
            p.lse[row * p.heads + head + 1] = state.w == 0.0f ? state.z : state.z + __logf(state.w);
        }
        return;
    }
    for (int head = 0; head < p.heads; ++head) {
        float m = p.bound_state[(slot * p.heads + head) * 2];
        float s = p.bound_state[(slot * p.heads + head) * 2 + 1];
        for (int64_t next = slot + 1; next <= last; ++next) {
            if (p.bound_row[next] == row) {
                csr::LseMerge(m, s, p.bound_state[(next * p.heads + head) * 2], p.bound_state[(next * p.heads + head) * 2 + 1]);
            }
        }
        p.lse[row * p.heads + head] = s == 0.0f ? m : m + __logf(s);
    }
}

// One warp per long run: the warp's 32 / lanes walkers (a walker = `lanes` lanes, one head each) take slots
// slot + w, slot + w + walkers, ...; their states are then folded by shuffles in walker order, so the result does not
// depend on scheduling.  The run's end is found once by a binary search over the chunks' first rows (rows are sorted).
__global__ void __launch_bounds__(kThreads) LongRunKernel(const LseParams p)
{
    const int64_t slots = p.chunks * 2;
    int64_t count = p.long_runs[0];
    count = count < kMaxLongRuns ? count : kMaxLongRuns;
    const int lane = threadIdx.x & 31;
    const int head = lane % p.lanes;
    const int walker = lane / p.lanes;
    const int walkers = 32 / p.lanes;
    const int64_t warp = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (kThreads / 32);
    for (int64_t k = warp; k < count; k += warps) {
        const int64_t slot = p.long_runs[1 + k];
        const int64_t row = p.bound_row[slot];
        // Inside a long run a chunk holds only this row: its first slot carries the row, its last slot is absent (-1).
        int64_t lo = (slot + 2) / 2, hi = p.chunks;  // first chunk whose first row exceeds `row`
        while (lo < hi) {
            const int64_t mid = (lo + hi) >> 1;
            if (p.bound_row[mid * 2] <= row) {
                lo = mid + 1;
            } else {
                hi = mid;
            }
        }
        const int64_t end = lo * 2 < slots ? lo * 2 : slots;  // slots [slot, end) may belong to the run
        float m = -INFINITY, s = 0.0f;
        if (head < p.heads) {
            // Eight slots per trip: their rows and states are loaded before any is merged (a hub row is a chain of
            // hundreds of slots per walker, and one load at a time made this kernel 0.2 ms), then merged in slot order.
            constexpr int kBatch = 8;
            for (int64_t base = slot + walker; base < end; base += static_cast<int64_t>(kBatch) * walkers) {
                int64_t owner[kBatch];
                float2 state[kBatch];
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    const int64_t next = base + static_cast<int64_t>(u) * walkers;
                    owner[u] = next < end ? p.bound_row[next] : -1;
                }
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    const int64_t next = base + static_cast<int64_t>(u) * walkers;
                    state[u] = make_float2(-INFINITY, 0.0f);
                    if (next < end) {  // every slot below `end` has a state cell, whoever owns it
                        state[u] = *reinterpret_cast<const float2*>(p.bound_state + (next * p.heads + head) * 2);
                    }
                }
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    if (owner[u] == row) {
                        csr::LseMerge(m, s, state[u].x, state[u].y);
                    }
                }
            }
        }
        for (int w = 1; w < walkers; ++w) {  // walker 0 gathers the others in order
            const float other_m = __shfl_sync(0xffffffffu, m, w * p.lanes + head);
            const float other_s = __shfl_sync(0xffffffffu, s, w * p.lanes + head);
            if (walker == 0) {
                csr::LseMerge(m, s, other_m, other_s);
            }
        }
        if (walker == 0 && head < p.heads && row >= 0 && row < p.rows) {
            p.lse[row * p.heads + head] = s == 0.0f ? m : m + __logf(s);
        }
    }
}

__global__ void FillKernel(float* out, float value, int64_t n)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        out[i] = value;
    }
}

inline int64_t Chunks(int64_t nnz) { return CeilDiv(nnz, kChunk); }

inline bool CheckDesc(const OpsgnnAttentionDesc* d)
{
    return d != nullptr && d->rows >= 0 && d->src_rows >= 0 && d->rows < 2147483647LL && d->src_rows < 2147483647LL && d->nnz >= 0 && d->heads >= 1 && d->heads <= 32 && d->width >= 1 &&
           (d->index_type == OPSGNN_I32 || d->index_type == OPSGNN_I64) && d->dtype == OPSGNN_F32;
}

}  // namespace attention
}  // namespace opsgnn

using namespace opsgnn;

extern "C" int opsgnn_attention_lse_workspace_bytes(const OpsgnnAttentionDesc* desc, int64_t* bytes)
{
    if (!attention::CheckDesc(desc) || bytes == nullptr) {
        return OPSGNN_ERR_INVALID;
    }
    const int64_t chunks = attention::Chunks(desc->nnz);
    *bytes = AlignUp((1 + attention::kMaxLongRuns) * 8, 256) + AlignUp(chunks * 2 * 8, 256) +
             AlignUp(chunks * 2 * desc->heads * 2 * 4, 256);
    return OPSGNN_OK;
}

extern "C" int opsgnn_attention_lse(const OpsgnnAttentionDesc* desc, const void* edge_rows, const void* col, const float* left,
                                    const float* right, float* logits, float* lse, void* workspace, int64_t workspace_bytes,
                                    void* stream)
{
    if (!attention::CheckDesc(desc)) {
        return OPSGNN_ERR_INVALID;
    }
    if (desc->rows == 0) {
        return OPSGNN_OK;
    }
    if (lse == nullptr || (desc->nnz > 0 && (edge_rows == nullptr || col == nullptr || left == nullptr || right == nullptr ||
                                             logits == nullptr))) {
        return OPSGNN_ERR_INVALID;
    }
    int64_t needed = 0;
    opsgnn_attention_lse_workspace_bytes(desc, &needed);
    if (desc->nnz > 0 && (workspace == nullptr || workspace_bytes < needed || !Aligned(workspace, 256))) {
        return OPSGNN_ERR_WORKSPACE;
    }
    cudaStream_t s = AsStream(stream);
    const int64_t cells = desc->rows * desc->heads;
    int64_t fill_blocks = CeilDiv(cells, 256);
    fill_blocks = fill_blocks < static_cast<int64_t>(SmCount()) * 8 ? fill_blocks : static_cast<int64_t>(SmCount()) * 8;
    attention::FillKernel<<<static_cast<unsigned>(fill_blocks), 256, 0, s>>>(lse, -INFINITY, cells);  // rows without edges
    if (desc->nnz == 0) {
        return LaunchStatus();
    }
    attention::LseParams p{};
    p.edge_rows = edge_rows;
    p.col = col;
    p.left = left;
    p.right = right;
    p.logits = logits;
    p.lse = lse;
    p.nnz = desc->nnz;
    p.rows = desc->rows;
    p.src_rows = desc->src_rows;
    p.chunks = attention::Chunks(desc->nnz);
    p.heads = static_cast<int>(desc->heads);
    p.lanes = 1;
    while (p.lanes < p.heads) {
        p.lanes <<= 1;
    }
    p.slope = desc->negative_slope;
    char* cursor = static_cast<char*>(workspace);
    p.long_runs = reinterpret_cast<int64_t*>(cursor);
    OPSGNN_CUDA_TRY(cudaMemsetAsync(p.long_runs, 0, sizeof(int64_t), s));
    cursor += AlignUp((1 + attention::kMaxLongRuns) * 8, 256);
    p.bound_row = reinterpret_cast<int64_t*>(cursor);
    cursor += AlignUp(p.chunks * 2 * 8, 256);
    p.bound_state = reinterpret_cast<float*>(cursor);
    const int64_t threads = p.chunks * p.lanes;
    const unsigned grid = static_cast<unsigned>(CeilDiv(threads, attention::kThreads));
    const bool wide = desc->index_type == OPSGNN_I64;
    if (p.heads == 8 && Aligned(left, 16) && Aligned(right, 16) && Aligned(logits, 16) && Aligned(lse, 16)) {
        const unsigned pairs = static_cast<unsigned>(CeilDiv(p.chunks * 2, attention::kThreads));
        if (wide) {
            attention::EdgeLogitLseQuadKernel<int64_t><<<pairs, attention::kThreads, 0, s>>>(p);
        } else {
            attention::EdgeLogitLseQuadKernel<int32_t><<<pairs, attention::kThreads, 0, s>>>(p);
        }
    } else if (p.lanes == 8) {
        if (wide) {
            attention::EdgeLogitLseTeamKernel<int64_t, 8><<<grid, attention::kThreads, 0, s>>>(p);
        } else {
            attention::EdgeLogitLseTeamKernel<int32_t, 8><<<grid, attention::kThreads, 0, s>>>(p);
        }
    } else if (p.lanes == 4) {
        if (wide) {
            attention::EdgeLogitLseTeamKernel<int64_t, 4><<<grid, attention::kThreads, 0, s>>>(p);
        } else {
            attention::EdgeLogitLseTeamKernel<int32_t, 4><<<grid, attention::kThreads, 0, s>>>(p);
        }
    } else if (wide) {
        attention::EdgeLogitLseKernel<int64_t><<<grid, attention::kThreads, 0, s>>>(p);
    } else {
        attention::EdgeLogitLseKernel<int32_t><<<grid, attention::kThreads, 0, s>>>(p);
    }
    const unsigned merge_grid = static_cast<unsigned>(CeilDiv(p.chunks * 2, attention::kThreads));
    attention::MergeBoundaryKernel<<<merge_grid, attention::kThreads, 0, s>>>(p);
    attention::LongRunKernel<<<static_cast<unsigned>(SmCount()) * 8, attention::kThreads, 0, s>>>(p);
    return LaunchStatus();
}

extern "C" int opsgnn_sorted_lse8_workspace_bytes(int64_t n, int64_t* bytes)
{
    if (n < 0 || bytes == nullptr) {
        return OPSGNN_ERR_INVALID;
    }
    const int64_t chunks = attention::Chunks(n);
    *bytes = AlignUp((1 + attention::kMaxLongRuns) * 8, 256) + AlignUp(chunks * 2 * 8, 256) + AlignUp(chunks * 2 * 8 * 2 * 4, 256);
    return OPSGNN_OK;
}

extern "C" int opsgnn_sorted_lse8(const void* labels, int index_type, const float* values, float* lse, int64_t n, int64_t groups,
                                  void* workspace, int64_t workspace_bytes, void* stream)
{
    if (n < 0 || groups < 0 || (index_type != OPSGNN_I32 && index_type != OPSGNN_I64)) {
        return OPSGNN_ERR_INVALID;
    }
    if (groups == 0) {
        return OPSGNN_OK;
    }
    if (lse == nullptr || !Aligned(lse, 16) || (n > 0 && (labels == nullptr || values == nullptr || !Aligned(values, 16)))) {
        return OPSGNN_ERR_INVALID;
    }
    if (groups >= (int64_t(1) << 31)) {  // group ids travel as 32-bit values inside the sweep
        return OPSGNN_ERR_LIMIT;
    }
    int64_t needed = 0;
    opsgnn_sorted_lse8_workspace_bytes(n, &needed);
    if (n > 0 && (workspace == nullptr || workspace_bytes < needed || !Aligned(workspace, 256))) {
        return OPSGNN_ERR_WORKSPACE;
    }
    cudaStream_t s = AsStream(stream);
    const int64_t cells = groups * 8;
    int64_t fill_blocks = CeilDiv(cells, 256);
    fill_blocks = fill_blocks < static_cast<int64_t>(SmCount()) * 8 ? fill_blocks : static_cast<int64_t>(SmCount()) * 8;
    attention::FillKernel<<<static_cast<unsigned>(fill_blocks), 256, 0, s>>>(lse, -INFINITY, cells);  // groups without elements
    if (n == 0) {
        return LaunchStatus();
    }
    attention::LseParams p{};
    p.edge_rows = labels;
    p.right = values;
    p.lse = lse;
    p.nnz = n;
    p.rows = groups;
    p.src_rows = n;
    p.chunks = attention::Chunks(n);
    p.heads = 8;
    p.lanes = 8;
    char* cursor = static_cast<char*>(workspace);
    p.long_runs = reinterpret_cast<int64_t*>(cursor);
    OPSGNN_CUDA_TRY(cudaMemsetAsync(p.long_runs, 0, sizeof(int64_t), s));
    cursor += AlignUp((1 + attention::kMaxLongRuns) * 8, 256);
    p.bound_row = reinterpret_cast<int64_t*>(cursor);
    cursor += AlignUp(p.chunks * 2 * 8, 256);
    p.bound_state = reinterpret_cast<float*>(cursor);
    const unsigned pairs = static_cast<unsigned>(CeilDiv(p.chunks * 2, attention::kThreads));
    if (index_type == OPSGNN_I64) {
        attention::EdgeLogitLseQuadKernel<int64_t, true><<<pairs, attention::kThreads, 0, s>>>(p);
    } else {
        attention::EdgeLogitLseQuadKernel<int32_t, true><<<pairs, attention::kThreads, 0, s>>>(p);
    }
    const unsigned merge_grid = static_cast<unsigned>(CeilDiv(p.chunks * 2, attention::kThreads));
    attention::MergeBoundaryKernel<<<merge_grid, attention::kThreads, 0, s>>>(p);
    attention::LongRunKernel<<<static_cast<unsigned>(SmCount()) * 8, attention::kThreads, 0, s>>>(p);
    return LaunchStatus();
}

extern "C" int opsgnn_attention_aggregate(const OpsgnnAttentionDesc* desc, const void* ptr, const void* col, const float* logits,
                                          const float* lse, const void* x, void* out, const void* plan, void* workspace,
                                          int64_t workspace_bytes, void* stream)
{
    if (!attention::CheckDesc(desc)) {
        return OPSGNN_ERR_INVALID;
    }
    const int64_t feat = desc->heads * desc->width;
    // The weighted bulk instance: 256-feature tiles of 16-byte vectors, a stage's column-side halves in its weight slot.
    if (feat % 256 != 0 || (desc->heads * 4) % 16 != 0 || desc->width % 4 != 0 ||
        (csr::kBulkStageBytes / 1024) * desc->heads * 4 > csr::kBulkWeightBytes) {
        return OPSGNN_ERR_UNSUPPORTED;
    }
    if (desc->rows == 0) {
        return OPSGNN_OK;
    }
    if (ptr == nullptr || out == nullptr || plan == nullptr || lse == nullptr ||
        (desc->nnz > 0 && (col == nullptr || logits == nullptr || x == nullptr))) {
        return OPSGNN_ERR_INVALID;
    }
    if (!Aligned(logits, 16) || !Aligned(x, 16) || !Aligned(out, 16)) {
        return OPSGNN_ERR_UNSUPPORTED;
    }
    OpsgnnCsrReduceDesc reduce{};
    reduce.rows = desc->rows;
    reduce.src_rows = desc->src_rows;
    reduce.feat = feat;
    reduce.nnz = desc->nnz;
    reduce.batches = 1;
    reduce.value_width = desc->heads;
    reduce.reduce = OPSGNN_REDUCE_SUM;
    reduce.ptr_type = desc->index_type;
    reduce.col_type = desc->index_type;
    reduce.in_type = OPSGNN_F32;
    reduce.out_type = OPSGNN_F32;
    return csr::RunAttention(reduce, ptr, col, logits, lse, x, out, plan, workspace, workspace_bytes, stream);
}
