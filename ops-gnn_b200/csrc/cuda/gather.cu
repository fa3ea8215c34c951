// Row gather with a bounded footprint: out[i, :] = src[index[i], :], the output cut into up to sixteen consecutive
// segments that may live in different buffers - this GPU's memory or a peer's (plain stores; no multicast anywhere).
//
// This is the exchange kernel of the sharded SpMM.  A rank packs the rows its peers want from its block of the dense
// operand, either into a local send buffer or straight into every peer's receive buffer (one launch serves all peers,
// so all of them receive at once).  The kernel runs beside the SpMM of an earlier stage and is bound by NVLink, not by
// the SMs, so its grid can be capped (`max_ctas`) to leave SM slots to the product.  The work unit is one 512-byte piece
// of a row per warp instruction (16 bytes per lane); every warp keeps kUnroll pieces (8 KiB) in flight, because a
// block's throughput is its bytes in flight over the link's round trip (measured between two B200s with 8 pieces in
// flight: 136 / 270 / 510 / 610 GB/s with 16 / 32 / 64 / 148 blocks).  Algorithmic bytes: rows * (index + 2 * row bytes).
#include "common.cuh"

namespace opsgnn {
namespace gather {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kUnroll = 16;
constexpr int kMaxSegments = OPSGNN_GATHER_MAX_SEGMENTS;

struct Params {
    const unsigned char* src;
    const void* index;
    int64_t rows;       // rows gathered in total
    int64_t src_rows;   // rows of src: indices are clamped into [0, src_rows)
    int64_t row_bytes;  // a multiple of 16
    int pieces_per_row; // ceil(row_bytes / 512)
    int segments;
    int64_t start[kMaxSegments + 1];   // segment s holds output rows [start[s], start[s + 1])
    unsigned char* out[kMaxSegments];  // base of segment s
};

template <class IndexT>
__global__ void __launch_bounds__(kThreads) GatherRowsKernel(const Params p)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    const int64_t warps = static_cast<int64_t>(gridDim.x) * kWarps;
    const int64_t total = p.rows * p.pieces_per_row;
    const IndexT* __restrict__ index = static_cast<const IndexT*>(p.index);
    const int lane_offset = lane * 16;
    for (int64_t first = warp * kUnroll; first < total; first += warps * kUnroll) {
        uint4 piece[kUnroll];
        unsigned char* target[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            target[u] = nullptr;
            const int64_t item = first + u;
            if (item >= total) {
                continue;
            }
            const int64_t row = item / p.pieces_per_row;
            const int64_t offset = (item - row * p.pieces_per_row) * 512 + lane_offset;
            if (offset >= p.row_bytes) {
                continue;
            }
            int64_t from = static_cast<int64_t>(__ldg(index + row));
            from = from < 0 ? 0 : (from >= p.src_rows ? p.src_rows - 1 : from);  // validated upstream; never fault
            piece[u] = __ldg(reinterpret_cast<const uint4*>(p.src + from * p.row_bytes + offset));
            int s = 0;
#pragma unroll
            for (int k = 1; k < kMaxSegments; ++k) {
                s += (k < p.segments && row >= p.start[k]) ? 1 : 0;
            }
            target[u] = p.out[s] + (row - p.start[s]) * p.row_bytes + offset;
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (target[u] != nullptr) {
                *reinterpret_cast<uint4*>(target[u]) = piece[u];
            }
        }
    }
}

// ---- gather_coo / gather_csr: batched row expansion ----------------------------------------------------------------------
// out[b, i, :] = src[b, from(b, i), :] with from = index[b, i] (COO) or the segment s with ptr[b, s] <= i < ptr[b, s + 1]
// (CSR; output rows before ptr[b, 0] are zero).  `lanes` lanes (a power of two) share one output row and move UNIT bytes
// per lane and step, so a row of a few bytes does not idle a warp.  Algorithmic bytes: out rows * (index + 2 * row bytes).
struct ExpandParams {
    const unsigned char* src;
    const int64_t* index;  // COO: [batches, out_rows]; CSR: [batches, segments + 1]
    unsigned char* out;
    int64_t batches, src_rows, out_rows, row_bytes;
    int csr;    // 1: index holds segment pointers
    int lanes;  // lanes per output row
};

template <class Unit> __global__ void __launch_bounds__(kThreads) ExpandRowsKernel(const ExpandParams p)
{
    const int lane = threadIdx.x & 31;
    const int within = lane & (p.lanes - 1);
    const int per_warp = 32 / p.lanes;
    const int64_t warp = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    const int64_t warps = static_cast<int64_t>(gridDim.x) * kWarps;
    const int64_t total = p.batches * p.out_rows;
    for (int64_t first = warp * per_warp; first < total; first += warps * per_warp) {
        const int64_t row = first + lane / p.lanes;
        if (row >= total) {
            continue;
        }
        const int64_t b = row / p.out_rows;
        const int64_t i = row - b * p.out_rows;
        int64_t from;
        if (p.csr) {
            const int64_t* ptr = p.index + b * (p.src_rows + 1);
            int64_t lo = 0, hi = p.src_rows + 1;  // first s with ptr[s] > i
            while (lo < hi) {
                const int64_t mid = (lo + hi) >> 1;
                if (__ldg(ptr + mid) <= i) {
                    lo = mid + 1;
                } else {
                    hi = mid;
                }
            }
            from = lo - 1;  // -1: the row lies before ptr[0]; src_rows: beyond the last pointer (never, rows = endpoint)
        } else {
            from = __ldg(p.index + row);
        }
        const bool covered = from >= 0 && from < p.src_rows;
        const Unit* source = reinterpret_cast<const Unit*>(p.src + (b * p.src_rows + (covered ? from : 0)) * p.row_bytes);
        Unit* target = reinterpret_cast<Unit*>(p.out + row * p.row_bytes);
        const int64_t units = p.row_bytes / static_cast<int64_t>(sizeof(Unit));
        for (int64_t u = within; u < units; u += p.lanes) {
            target[u] = covered ? __ldg(source + u) : Unit{};
        }
    }
}

template <class Unit> int LaunchExpand(ExpandParams p, cudaStream_t stream)
{
    const int64_t units = p.row_bytes / static_cast<int64_t>(sizeof(Unit));
    int lanes = 1;
    while (lanes < 32 && lanes < units) {
        lanes <<= 1;
    }
    p.lanes = lanes;
    const int64_t total = p.batches * p.out_rows;
    int64_t ctas = CeilDiv(total, static_cast<int64_t>(kWarps) * (32 / lanes));
    const int64_t cap = static_cast<int64_t>(SmCount()) * 16;
    ctas = ctas < cap ? ctas : cap;
    ExpandRowsKernel<Unit><<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(p);
    return LaunchStatus();
}

}  // namespace gather
}  // namespace opsgnn

using namespace opsgnn;

extern "C" int opsgnn_gather_expand(const void* src, const int64_t* index, void* out, int64_t batches, int64_t src_rows,
                                    int64_t out_rows, int64_t row_bytes, int csr, void* stream)
{
    if (batches < 0 || src_rows < 0 || out_rows < 0 || row_bytes < 0) {
        return OPSGNN_ERR_INVALID;
    }
    if (batches == 0 || out_rows == 0 || row_bytes == 0) {
        return OPSGNN_OK;
    }
    if (out == nullptr || index == nullptr || (src_rows > 0 && src == nullptr)) {
        return OPSGNN_ERR_INVALID;
    }
    gather::ExpandParams p{};
    p.src = static_cast<const unsigned char*>(src);
    p.index = index;
    p.out = static_cast<unsigned char*>(out);
    p.batches = batches;
    p.src_rows = src_rows;
    p.out_rows = out_rows;
    p.row_bytes = row_bytes;
    p.csr = csr ? 1 : 0;
    cudaStream_t s = AsStream(stream);
    const uintptr_t mix = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(out) | static_cast<uintptr_t>(row_bytes);
    if (mix % 16 == 0) {
        return gather::LaunchExpand<uint4>(p, s);
    }
    if (mix % 8 == 0) {
        return gather::LaunchExpand<uint2>(p, s);
    }
    if (mix % 4 == 0) {
        return gather::LaunchExpand<uint32_t>(p, s);
    }
    if (mix % 2 == 0) {
        return gather::LaunchExpand<uint16_t>(p, s);
    }
    return gather::LaunchExpand<uint8_t>(p, s);
}

extern "C" int opsgnn_gather_rows(const void* src, const void* index, int index_type, int64_t rows, int64_t src_rows,
                                  int64_t row_bytes, int segments, const int64_t* segment_rows, void* const* segment_out,
                                  int max_ctas, void* stream)
{
    if (rows < 0 || src_rows < 0 || row_bytes < 0 || segments < 1 || segments > gather::kMaxSegments ||
        segment_rows == nullptr || segment_out == nullptr) {
        return OPSGNN_ERR_INVALID;
    }
    if (index_type != OPSGNN_I32 && index_type != OPSGNN_I64) {
        return OPSGNN_ERR_INVALID;
    }
    if (rows == 0 || row_bytes == 0) {
        return OPSGNN_OK;
    }
    if (src == nullptr || index == nullptr || src_rows == 0 || row_bytes % 16 != 0 || !Aligned(src, 16)) {
        return OPSGNN_ERR_INVALID;
    }
    gather::Params p{};
    p.src = static_cast<const unsigned char*>(src);
    p.index = index;
    p.rows = rows;
    p.src_rows = src_rows;
    p.row_bytes = row_bytes;
    p.pieces_per_row = static_cast<int>(CeilDiv(row_bytes, 512));
    p.segments = segments;
    int64_t at = 0;
    for (int s = 0; s < segments; ++s) {
        if (segment_rows[s] < 0 || (segment_rows[s] > 0 && (segment_out[s] == nullptr || !Aligned(segment_out[s], 16)))) {
            return OPSGNN_ERR_INVALID;
        }
        p.start[s] = at;
        p.out[s] = static_cast<unsigned char*>(segment_out[s]);
        at += segment_rows[s];
    }
    for (int s = segments; s <= gather::kMaxSegments; ++s) {
        p.start[s] = at;
    }
    if (at != rows) {
        return OPSGNN_ERR_INVALID;
    }
    const int64_t total = rows * p.pieces_per_row;
    int64_t ctas = CeilDiv(total, static_cast<int64_t>(gather::kWarps) * gather::kUnroll);
    const int64_t cap = max_ctas > 0 ? max_ctas : static_cast<int64_t>(SmCount()) * 8;
    ctas = ctas < cap ? ctas : cap;
    cudaStream_t s = AsStream(stream);
    if (index_type == OPSGNN_I64) {
        gather::GatherRowsKernel<int64_t><<<static_cast<unsigned>(ctas), gather::kThreads, 0, s>>>(p);
    } else {
        gather::GatherRowsKernel<int32_t><<<static_cast<unsigned>(ctas), gather::kThreads, 0, s>>>(p);
    }
    return LaunchStatus();
}
