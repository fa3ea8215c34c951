// CSR reduce engine for sm_100a.
//
//   out[b, r, k] = reduce_{e in [ptr[r], ptr[r+1])}  w(e, k) * mat[b, col(e), k]
//
// One kernel family serves weighted/unweighted SpMM (col = column indices), segment_csr / segment_coo
// (col(e) = e) and segment log-sum-exp.  Design, in the order the data flows:
//
//  * Work is the merged list of "edges" and "row ends" (merge-path).  Every thread block owns kItemsPerCta
//    consecutive items of that list and every warp kItemsPerWarp of them, so a power-law row with millions of
//    edges is spread over many blocks and a run of empty rows costs the same as a run of edges.  The block's
//    start row comes from a plan (one binary search per block, built once per graph by PlanKernel).
//  * The block stages its row ends, column offsets and scalar weights in shared memory with plain coalesced
//    loads; each warp then walks its items with warp-uniform control flow: all 32 lanes work on the same edge and
//    own different features, so a gathered dense row is read with one or two 16-byte loads per lane (a 512-byte
//    or 1-KiB fully coalesced request per warp) and kEdgeBatch rows are in flight per warp before the first use.
//  * Instances (template flags of ReduceKernel): BULK keeps the gathered rows of a batch in a per-warp ring in shared
//    memory instead of registers (bulk copies + mbarriers for rows of 512 bytes and more); NARROW lets several lane
//    groups share a warp when a row is 16 to 256 bytes (per-lane cp.async copies, partial results merged by shuffles
//    at row ends); GENERAL adds one weight per feature or per feature group (with BULK: per-group weights ride in the
//    ring beside the rows).  Everything else (extrema under three tie / NaN rules, online log-sum-exp, mean) is shared.
//  * A row that ends inside the warp's items is written with streaming 16-byte stores.  Edges of a row whose end
//    lies in a later warp are a "carry": carries are combined in item order after a block barrier, rows that
//    end in the same block are patched in place, and at most one carry per block goes to global scratch where
//    FixupKernel adds it to the row in block order.  No atomics: results are bitwise reproducible.
//
// Algorithmic bytes per launch (the roofline numerator): nnz*(sizeof(col)+sizeof(val)+K*sizeof(T)) +
// rows*(sizeof(ptr)+K*sizeof(O)) (+ rows*K*8 for arg).
#pragma once

#include <cstdlib>

#include "common.cuh"

namespace opsgnn {
namespace csr {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kItemsPerWarp = 128;
constexpr int kItemsPerCta = kWarps * kItemsPerWarp;

enum ReduceKind { kSum = 0, kExtremum = 1, kLogSumExp = 2 };

struct Identity {};  // col(e) = e

struct Params {
    const void* ptr;
    const void* col;
    const void* val;
    const void* mat;
    void* out;
    int64_t* arg;
    const int64_t* plan;  // start row of every block, num_cta + 1 entries
    void* carry_val;      // [num_cta][carry_stride] accumulators
    int64_t* carry_arg;   // [num_cta][carry_stride] (extrema only)
    int64_t* carry_row;   // [num_cta] row that receives the block's carry, -1 for none
    int64_t rows;
    int64_t src_rows;
    int64_t feat;
    int64_t nnz;
    int64_t batches;
    int64_t arg_none;
    int64_t num_cta;
    int64_t carry_stride;  // gridDim.y * TILE
    unsigned long long* debug;  // OPSGNN_CHECKED builds: {violations, first site, index, limit}
    unsigned long long* status;       // head of the workspace: number of bulk waits that ran out of polls in this launch
    unsigned long long* status_sink;  // optional second place for the same report (device-visible, e.g. mapped host memory)
    uint32_t wait_polls;              // polls of one mbarrier wait before the warp gives up (kBulkSpinLimit by default)
    int tiles_per_batch;
    int mean;      // kSum: divide by the row's edge count
    int is_min;    // kExtremum
    int extremum;  // OPSGNN_EXTREMUM_*
    int has_val;
    int wide;      // 0: one weight per edge (or none); 1: one per (edge, feature); 2: one per (edge, feature group)
    int64_t val_width;  // weights per edge
    int64_t val_group;  // wide == 2: consecutive features that share a weight (feat / val_width)
    int lanes_per_row;  // narrow instance: lanes that share one gathered row (a power of two below 32)
    // Attention mode of the weighted bulk instance (fp32): `val` holds one LOGIT per (edge, feature group) and the weight
    // is formed on the fly, w = exp(val[e, h] - att_lse[row, h]): the softmax over the row's edges given the row's
    // log-sum-exp, which is read once per row.  The softmax weights themselves are never in memory.
    const float* att_lse;
    int attention;
};

// Self-checking build (-DOPSGNN_CHECKED): every global access of the reduce kernel is bounds-checked; a bad index is
// recorded (first site wins) and the access skipped, so a wrong index shows up as a report instead of a fault.
#ifdef OPSGNN_CHECKED
__device__ __forceinline__ bool GuardFail(unsigned long long* debug, int site, int64_t index, int64_t limit)
{
    if (debug != nullptr && atomicAdd(debug, 1ULL) == 0ULL) {
        debug[1] = static_cast<unsigned long long>(site);
        debug[2] = static_cast<unsigned long long>(index);
        debug[3] = static_cast<unsigned long long>(limit);
    }
    return false;
}
#define OPSGNN_GUARD(site, index, limit) \
    (((index) >= 0 && (index) < (limit)) ? true : GuardFail(p.debug, (site), (index), (limit)))
#else
#define OPSGNN_GUARD(site, index, limit) true
#endif

__host__ __device__ inline int64_t NumCta(int64_t rows, int64_t nnz) { return (rows + nnz + kItemsPerCta - 1) / kItemsPerCta; }

// Edges actually covered by the pointer array, given the host's upper bound (the grid is sized for the bound).
__host__ __device__ inline int64_t ActualEdges(int64_t first, int64_t last, int64_t bound)
{
    const int64_t span = last - first;
    return span < 0 ? 0 : (span > bound ? bound : span);
}

// ---- plan: start row of each block's diagonal ----------------------------------------------------------------
template <class PtrT>
__global__ void PlanKernel(const PtrT* __restrict__ ptr, int64_t rows, int64_t nnz, int64_t num_cta,
                           int64_t* __restrict__ plan)
{
    const int64_t b = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (b > num_cta) {
        return;
    }
    // Edges are counted from ptr[0]: segment pointers need not start at zero nor cover every source row.
    const int64_t base = static_cast<int64_t>(ptr[0]);
    nnz = ActualEdges(base, static_cast<int64_t>(ptr[rows]), nnz);
    const int64_t total = rows + nnz;
    int64_t diag = b * kItemsPerCta;
    diag = diag < total ? diag : total;
    int64_t lo = diag > nnz ? diag - nnz : 0;
    int64_t hi = diag < rows ? diag : rows;
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (static_cast<int64_t>(ptr[mid + 1]) - base <= diag - 1 - mid) {
            lo = mid + 1;
        } else {
            hi = mid;
        }
    }
    plan[b] = lo;
}

// ---- element algebra -----------------------------------------------------------------------------------------
template <class A> __device__ __forceinline__ bool IsNan(A v) { return v != v; }

// Extremum update; `arg < 0` means nothing selected yet.  Earlier items are offered first, so strict compares
// keep the first occurrence among ties.
template <class A, class I = int64_t>
__device__ __forceinline__ void ExtremumOffer(A& acc, I& arg, A v, I where, int is_min, int rule)
{
    const bool better = is_min ? (v < acc) : (v > acc);
    bool take;
    if (rule == OPSGNN_EXTREMUM_IGNORE_NAN) {
        take = !IsNan(v) && (arg < 0 || better);
    } else if (rule == OPSGNN_EXTREMUM_PROPAGATE_NAN) {
        take = arg < 0 || better || (IsNan(v) && !IsNan(acc));
    } else if (rule == OPSGNN_EXTREMUM_SEEDED_LAST) {
        take = is_min ? (v <= acc) : (v >= acc);  // later edges are offered later: the last of equal values stays
    } else {
        take = better;
    }
    if (take) {
        acc = v;
        arg = where;
    }
}

// Seed of the "seeded" rule: the finite extreme of the storage dtype T, held in the accumulator type.
template <class A, class T> __device__ __forceinline__ A ExtremumSeed(int is_min, int rule)
{
    if (rule == OPSGNN_EXTREMUM_SEEDED || rule == OPSGNN_EXTREMUM_SEEDED_LAST) {
        return is_min ? static_cast<A>(Limits<T>::Max()) : static_cast<A>(Limits<T>::Lowest());
    }
    return A(0);
}

// log(exp(a) + exp(b)) with the conventions of torch.logsumexp: -inf is the empty sum, +inf absorbs, NaN spreads.
__device__ __forceinline__ float LogAddExp(float a, float b)
{
    const float hi = fmaxf(a, b);  // fmaxf drops a NaN operand, so NaN is re-injected below
    const float lo = fminf(a, b);
    if (IsNan(a) || IsNan(b)) {
        return a + b;
    }
    if (hi == lo) {  // covers (+inf,+inf) and (-inf,-inf) without inf-inf
        return isinf(hi) ? hi : hi + 0.6931471805599453f;
    }
    return hi + log1pf(__expf(lo - hi));
}

// Online log-sum-exp state (running maximum m, sum of exp(x - m)).
__device__ __forceinline__ void LseOffer(float& m, float& s, float x)
{
    if (x > m) {
        s = s * __expf(m - x) + 1.0f;  // m = -inf initially: s = 0 * 0 + 1
        m = x;
    } else {
        const float d = (x == m) ? 0.0f : x - m;  // equal infinities contribute exp(0)
        s += __expf(d);                            // NaN input: d = NaN, s = NaN
    }
}

// Merge of two online states (maximum, sum of exp(x - maximum)); symmetric in its operands.  The maximum is never
// NaN (a NaN input lands in the sum), equal maxima - infinite ones included - add their sums unscaled.
__device__ __forceinline__ void LseMerge(float& m, float& s, float other_m, float other_s)
{
    const bool mine_high = m >= other_m;
    const float hi = mine_high ? m : other_m;
    const float lo = mine_high ? other_m : m;
    const float s_hi = mine_high ? s : other_s;
    const float s_lo = mine_high ? other_s : s;
    const float scale = (hi == lo) ? 1.0f : __expf(lo - hi);
    m = hi;
    s = s_hi + s_lo * scale;
}

__device__ __forceinline__ float LseFinish(float m, float s)
{
    if (s == 0.0f) {
        return m;  // empty: m = -inf
    }
    return m + __logf(s);
}

// Merge of two partial extrema taken under the same rule over disjoint edge sets: the result is what one scan over
// the union in edge order would have selected (first NaN under the propagating rule, else the extremum with the
// smallest position among ties).  Symmetric in its two operands.
template <class A, class I = int64_t>
__device__ __forceinline__ void ExtremumMerge(A& acc, I& arg, A other, I other_arg, int is_min, int rule)
{
    if (other_arg < 0) {
        return;
    }
    if (arg < 0) {
        acc = other;
        arg = other_arg;
        return;
    }
    if (rule == OPSGNN_EXTREMUM_PROPAGATE_NAN && (IsNan(acc) || IsNan(other))) {
        if (IsNan(other) && (!IsNan(acc) || other_arg < arg)) {
            acc = other;
            arg = other_arg;
        }
        return;
    }
    const bool better = is_min ? (other < acc) : (other > acc);
    const bool tie_goes_to_other = rule == OPSGNN_EXTREMUM_SEEDED_LAST ? other_arg > arg : other_arg < arg;
    if (better || (other == acc && tie_goes_to_other)) {
        acc = other;
        arg = other_arg;
    }
}

template <class V> __device__ __forceinline__ V ShuffleXor(V v, int mask) { return __shfl_xor_sync(0xffffffffu, v, mask); }
__device__ __forceinline__ int64_t ShuffleXor(int64_t v, int mask)
{
    return static_cast<int64_t>(__shfl_xor_sync(0xffffffffu, static_cast<long long>(v), mask));
}

// ---- bulk-copy (TMA 1-D) ring ------------------------------------------------------------------------------------
#ifndef OPSGNN_PACKED_FMA
#define OPSGNN_PACKED_FMA 1  // 0: scalar multiply-adds (comparison builds)
#endif
#ifndef OPSGNN_BULK_STAGES
#define OPSGNN_BULK_STAGES 2
#endif
#ifndef OPSGNN_SUM_BLOCKS_PER_SM
#define OPSGNN_SUM_BLOCKS_PER_SM 3  // resident blocks the lean bulk sum instances are compiled for (register budget)
#endif
#ifndef OPSGNN_BULK_STAGE_BYTES
#define OPSGNN_BULK_STAGE_BYTES 3072
#endif
constexpr int kBulkStages = OPSGNN_BULK_STAGES;            // stages per warp
constexpr int kBulkStageBytes = OPSGNN_BULK_STAGE_BYTES;   // bytes per stage: 3 rows of 1 KiB, 6 of 512 B, ...
constexpr int kBulkWarpBytes = kBulkStages * kBulkStageBytes;
constexpr int kBulkSmemBytes = kWarps * kBulkWarpBytes + kWarps * kBulkStages * 8;
// Per-group weights (one per edge and feature group, e.g. attention heads) ride along with the rows of a stage: the
// weights of the stage's edges are contiguous in memory, so one more bulk copy per stage brings them in.
constexpr int kBulkWeightBytes = 256;  // per stage: rows per stage x weights per edge x sizeof(T) must fit
constexpr int kBulkSmemBytesWeighted = kBulkSmemBytes + kWarps * kBulkStages * kBulkWeightBytes;
// A failed try_wait may suspend the thread for up to this many nanoseconds (it wakes as soon as the phase completes),
// so a waiting warp does not burn issue slots polling; the poll count bounds the wait to a few seconds in total, past
// which the warp counts itself in the launch's status word (Params::status, and Params::status_sink when one is
// registered), waits - bounded again - for its copies still in flight and leaves its remaining rows unwritten.  The
// host reads the status word and turns a non-zero count into an error; a launch never hangs on a copy.
constexpr uint32_t kBulkWaitHintNs = 100000u;
constexpr uint32_t kBulkSpinLimit = 1u << 15;

__device__ __forceinline__ uint32_t SharedAddress(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void MbarInit(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void MbarExpectTx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool MbarTryWait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(kBulkWaitHintNs)
        : "memory");
    return done != 0;
}
// Global -> shared bulk copy; source and destination 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void BulkLoad(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// Two ways to fill the ring.  Wide rows (512 bytes and more): one `cp.async.bulk` per gathered row, completion on an
// mbarrier per stage.  Narrow rows: per-lane 16-byte `cp.async.cg` copies, so one warp instruction moves 32 / lanes
// per row rows, completion by commit / wait groups.  Measured on an R-MAT graph (64M edges): bulk copies win by 3-4 %
// at 512-byte and 1-KiB rows, per-lane copies by 5-25 % below that (a bulk copy is issued once per active lane).

__device__ __forceinline__ void AsyncCopy16(uint32_t dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void AsyncCommit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING> __device__ __forceinline__ void AsyncWait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory");
}

template <class T, class O, class PtrT, class ColT, int VEC, int NV, int RK> struct Traits {
    using A = typename AccOf<T>::type;
    static constexpr int kTile = 32 * VEC * NV;
    static constexpr int kElems = VEC * NV;
    // Gathered rows in flight per warp before the first use: about 256 bytes per lane for sums (sixteen 16-byte
    // loads with one vector per lane, eight pairs with two), half of that where positions ride along.
    static constexpr int kEdgeBatch = (RK == kSum) ? (NV == 1 ? 16 : 8) : (NV == 1 ? 8 : 4);
};

// ---- main kernel ---------------------------------------------------------------------------------------------
// GENERAL = false is the lean instance for calls without weights or with one weight per edge (the weight is staged
// in shared memory, 1 when absent); GENERAL = true also handles one weight per feature or per feature group.
//
// BULK = true gathers the dense rows with the bulk-copy engine instead of per-lane loads: one lane issues one
// `cp.async.bulk` per gathered row segment (up to 1 KiB) into a per-warp ring of kBulkStages stages in shared
// memory, completion is tracked by one mbarrier per stage, and the lanes read their 16-byte vectors back with
// conflict-free shared loads.  Rows in flight then cost shared memory instead of registers (6 KiB per warp), which
// leaves room for three resident blocks per SM, and one instruction moves a whole row.
//
// NARROW = true (bulk only, NV == 1) is for rows narrower than one warp of 16-byte vectors (16 to 256 bytes, a power
// of two): p.lanes_per_row lanes share a gathered row and the 32 / lanes_per_row lane groups take different edges of
// the same run, so no lane idles; the groups' partial results are merged with shuffles when the row ends.
template <class T, class O, class PtrT, class ColT, int VEC, int NV, int RK, bool GENERAL, bool BULK, bool NARROW = false>
__global__ void __launch_bounds__(kThreads, BULK ? OPSGNN_SUM_BLOCKS_PER_SM : 2)
    ReduceKernel(const Params p)
{
    static_assert(!NARROW || (BULK && NV == 1 && !GENERAL), "the narrow layout exists for lean bulk instances only");
    constexpr bool kRingAsync = NARROW;
    static_assert(NARROW || (BULK ? kBulkStageBytes / (32 * VEC * NV * static_cast<int>(sizeof(T))) : 16) <= 16,
                  "the slot dispatch below enumerates sixteen slots");
    using TR = Traits<T, O, PtrT, ColT, VEC, NV, RK>;
    using A = typename TR::A;
    constexpr int TILE = TR::kTile;
    constexpr int ELEMS = TR::kElems;
    constexpr int kRowBytes = TILE * static_cast<int>(sizeof(T));  // one staged row segment
    constexpr int EB = BULK ? kBulkStageBytes / kRowBytes : TR::kEdgeBatch;
    constexpr bool kIdentity = std::is_same<ColT, Identity>::value;
    constexpr bool kHasArg = RK == kExtremum;
    // sums in float with an even vector width fold two elements per instruction
    constexpr bool kPackedFma = OPSGNN_PACKED_FMA && RK == kSum && std::is_same<typename Traits<T, O, PtrT, ColT, VEC, NV, RK>::A, float>::value && VEC % 2 == 0;

    __shared__ int s_end[kItemsPerCta + 1];
    __shared__ int32_t s_col[kItemsPerCta];  // col(e), clamped to the source rows (fewer than 2^31, checked on the host)
    // edge weights, already widened (1 when the call has none); the weighted bulk instance keeps its weights in the ring
    __shared__ A s_val[(GENERAL && BULK) ? 1 : kItemsPerCta];
    __shared__ int s_split[kWarps + 1];
    __shared__ int s_carry_row[kWarps];
    // Carries of the eight warps.  The bulk variant parks them in each warp's (by then drained) ring instead.
    __shared__ A s_carry_static[BULK ? 1 : kWarps][BULK ? 1 : TILE];
    __shared__ int64_t s_carry_arg_static[(kHasArg && !BULK) ? kWarps : 1][(kHasArg && !BULK) ? TILE : 1];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int64_t cta = blockIdx.x;
    const int batch = blockIdx.y / p.tiles_per_batch;
    const int tile = blockIdx.y - batch * p.tiles_per_batch;
    const int64_t kbase = static_cast<int64_t>(tile) * TILE;
    const int64_t K = p.feat;
    // Lane layout: `lpg` lanes share one gathered row; group `grp` takes every `groups`-th edge of a run.
    const int lpg = NARROW ? p.lanes_per_row : 32;
    const int groups = NARROW ? 32 / lpg : 1;
    const int grp = NARROW ? lane / lpg : 0;
    const int lane_in = NARROW ? (lane & (lpg - 1)) : lane;
    const int row_bytes = NARROW ? lpg * VEC * static_cast<int>(sizeof(T)) : kRowBytes;  // one staged row segment
    const int eb = NARROW ? kBulkStageBytes / row_bytes : EB;                            // rows per stage / batch

    const PtrT* __restrict__ ptr = static_cast<const PtrT*>(p.ptr);
    const T* __restrict__ mat = static_cast<const T*>(p.mat) + static_cast<int64_t>(batch) * p.src_rows * K;
    const T* __restrict__ val = static_cast<const T*>(p.val);
    O* __restrict__ out = static_cast<O*>(p.out) + static_cast<int64_t>(batch) * p.rows * K;
    int64_t* __restrict__ arg = kHasArg ? p.arg + static_cast<int64_t>(batch) * p.rows * K : nullptr;

    // ---- stage this block's items --------------------------------------------------------------------------
    const int64_t base = static_cast<int64_t>(ptr[0]);
    const int64_t total = p.rows + ActualEdges(base, static_cast<int64_t>(ptr[p.rows]), p.nnz);
    const int64_t d0 = cta * kItemsPerCta;
    if (d0 >= total) {  // the grid is sized for the host's edge bound
        if (tid == 0 && blockIdx.y == 0) {
            p.carry_row[cta] = -1;
        }
        return;
    }
    const int64_t d1 = (d0 + kItemsPerCta < total) ? d0 + kItemsPerCta : total;
    const int64_t row0 = OPSGNN_GUARD(1, cta + 1, p.num_cta + 1) ? p.plan[cta] : 0;
    const int64_t row1 = OPSGNN_GUARD(1, cta + 1, p.num_cta + 1) ? p.plan[cta + 1] : 0;
    const int64_t e0 = d0 - row0;  // first edge of the block, counted from `base`
    const int64_t a0 = base + e0;  // the same edge as an absolute position in col / val / the source rows
    int nR = static_cast<int>(row1 - row0);
    int nE = static_cast<int>((d1 - row1) - e0);
    // A malformed plan or pointer array must not index outside the staging buffers.
    nR = nR < 0 ? 0 : (nR > kItemsPerCta ? kItemsPerCta : nR);
    nE = nE < 0 ? 0 : (nE > kItemsPerCta ? kItemsPerCta : nE);

    for (int i = tid; i < nR; i += kThreads) {
        int64_t rel = (OPSGNN_GUARD(2, row0 + 1 + i, p.rows + 1) ? static_cast<int64_t>(LoadStream(ptr + row0 + 1 + i)) : 0) - a0;
        rel = rel < 0 ? 0 : (rel > nE ? nE : rel);
        s_end[i] = static_cast<int>(rel);
    }
    if (tid == 0) {
        s_end[nR] = 0x7fffffff;
    }
    for (int j = tid; j < nE; j += kThreads) {
        int64_t c;
        if constexpr (kIdentity) {
            c = a0 + j;
        } else {
            c = OPSGNN_GUARD(3, a0 + j, p.nnz) ? static_cast<int64_t>(LoadStream(static_cast<const ColT*>(p.col) + a0 + j)) : 0;
        }
        c = c < 0 ? 0 : (c >= p.src_rows ? p.src_rows - 1 : c);  // validated upstream; never fault on a bad index
        s_col[j] = static_cast<int32_t>(c);
        if constexpr (!GENERAL) {
            s_val[j] = p.has_val ? Widen<A, T>(LoadStream(val + a0 + j)) : A(1);
        } else if constexpr (!BULK) {
            if (p.has_val && p.wide == 0) {
                s_val[j] = Widen<A, T>(LoadStream(val + a0 + j));
            }
        }
    }
    __syncthreads();
    if (tid <= kWarps) {
        int diag = tid * kItemsPerWarp;
        diag = diag < nR + nE ? diag : nR + nE;
        int lo = diag > nE ? diag - nE : 0;
        int hi = diag < nR ? diag : nR;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (s_end[mid] <= diag - 1 - mid) {
                lo = mid + 1;
            } else {
                hi = mid;
            }
        }
        s_split[tid] = lo;
    }
    __syncthreads();

    // ---- bulk ring of this warp ------------------------------------------------------------------------------------
    extern __shared__ __align__(128) unsigned char dyn_smem[];
    unsigned char* ring = dyn_smem + (BULK ? warp * kBulkWarpBytes : 0);
    const uint32_t ring_addr = BULK ? SharedAddress(ring) : 0u;
    const uint32_t bar_addr = BULK ? SharedAddress(dyn_smem + kWarps * kBulkWarpBytes + warp * kBulkStages * 8) : 0u;
    // weighted bulk instance: [stage][edge][weight] behind the barriers, kBulkWeightBytes per stage
    const T* weight_ring = reinterpret_cast<const T*>(dyn_smem + kWarps * kBulkWarpBytes + kWarps * kBulkStages * 8 +
                                                      ((GENERAL && BULK) ? warp * kBulkStages * kBulkWeightBytes : 0));
    const uint32_t weight_addr = (GENERAL && BULK) ? SharedAddress(weight_ring) : 0u;
    const uint32_t weight_row_bytes = static_cast<uint32_t>(p.val_width * static_cast<int64_t>(sizeof(T)));
    constexpr bool kAttention = GENERAL && BULK && std::is_same<T, float>::value && RK == kSum;
    if constexpr (BULK && !kRingAsync) {
        if (lane == 0) {
#pragma unroll
            for (int st = 0; st < kBulkStages; ++st) {
                MbarInit(bar_addr + st * 8, 1);
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
    }

    auto carry_of = [&](int w) -> A* {
        if constexpr (BULK) {
            return reinterpret_cast<A*>(dyn_smem + w * kBulkWarpBytes);
        } else {
            return s_carry_static[w];
        }
    };
    auto carry_arg_of = [&](int w) -> int64_t* {
        if constexpr (BULK) {
            return reinterpret_cast<int64_t*>(dyn_smem + w * kBulkWarpBytes + 2048);
        } else {
            return s_carry_arg_static[w];
        }
    };

    // ---- per-warp walk ---------------------------------------------------------------------------------------
    int dw0 = warp * kItemsPerWarp;
    int dw1 = dw0 + kItemsPerWarp;
    dw0 = dw0 < nR + nE ? dw0 : nR + nE;
    dw1 = dw1 < nR + nE ? dw1 : nR + nE;
    int i = s_split[warp];
    const int i1 = s_split[warp + 1];
    int j = dw0 - i;
    const int j1 = dw1 - i1;

    // feature offsets owned by this lane: vector v covers [koff[v], koff[v] + VEC)
    bool live[NV];
    int64_t koff[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        koff[v] = kbase + static_cast<int64_t>(v * 32 + lane_in) * VEC;
        live[v] = BULK || koff[v] < K;  // the bulk variant is only launched when the tiles cover K exactly
    }

    // Per-lane row bases: a gathered vector is lane_base[v] + col * K, one 32x32->64 multiply-add per load.
    const int K32 = static_cast<int>(K);
    const T* lane_base[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        lane_base[v] = mat + koff[v];
    }

    int64_t group_of[NV];  // wide == 2: weight slot of each owned vector
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        group_of[v] = p.wide == 2 ? koff[v] / p.val_group : 0;
    }

    A acc[ELEMS];
    A aux[RK == kLogSumExp ? ELEMS : 1];       // sum of exponentials
    int where[kHasArg ? ELEMS : 1];            // selected edge as an index into the block's staged edges, -1 for none
    const A seed = (RK == kExtremum) ? ExtremumSeed<A, T>(p.is_min, p.extremum) : A(0);
    auto reset = [&]() {
#pragma unroll
        for (int q = 0; q < ELEMS; ++q) {
            if constexpr (RK == kLogSumExp) {
                acc[q] = -INFINITY;
                aux[q] = 0;
            } else {
                acc[q] = seed;
            }
            if constexpr (kHasArg) {
                where[q] = -1;
            }
        }
    };
    reset();
    bool dirty = false;

    // Narrow layout: fold the lane groups' partial results into every group (xor butterfly, the same value in all).
    auto merge_groups = [&]() {
        if constexpr (NARROW) {
            for (int off = lpg; off < 32; off <<= 1) {
#pragma unroll
                for (int q = 0; q < ELEMS; ++q) {
                    if constexpr (RK == kSum) {
                        acc[q] += ShuffleXor(acc[q], off);
                    } else if constexpr (RK == kLogSumExp) {
                        const A other_max = ShuffleXor(acc[q], off);
                        const A other_sum = ShuffleXor(aux[q], off);
                        LseMerge(acc[q], aux[q], other_max, other_sum);
                    } else {
                        const A other = ShuffleXor(acc[q], off);
                        const int other_arg = ShuffleXor(where[q], off);
                        ExtremumMerge<A, int>(acc[q], where[q], other, other_arg, p.is_min, p.extremum);
                    }
                }
            }
        }
    };

    auto flush = [&](int local_row) {
        const int64_t row = row0 + local_row;
        merge_groups();
        A scale = A(1);
        bool divide = false;
        if constexpr (RK == kSum) {
            if (p.mean) {
                const int64_t degree = static_cast<int64_t>(ptr[row + 1]) - static_cast<int64_t>(ptr[row]);
                if (degree > 0) {
                    scale = static_cast<A>(degree);
                    divide = true;
                }
            }
        }
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            if (!live[v] || grp != 0) {
                continue;
            }
            A finished[VEC];
            Pack<int64_t, VEC> packed_arg;
#pragma unroll
            for (int c = 0; c < VEC; ++c) {
                A value = acc[v * VEC + c];
                if constexpr (RK == kSum) {
                    if (divide) {
                        value = value / scale;
                    }
                } else if constexpr (RK == kLogSumExp) {
                    value = LseFinish(value, aux[v * VEC + c]);
                } else {
                    const int w = where[v * VEC + c];
                    if (w < 0) {
                        value = A(0);
                    }
                    packed_arg.v[c] = w < 0 ? p.arg_none : a0 + w;
                }
                finished[c] = value;
            }
            const Pack<O, VEC> packed = Repack<O, A, VEC>(finished);
            const int64_t at = row * K + koff[v];
            if (!OPSGNN_GUARD(5, at + VEC - 1, p.rows * K)) {
                continue;
            }
            if constexpr (sizeof(O) * VEC == 32) {
                StoreStream<O, VEC / 2>(out + at, *reinterpret_cast<const Pack<O, VEC / 2>*>(&packed.v[0]));
                StoreStream<O, VEC / 2>(out + at + VEC / 2,
                                        *reinterpret_cast<const Pack<O, VEC / 2>*>(&packed.v[VEC / 2]));
            } else {
                StoreStream<O, VEC>(out + at, packed);
            }
            if constexpr (kHasArg) {
#pragma unroll
                for (int c = 0; c < VEC; c += 2) {
                    if constexpr (VEC >= 2) {
                        StoreStream<int64_t, 2>(arg + at + c, *reinterpret_cast<Pack<int64_t, 2>*>(&packed_arg.v[c]));
                    } else {
                        arg[at] = packed_arg.v[0];
                    }
                }
            }
        }
    };

    // Edges are gathered EB at a time regardless of row boundaries, so short rows do not shrink the number of loads in
    // flight; the batch is then consumed run by run, one run per row that owns part of it.  Every branch below is
    // uniform across the warp.
    // Bulk path: batch b of this warp (edges j0 + b*EB ...) is copied into stage b % kBulkStages.
    const int j0 = j;
    const uint32_t seg_bytes =
        static_cast<uint32_t>((K - kbase < TILE ? K - kbase : static_cast<int64_t>(TILE)) * static_cast<int64_t>(sizeof(T)));
    auto issue = [&](int b) {
        const int first = j0 + b * eb;
        if constexpr (kRingAsync) {
            // One commit group per batch, empty ones included, so "all but the newest kBulkStages - 1 groups" always
            // means "every batch up to the one about to be consumed".
            const int n = (first >= j1) ? 0 : ((j1 - first < eb) ? j1 - first : eb);
            const uint32_t stage_addr = ring_addr + static_cast<uint32_t>((b % kBulkStages) * kBulkStageBytes);
            for (int rr = 0; rr < n; rr += groups) {
                const int r = rr + grp;
                if (r < n) {
                    AsyncCopy16(stage_addr + static_cast<uint32_t>(r * row_bytes + lane_in * 16),
                                lane_base[0] + static_cast<int64_t>(s_col[first + r]) * K32);
                }
            }
            AsyncCommit();
            return;
        }
        if (first >= j1) {
            return;
        }
        const int n = (j1 - first < eb) ? j1 - first : eb;
        const int st = b % kBulkStages;
        const bool leader = lane == 0;
        if (leader) {
            if constexpr (GENERAL) {
                MbarExpectTx(bar_addr + st * 8, static_cast<uint32_t>(n) * (seg_bytes + weight_row_bytes));
                BulkLoad(weight_addr + static_cast<uint32_t>(st * kBulkWeightBytes), val + (a0 + first) * p.val_width,
                         static_cast<uint32_t>(n) * weight_row_bytes, bar_addr + st * 8);
            } else {
                MbarExpectTx(bar_addr + st * 8, static_cast<uint32_t>(n) * seg_bytes);
            }
        }
        if constexpr (kIdentity) {
            // Consecutive source rows: when a row segment is the whole row, the stage is one contiguous copy.
            if (p.tiles_per_batch == 1 && a0 + first + n <= p.src_rows) {
                if (leader) {
                    BulkLoad(ring_addr + static_cast<uint32_t>(st * kBulkStageBytes), mat + (a0 + first) * K,
                             static_cast<uint32_t>(n) * seg_bytes, bar_addr + st * 8);
                }
                return;
            }
        }
        // Lanes 0 .. n - 1 issue one copy each.  (One elected lane issuing the stage's copies in a row measured slower:
        // F = 256 fp32 37.2 against 34.3 ms, bf16 26.0 against 23.7 ms, 12 more warp instructions per edge.)
        for (int r = lane; r < n; r += 32) {
            if (OPSGNN_GUARD(4, static_cast<int64_t>(s_col[first + r]) * K + kbase + TILE - 1, p.src_rows * K + TILE)) {
                BulkLoad(ring_addr + static_cast<uint32_t>(st * kBulkStageBytes + r * row_bytes),
                         mat + (static_cast<int64_t>(s_col[first + r]) * K32 + kbase), seg_bytes, bar_addr + st * 8);
            }
        }
    };
    // Attention mode: the log-sum-exp of the current row for this lane's feature groups.
    float att_norm[NV];
    int att_row = -1;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        att_norm[v] = 0.0f;
    }
    int batch_id = 0;
    bool stalled = false;
    if constexpr (BULK) {
#pragma unroll
        for (int st = 0; st < kBulkStages; ++st) {
            issue(st);
        }
    }
    while (j < j1 || i < i1) {
        const int nb = (j1 - j < eb) ? j1 - j : eb;
        Pack<T, VEC> x[BULK ? 1 : EB][NV];
        const unsigned char* stage = ring + (batch_id % kBulkStages) * kBulkStageBytes;
        if constexpr (BULK && kRingAsync) {
            if (nb > 0) {
                AsyncWait<kBulkStages - 1>();
                __syncwarp();  // a row is read by other lanes than the ones that copied it
            }
        } else if constexpr (BULK) {
            if (nb > 0) {
                const uint32_t bar = bar_addr + (batch_id % kBulkStages) * 8;
                const uint32_t parity = static_cast<uint32_t>(batch_id / kBulkStages) & 1u;
                // At most p.wait_polls polls (each may sleep up to kBulkWaitHintNs); zero polls gives up at once, which
                // is how the error path is exercised without a copy that never lands.
                stalled = true;
                for (uint32_t spins = 0; spins < p.wait_polls; ++spins) {
                    if (MbarTryWait(bar, parity)) {
                        stalled = false;
                        break;
                    }
                }
                stalled = __any_sync(0xffffffffu, stalled);  // one verdict per warp: lanes poll independently
                if (stalled) {  // never expected: report it and leave instead of hanging
                    if (lane == 0) {
                        atomicAdd(p.status, 1ULL);
                        if (p.status_sink != nullptr) {
                            *reinterpret_cast<volatile unsigned long long*>(p.status_sink) = 1ULL;
                            __threadfence_system();
                        }
                    }
                    break;
                }
            }
        } else {
#pragma unroll
            for (int t = 0; t < EB; ++t) {
                if (t < nb) {
                    const int column = s_col[j + t];
#pragma unroll
                    for (int v = 0; v < NV; ++v) {
                        if (live[v] && OPSGNN_GUARD(4, static_cast<int64_t>(s_col[j + t]) * K + koff[v] + VEC - 1, p.src_rows * K)) {
                            x[t][v] = LoadGather<T, VEC>(lane_base[v] + static_cast<int64_t>(column) * K32);
                        }
                    }
                }
            }
        }
        int t_begin = 0;
        for (;;) {
            int t_end = nb;
            bool row_ends = false;
            if (i < i1) {
                const int rel = s_end[i] - j;
                t_end = rel < nb ? rel : nb;
                row_ends = rel <= nb || nb == 0;  // nb == 0: only row ends are left, always make progress
            }
            // One gathered edge (slot t of the batch) folded into the accumulators; t is a compile-time constant so
            // the batch registers are indexed statically.
            auto consume = [&](auto slot, auto rule_c) {
                constexpr int kRule = decltype(rule_c)::value;  // the extremum rule, fixed per copy of the loop body
                const int t = static_cast<int>(slot);  // compile-time for the register path, run-time for the ring
                {
                    const int e = j + t;
                    A w = A(1);
                    if constexpr (!GENERAL) {
                        w = s_val[e];  // staged as 1 when the call has no weights
                    } else if constexpr (!BULK) {
                        if (p.has_val && p.wide == 0) {
                            w = s_val[e];
                        }
                    }
#pragma unroll
                    for (int v = 0; v < NV; ++v) {
                        if (!live[v]) {
                            continue;
                        }
                        Pack<T, VEC> wv;
                        if constexpr (GENERAL && BULK) {  // one weight per (edge, feature group), staged with the rows
                            w = Widen<A, T>(weight_ring[(batch_id % kBulkStages) * (kBulkWeightBytes / static_cast<int>(sizeof(T))) +
                                                        t * static_cast<int>(p.val_width) + static_cast<int>(group_of[v])]);
                            if constexpr (kAttention) {
                                if (p.attention) {  // the staged value is the edge's logit
                                    w = static_cast<A>(__expf(static_cast<float>(w) - att_norm[v]));
                                }
                            }
                        } else if constexpr (GENERAL) {
                            if (p.wide == 1) {
                                wv = LoadGather<T, VEC>(val + (a0 + e) * K + koff[v]);
                            } else if (p.wide == 2) {
                                w = Widen<A, T>(LoadNc(val + (a0 + e) * p.val_width + group_of[v]));
                            }
                        }
                        A xs[VEC];
                        if constexpr (BULK) {
                            const Pack<T, VEC> staged = LoadPlain<T, VEC>(
                                reinterpret_cast<const T*>(stage + t * row_bytes) + (v * 32 + lane_in) * VEC);
                            Unpack<A, T, VEC>(staged, xs);
                        } else {
                            Unpack<A, T, VEC>(x[decltype(slot)::value][v], xs);
                        }
                        A ws[VEC];
                        if constexpr (GENERAL) {
                            if (p.wide == 1) {
                                Unpack<A, T, VEC>(wv, ws);
                            }
                        }
                        if constexpr (kPackedFma) {
                            // Two products per instruction (fma.rn.f32x2): the same rounding as the scalar form.
#pragma unroll
                            for (int c = 0; c < VEC; c += 2) {
                                const int q = v * VEC + c;
                                float w0 = w, w1 = w;
                                if constexpr (GENERAL) {
                                    if (p.wide == 1) {
                                        w0 = ws[c];
                                        w1 = ws[c + 1];
                                    }
                                }
                                const float2 sum = __ffma2_rn(make_float2(w0, w1), make_float2(xs[c], xs[c + 1]),
                                                              make_float2(acc[q], acc[q + 1]));
                                acc[q] = sum.x;
                                acc[q + 1] = sum.y;
                            }
                        } else {
#pragma unroll
                        for (int c = 0; c < VEC; ++c) {
                            const int q = v * VEC + c;
                            A value = xs[c];
                            if constexpr (GENERAL) {
                                if (p.wide == 1) {
                                    w = ws[c];
                                }
                            }
                            if constexpr (RK == kSum) {
                                acc[q] += w * value;
                            } else if constexpr (RK == kExtremum) {
                                value = value * w;  // w == 1 leaves every value, NaN and infinity included, as it is
                                ExtremumOffer<A, int>(acc[q], where[q], value, e, p.is_min, kRule);
                            } else {
                                LseOffer(acc[q], aux[q], value);
                            }
                        }
                        }
                    }
                }
            };
            // Slots [t_begin, t_end) belong to the current row: jump to the first one and fall through until the
            // run ends, so a batch that spans several rows is not rescanned slot by slot for each of them.
#define OPSGNN_SLOT(N)                                             \
    case N:                                                        \
        if constexpr (N < EB) {                                    \
            if (N >= t_end) {                                      \
                break;                                             \
            }                                                      \
            consume(std::integral_constant<int, N>{}, rule_c);     \
        }
            if constexpr (kAttention) {
                if (p.attention && t_end > t_begin && att_row != i) {  // first edges of a new row in this warp
                    att_row = i;
                    const int64_t at = (row0 + i) * p.val_width;
#pragma unroll
                    for (int v = 0; v < NV; ++v) {
                        att_norm[v] = __ldg(p.att_lse + at + group_of[v]);
                    }
                }
            }
            if constexpr (RK == kLogSumExp && BULK) {
                // The run sits in shared memory, so it is read twice: once for the maximum of the run, once for the
                // sum of exponentials against the updated maximum.  One exponential and no branch per element; the
                // running sum is rescaled once per run.  fmaxf drops NaN, which then enters the sum as exp(NaN).
                A run_max[ELEMS];
#pragma unroll
                for (int q = 0; q < ELEMS; ++q) {
                    run_max[q] = -INFINITY;
                }
                for (int tt = t_begin; tt < t_end; tt += groups) {
                    if (tt + grp < t_end) {
#pragma unroll
                        for (int v = 0; v < NV; ++v) {
                            A xs[VEC];
                            Unpack<A, T, VEC>(LoadPlain<T, VEC>(reinterpret_cast<const T*>(stage + (tt + grp) * row_bytes) +
                                                                (v * 32 + lane_in) * VEC), xs);
#pragma unroll
                            for (int c = 0; c < VEC; ++c) {
                                run_max[v * VEC + c] = fmaxf(run_max[v * VEC + c], xs[c]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int q = 0; q < ELEMS; ++q) {
                    const A top = fmaxf(acc[q], run_max[q]);
                    if (top != acc[q]) {  // never taken for equal infinities, so no inf - inf
                        aux[q] *= __expf(acc[q] - top);
                        acc[q] = top;
                    }
                }
                for (int tt = t_begin; tt < t_end; tt += groups) {
                    if (tt + grp < t_end) {
#pragma unroll
                        for (int v = 0; v < NV; ++v) {
                            A xs[VEC];
                            Unpack<A, T, VEC>(LoadPlain<T, VEC>(reinterpret_cast<const T*>(stage + (tt + grp) * row_bytes) +
                                                                (v * 32 + lane_in) * VEC), xs);
#pragma unroll
                            for (int c = 0; c < VEC; ++c) {
                                const int q = v * VEC + c;
                                aux[q] += __expf(xs[c] == acc[q] ? A(0) : xs[c] - acc[q]);
                            }
                        }
                    }
                }
            } else {
            // The run is folded by one copy of the loop body per extremum rule (the rule is uniform over the launch), so
            // the per-element update compiles against a constant rule instead of testing it for every element.
            auto fold_run = [&](auto rule_c) {
            if constexpr (NARROW) {
                for (int tt = t_begin; tt < t_end; tt += groups) {
                    if (tt + grp < t_end) {
                        consume(tt + grp, rule_c);
                    }
                }
            } else if constexpr (BULK && EB > 4) {
                for (int t = t_begin; t < t_end; ++t) {
                    consume(t, rule_c);
                }
            } else {
            switch (t_begin) {  // register path and four-row bulk stages: slots are compile-time, offsets immediates (six-row stages measured slower this way: bf16 F = 256 25.2 against 23.5 ms)
                OPSGNN_SLOT(0)
                OPSGNN_SLOT(1)
                OPSGNN_SLOT(2)
                OPSGNN_SLOT(3)
                OPSGNN_SLOT(4)
                OPSGNN_SLOT(5)
                OPSGNN_SLOT(6)
                OPSGNN_SLOT(7)
                OPSGNN_SLOT(8)
                OPSGNN_SLOT(9)
                OPSGNN_SLOT(10)
                OPSGNN_SLOT(11)
                OPSGNN_SLOT(12)
                OPSGNN_SLOT(13)
                OPSGNN_SLOT(14)
                OPSGNN_SLOT(15)
                default:
                    break;
            }
            }
            };
            if constexpr (RK == kExtremum) {
                switch (p.extremum) {
                    case OPSGNN_EXTREMUM_IGNORE_NAN:
                        fold_run(std::integral_constant<int, OPSGNN_EXTREMUM_IGNORE_NAN>{});
                        break;
                    case OPSGNN_EXTREMUM_PROPAGATE_NAN:
                        fold_run(std::integral_constant<int, OPSGNN_EXTREMUM_PROPAGATE_NAN>{});
                        break;
                    case OPSGNN_EXTREMUM_SEEDED:
                        fold_run(std::integral_constant<int, OPSGNN_EXTREMUM_SEEDED>{});
                        break;
                    default:
                        fold_run(std::integral_constant<int, OPSGNN_EXTREMUM_SEEDED_LAST>{});
                        break;
                }
            } else {
                fold_run(std::integral_constant<int, 0>{});
            }
            }
#undef OPSGNN_SLOT
            if (t_end > t_begin) {
                dirty = true;
            }
            t_begin = t_end;
            if (!row_ends) {
                break;
            }
            flush(i);
            reset();
            dirty = false;
            ++i;
        }
        j += nb;
        if constexpr (BULK) {
            if (nb > 0) {
                __syncwarp();  // every lane has read its part of the stage before the stage is refilled
                issue(batch_id + kBulkStages);
                ++batch_id;
            }
        }
    }
    if constexpr (BULK && kRingAsync) {
        AsyncWait<0>();  // nothing is outstanding by construction; the ring is about to hold the carries
    } else if constexpr (BULK) {
        if (stalled) {
            // Give copies still in flight a bounded chance to land before the block's shared memory is released.
            for (int b = batch_id; b < batch_id + kBulkStages; ++b) {
                if (j0 + b * eb < j1) {
                    uint32_t spins = 0;
                    while (!MbarTryWait(bar_addr + (b % kBulkStages) * 8, static_cast<uint32_t>(b / kBulkStages) & 1u) &&
                           ++spins <= kBulkSpinLimit) {
                    }
                }
            }
        }
    }

    // ---- carries -------------------------------------------------------------------------------------------------
    if (lane == 0) {
        s_carry_row[warp] = dirty ? i1 : -1;
    }
    if (dirty) {
        merge_groups();
    }
    if (dirty && grp == 0) {
#pragma unroll
        for (int v = 0; v < NV; ++v) {
#pragma unroll
            for (int c = 0; c < VEC; ++c) {
                const int q = v * VEC + c;
                const int f = (v * 32 + lane_in) * VEC + c;
                if constexpr (RK == kLogSumExp) {
                    carry_of(warp)[f] = LseFinish(acc[q], aux[q]);
                } else {
                    carry_of(warp)[f] = acc[q];
                }
                if constexpr (kHasArg) {
                    carry_arg_of(warp)[f] = where[q] < 0 ? int64_t(-1) : a0 + where[q];
                }
            }
        }
    }
    __syncthreads();

    bool any = false;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        any |= s_carry_row[w] >= 0;
    }
    if (tid == 0 && blockIdx.y == 0) {
        bool leaves = false;  // a carry whose row ends in a later block
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            leaves |= s_carry_row[w] >= nR && s_carry_row[w] >= 0;
        }
        p.carry_row[cta] = leaves ? row0 + nR : -1;
    }
    if (!any) {
        return;
    }
    A* __restrict__ carry_val = static_cast<A*>(p.carry_val) + cta * p.carry_stride + static_cast<int64_t>(blockIdx.y) * TILE;
    int64_t* __restrict__ carry_arg =
        kHasArg ? p.carry_arg + cta * p.carry_stride + static_cast<int64_t>(blockIdx.y) * TILE : nullptr;

    for (int f = tid; f < TILE; f += kThreads) {
        const int64_t k = kbase + f;
        if (k >= K) {
            continue;
        }
        int run_row = -1;
        A run_acc = A(0);
        int64_t run_arg = -1;
        auto apply = [&]() {
            if (run_row < 0) {
                return;
            }
            if (run_row >= nR) {  // the row ends in a later block
                if (!OPSGNN_GUARD(6, cta * p.carry_stride + static_cast<int64_t>(blockIdx.y) * TILE + f,
                                  p.num_cta * p.carry_stride)) {
                    return;
                }
                carry_val[f] = run_acc;
                if constexpr (kHasArg) {
                    carry_arg[f] = run_arg;
                }
                return;
            }
            const int64_t row = row0 + run_row;
            const int64_t at = row * K + k;
            if (!OPSGNN_GUARD(7, at, p.rows * K)) {
                return;
            }
            if constexpr (RK == kSum) {
                A add = run_acc;
                if (p.mean) {
                    const int64_t degree = static_cast<int64_t>(ptr[row + 1]) - static_cast<int64_t>(ptr[row]);
                    if (degree > 0) {
                        add = add / static_cast<A>(degree);
                    }
                }
                out[at] = Narrow<O, A>(add + Widen<A, O>(out[at]));
            } else if constexpr (RK == kLogSumExp) {
                out[at] = Narrow<O, A>(LogAddExp(run_acc, Widen<A, O>(out[at])));
            } else {
                const int64_t tail_arg = arg[at];
                if (tail_arg != p.arg_none || run_arg >= 0) {
                    A best = run_acc;
                    int64_t best_arg = run_arg;
                    if (tail_arg != p.arg_none) {
                        ExtremumOffer<A>(best, best_arg, Widen<A, O>(out[at]), tail_arg, p.is_min, p.extremum);
                    }
                    if (best_arg >= 0) {
                        out[at] = Narrow<O, A>(best);
                        arg[at] = best_arg;
                    }
                }
            }
        };
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const int r = s_carry_row[w];
            if (r < 0) {
                continue;
            }
            const A value = carry_of(w)[f];
            if (r != run_row) {
                apply();
                run_row = r;
                run_acc = value;
                if constexpr (kHasArg) {
                    run_arg = carry_arg_of(w)[f];
                }
            } else if constexpr (RK == kSum) {
                run_acc += value;
            } else if constexpr (RK == kLogSumExp) {
                run_acc = LogAddExp(run_acc, value);
            } else {
                const int64_t a = carry_arg_of(w)[f];
                if (a >= 0) {
                    ExtremumOffer<A>(run_acc, run_arg, value, a, p.is_min, p.extremum);
                }
            }
        }
        apply();
    }
}

// ---- cross-block carries ---------------------------------------------------------------------------------------
// One warp per block index: the first block of a run of equal carry rows sums the run in block order and patches
// the row, so the result does not depend on scheduling.
template <class T, class O, class PtrT, int RK>
__global__ void __launch_bounds__(kThreads) FixupKernel(const Params p)
{
    using A = typename AccOf<T>::type;
    constexpr bool kHasArg = RK == kExtremum;
    const int lane = threadIdx.x & 31;
    const int64_t b = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    if (b >= p.num_cta) {
        return;
    }
    const int64_t row = p.carry_row[b];
    if (row < 0 || row >= p.rows || (b > 0 && p.carry_row[b - 1] == row)) {
        return;
    }
    const PtrT* __restrict__ ptr = static_cast<const PtrT*>(p.ptr);
    const A* __restrict__ carry_val = static_cast<const A*>(p.carry_val);
    const int64_t K = p.feat;
    const int64_t tile = p.carry_stride / (p.tiles_per_batch * p.batches);
    A scale = A(1);
    bool divide = false;
    if (RK == kSum && p.mean) {
        const int64_t degree = static_cast<int64_t>(ptr[row + 1]) - static_cast<int64_t>(ptr[row]);
        if (degree > 0) {
            scale = static_cast<A>(degree);
            divide = true;
        }
    }
    const int64_t width = p.batches * K;
    // Four features per lane when one batch, float accumulators and aligned rows allow it (the SpMM / segment sums):
    // the loop is a chain of dependent loads, so fewer and wider steps are what shortens it.
    if constexpr ((RK == kSum || RK == kLogSumExp) && std::is_same<A, float>::value && sizeof(O) >= 2) {
        if (p.batches == 1 && K % 4 == 0 && p.carry_stride % 4 == 0 &&
            ((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(carry_val)) & 15) == 0) {
            O* out = static_cast<O*>(p.out);
            for (int64_t k = static_cast<int64_t>(lane) * 4; k < K; k += 128) {
                // tiles are padded to `tile` features inside a carry row; K % 4 == 0 keeps a vector inside one tile
                const int64_t f = (k / tile) * tile + k % tile;
                float run[4];
                Unpack<float, float, 4>(LoadPlain<float, 4>(carry_val + b * p.carry_stride + f), run);
                for (int64_t n = b + 1; n < p.num_cta && p.carry_row[n] == row; ++n) {
                    float more[4];
                    Unpack<float, float, 4>(LoadPlain<float, 4>(carry_val + n * p.carry_stride + f), more);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        run[c] = RK == kSum ? run[c] + more[c] : LogAddExp(run[c], more[c]);
                    }
                }
                float old[4];
                Unpack<float, O, 4>(LoadPlain<O, 4>(out + row * K + k), old);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if constexpr (RK == kSum) {
                        old[c] = (divide ? run[c] / scale : run[c]) + old[c];
                    } else {
                        old[c] = LogAddExp(run[c], old[c]);
                    }
                }
                StorePlain<O, 4>(out + row * K + k, Repack<O, float, 4>(old));
            }
            return;
        }
    }
    for (int64_t x = lane; x < width; x += 32) {
        const int64_t batch = x / K;
        const int64_t k = x - batch * K;
        // position of feature k of this batch inside a carry row: tiles are padded to `tile` features
        const int64_t f = (batch * p.tiles_per_batch + k / tile) * tile + k % tile;
        A run_acc = carry_val[b * p.carry_stride + f];
        int64_t run_arg = kHasArg ? p.carry_arg[b * p.carry_stride + f] : 0;
        for (int64_t n = b + 1; n < p.num_cta && p.carry_row[n] == row; ++n) {
            const A value = carry_val[n * p.carry_stride + f];
            if constexpr (RK == kSum) {
                run_acc += value;
            } else if constexpr (RK == kLogSumExp) {
                run_acc = LogAddExp(run_acc, value);
            } else {
                const int64_t a = p.carry_arg[n * p.carry_stride + f];
                if (a >= 0) {
                    ExtremumOffer<A>(run_acc, run_arg, value, a, p.is_min, p.extremum);
                }
            }
        }
        O* out = static_cast<O*>(p.out);
        const int64_t at = (batch * p.rows + row) * K + k;
        if constexpr (RK == kSum) {
            if (divide) {
                run_acc = run_acc / scale;
            }
            out[at] = Narrow<O, A>(run_acc + Widen<A, O>(out[at]));
        } else if constexpr (RK == kLogSumExp) {
            out[at] = Narrow<O, A>(LogAddExp(run_acc, Widen<A, O>(out[at])));
        } else {
            const int64_t tail_arg = p.arg[at];
            if (tail_arg != p.arg_none) {
                ExtremumOffer<A>(run_acc, run_arg, Widen<A, O>(out[at]), tail_arg, p.is_min, p.extremum);
            }
            if (run_arg >= 0) {
                out[at] = Narrow<O, A>(run_acc);
                p.arg[at] = run_arg;
            }
        }
    }
}

// ---- host-side launch ----------------------------------------------------------------------------------------
template <class T, class O, class PtrT, class ColT, int VEC, int NV, int RK, bool GENERAL = true, bool BULK = false,
          bool NARROW = false>
int Launch(Params p, cudaStream_t stream)
{
    constexpr int TILE = 32 * VEC * NV;
    p.tiles_per_batch = static_cast<int>(CeilDiv(p.feat, TILE));
    const int64_t grid_y = p.tiles_per_batch * p.batches;
    if (grid_y > 65535 || p.num_cta > 2147483647LL) {
        return OPSGNN_ERR_LIMIT;
    }
    p.carry_stride = grid_y * TILE;
    const dim3 grid(static_cast<unsigned>(p.num_cta), static_cast<unsigned>(grid_y));
    auto kernel = ReduceKernel<T, O, PtrT, ColT, VEC, NV, RK, GENERAL, BULK, NARROW>;
    const size_t dynamic = BULK ? (GENERAL ? kBulkSmemBytesWeighted : kBulkSmemBytes) : 0;
    if (BULK) {
        static bool configured[64] = {false};  // per device and instance: opt in to more than 48 KiB of dynamic shared memory
        int device = 0;
        OPSGNN_CUDA_TRY(cudaGetDevice(&device));
        if (device >= 0 && device < 64 && !configured[device]) {
            OPSGNN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(dynamic)));
            configured[device] = true;
        }
    }
    kernel<<<grid, kThreads, dynamic, stream>>>(p);
    int status = LaunchStatus();
    if (status != OPSGNN_OK) {
        return status;
    }
    const unsigned fix_grid = static_cast<unsigned>(CeilDiv(p.num_cta, kWarps));
    FixupKernel<T, O, PtrT, RK><<<fix_grid, kThreads, 0, stream>>>(p);
    return LaunchStatus();
}

// Picks the lane layout: 16-byte vectors when the feature width and base addresses allow it.
template <class T, class O, class PtrT, class ColT, int RK>
int LaunchShaped(const Params& p, cudaStream_t stream)
{
    constexpr int kVec = 16 / sizeof(T);
    const bool vector_ok = sizeof(T) <= 4 && sizeof(T) >= 2 && p.feat % kVec == 0 && Aligned(p.mat, 16) && Aligned(p.out, 16) &&
                           (p.wide != 1 || Aligned(p.val, 16)) && (p.wide != 2 || p.val_group % kVec == 0) &&
                           (RK != kExtremum || Aligned(p.arg, 16));
    const bool lean = p.wide == 0;  // no weights or one per edge: the instance without per-feature weight code
    // Bulk-copy gathers for the lean instances (the hot SpMM / segment paths); OPSGNN_NO_BULK=1 keeps the register
    // gathers for comparison runs.
    static const bool bulk_allowed = std::getenv("OPSGNN_NO_BULK") == nullptr;
    const bool bulk = lean && bulk_allowed;
    if constexpr (sizeof(T) == 4 || sizeof(T) == 2) {
        // Rows of 16 to 256 bytes (a power of two): several edges per warp instruction instead of idle lanes.  (512-byte
        // rows through the same per-lane asynchronous copies measured slower than the bulk ring: bf16 F = 256 29.5
        // against 23.7 ms, 91 against 68 warp instructions per edge.)
        const int64_t vectors = p.feat / kVec;
        if (bulk && vector_ok && vectors >= 1 && vectors <= 16 && (vectors & (vectors - 1)) == 0) {
            Params narrow = p;
            narrow.lanes_per_row = static_cast<int>(vectors);
            return Launch<T, O, PtrT, ColT, kVec, 1, RK, false, true, true>(narrow, stream);
        }
    }
    // One weight per (edge, feature group): bulk gathers with the weights staged beside the rows, when a stage's
    // weights fit their slot and every copy is 16-byte aligned.
    auto weighted_bulk = [&](int tile, int rows_per_stage) {
        const int64_t row_bytes = p.val_width * static_cast<int64_t>(sizeof(T));
        return bulk_allowed && p.wide == 2 && RK == kSum && vector_ok && p.feat % tile == 0 && Aligned(p.val, 16) &&
               row_bytes % 16 == 0 && rows_per_stage * row_bytes <= kBulkWeightBytes;
    };
    constexpr bool kIdentity = std::is_same<ColT, Identity>::value;  // segment calls never carry per-feature weights
    if constexpr (!kIdentity && RK == kSum && sizeof(T) == 4) {
        if (weighted_bulk(256, kBulkStageBytes / 1024)) {
            return Launch<T, O, PtrT, ColT, 4, 2, RK, true, true>(p, stream);
        }
    } else if constexpr (!kIdentity && RK == kSum && sizeof(T) == 2) {
        if (weighted_bulk(256, kBulkStageBytes / 512)) {
            return Launch<T, O, PtrT, ColT, 8, 1, RK, true, true>(p, stream);
        }
    }
    // One lane layout: bulk ring when the tiles cover the width exactly, else register gathers (lean or general).
    auto shaped = [&](auto vec, auto nv) {
        constexpr int VEC = decltype(vec)::value;
        constexpr int NV = decltype(nv)::value;
        if (bulk && p.feat % (32 * VEC * NV) == 0) {
            return Launch<T, O, PtrT, ColT, VEC, NV, RK, false, true>(p, stream);
        }
        if constexpr (kIdentity) {
            return Launch<T, O, PtrT, ColT, VEC, NV, RK, false>(p, stream);
        } else {
            return lean ? Launch<T, O, PtrT, ColT, VEC, NV, RK, false>(p, stream)
                        : Launch<T, O, PtrT, ColT, VEC, NV, RK, true>(p, stream);
        }
    };
    if constexpr (sizeof(T) == 4) {
        if (vector_ok && p.feat > 128) {
            return shaped(std::integral_constant<int, 4>{}, std::integral_constant<int, 2>{});
        }
        if (vector_ok) {
            return shaped(std::integral_constant<int, 4>{}, std::integral_constant<int, 1>{});
        }
    } else if constexpr (sizeof(T) == 2) {
        if (vector_ok) {
            return shaped(std::integral_constant<int, 8>{}, std::integral_constant<int, 1>{});
        }
    }
    if constexpr (kIdentity) {
        return Launch<T, O, PtrT, ColT, 1, 4, RK, false>(p, stream);
    } else {
        return Launch<T, O, PtrT, ColT, 1, 4, RK, true>(p, stream);
    }
}

}  // namespace csr
}  // namespace opsgnn
