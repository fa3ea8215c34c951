/*
 * opsgnn_b200.h — C ABI of the B200 (sm_100a) kernels behind the ops_gnn sparse
 * message-passing operators.
 *
 * Every entry point takes raw device pointers, plain sizes and a CUDA stream
 * (passed as void*), enqueues its work on that stream and returns without
 * synchronising.  The return value is 0 on success, a positive cudaError_t when
 * a CUDA call failed, or one of the negative OPSGNN_ERR_* codes when the
 * arguments were rejected before anything was launched.  Nothing throws across
 * this boundary, nothing here allocates device memory: scratch is passed in by
 * the caller and sized by the *_workspace_bytes / *_plan_bytes queries.
 *
 * The citations "replaces <file>:<line>" name the launcher of the reference
 * project (Atlas-Ascend-Fork/ops-gnn, paths relative to its root) that the
 * entry point stands in for.
 */
#ifndef OPSGNN_B200_H
#define OPSGNN_B200_H

#include <stdint.h>

#if defined(__GNUC__)
#define OPSGNN_API __attribute__((visibility("default")))
#else
#define OPSGNN_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define OPSGNN_OK 0
#define OPSGNN_ERR_INVALID (-1)     /* bad shape / null pointer / bad enum     */
#define OPSGNN_ERR_UNSUPPORTED (-2) /* dtype or mode combination not built     */
#define OPSGNN_ERR_WORKSPACE (-3)   /* workspace too small or misaligned       */
#define OPSGNN_ERR_LIMIT (-4)       /* size beyond a documented fixed maximum  */
#define OPSGNN_ERR_TIMEOUT (-5)     /* a bounded device-side wait ran out      */

/* ---- dtype ids (0..4 as csrc/npu/torch_sparse_spmm/op_host/torch_sparse_spmm.cpp:19-36) */
#define OPSGNN_F32 0
#define OPSGNN_F16 1
#define OPSGNN_BF16 2
#define OPSGNN_I8 3
#define OPSGNN_I32 4
#define OPSGNN_I64 5
#define OPSGNN_U8 6
#define OPSGNN_I16 7
#define OPSGNN_F64 8

/* ---- reductions of the CSR engine -------------------------------------- */
#define OPSGNN_REDUCE_SUM 0
#define OPSGNN_REDUCE_MEAN 1
#define OPSGNN_REDUCE_MIN 2
#define OPSGNN_REDUCE_MAX 3
#define OPSGNN_REDUCE_LOGSUMEXP 4

/* ---- extremum rules (who wins, what NaN does) --------------------------- */
/* first edge among ties, NaN never selected, row without a selectable value
 * gives 0 and arg = arg_none (torch_sparse_spmm_kernel.h:56-67). */
#define OPSGNN_EXTREMUM_IGNORE_NAN 0
/* first occurrence among ties, the first NaN wins and sticks (torch.min/max and
 * scatter_reduce_(amin/amax) behaviour used by the segment_csr and spmm goldens). */
#define OPSGNN_EXTREMUM_PROPAGATE_NAN 1
/* strict compare against a +/-finite-max seed: NaN and values not better than
 * the seed never win; an unbeaten seed gives 0 (test/segment_coo/arch35/golden.py:42-58,132-148). */
#define OPSGNN_EXTREMUM_SEEDED 2
/* scatter's rule (test/scatter/arch35/golden.py:85-124, csrc/npu/scatter/op_kernel/arch35/scatter_kernel_minmax.h:116-147):
 * non-strict compare against the +/-finite-max seed, so the LAST edge among ties wins; NaN and values beyond the seed
 * (an infinity on the wrong side) never win; an unbeaten seed gives 0 and arg = arg_none. */
#define OPSGNN_EXTREMUM_SEEDED_LAST 3

OPSGNN_API const char* opsgnn_status_string(int status);
/* Number of SMs of the current device (replaces ResolveAivCoreNum,
 * csrc/npu/common/aiv_launch_utils.h:22-37). */
OPSGNN_API int opsgnn_sm_count(int* count);

/* ======================================================================== */
/* CSR reduce engine: SpMM, segment_csr, segment_coo, segment_logsumexp      */
/* ======================================================================== */

/*
 * out[b, r, k] = reduce over e in [ptr[r], ptr[r+1]) of  w(e,k) * mat[b, col(e), k]
 *
 * col == NULL means col(e) = e (a segment reduction over consecutive rows of
 * mat); val == NULL means w = 1.  The work is split into equal shares of
 * (edges + row ends) by a merge-path plan, so a row with millions of edges is
 * spread over many thread blocks; partial rows are recombined in a fixed order
 * (results are bitwise reproducible).
 */
typedef struct OpsgnnCsrReduceDesc {
    int64_t rows;        /* M: output rows / segments                              */
    int64_t src_rows;    /* N: rows of mat (gather domain)                         */
    int64_t feat;        /* K: features per row                                    */
    int64_t nnz;         /* E: edges; with col == NULL must equal src_rows or less */
    int64_t batches;     /* B: leading batch count of mat/out (>= 1)               */
    int64_t value_width; /* 0 (val NULL), 1 (one weight per edge), K, or a divisor */
                         /* W of K: val is [E, W] and feature k uses val[e, k/(K/W)] */
                         /* (one attention weight per head)                        */
    int64_t arg_none;    /* arg written where no element was selected              */
    int32_t reduce;      /* OPSGNN_REDUCE_*                                        */
    int32_t extremum;    /* OPSGNN_EXTREMUM_* (min/max only)                       */
    int32_t ptr_type;    /* OPSGNN_I32 or OPSGNN_I64: dtype of ptr                 */
    int32_t col_type;    /* OPSGNN_I32 or OPSGNN_I64: dtype of col (ignored if NULL)*/
    int32_t in_type;     /* dtype of mat and val                                   */
    int32_t out_type;    /* dtype of out                                           */
} OpsgnnCsrReduceDesc;

/* Bytes of the merge-path plan for a CSR structure with `rows` rows and `nnz` edges. */
OPSGNN_API int opsgnn_csr_plan_bytes(int64_t rows, int64_t nnz, int64_t* bytes);
/* Builds the plan (one binary search per thread block of the reduce kernel).  It
 * depends on ptr only and may be reused for every call on the same graph. */
OPSGNN_API int opsgnn_csr_plan_build(const void* ptr, int ptr_type, int64_t rows, int64_t nnz, void* plan, void* stream);
/* Bytes of carry scratch needed by opsgnn_csr_reduce for this descriptor. */
OPSGNN_API int opsgnn_csr_reduce_workspace_bytes(const OpsgnnCsrReduceDesc* desc, int64_t* bytes);
/*
 * Replaces TorchSparseSpmm (csrc/npu/torch_sparse_spmm/op_kernel/arch35/torch_sparse_spmm.cpp:38-57),
 * SpmmSum/SpmmMax/SpmmMin and UnifiedSpmm (csrc/npu/common/spmm/spmm_utils.h:156-186,
 * csrc/npu/unified_spmm/op_host/unified_spmm.cpp:116-158), SegmentCsr
 * (csrc/npu/segment_csr/op_kernel/arch35/segment_csr.h:132-139), the reduction half of SegmentCoo
 * (csrc/npu/segment_coo/op_kernel/arch35/segment_coo.h:13-14) and the segment_logsumexp launch
 * (csrc/npu/segment_logsumexp/op_host/segment_logsumexp.cpp:133-168).
 * arg (int64, same shape as out) is required for min/max and ignored otherwise.
 */
OPSGNN_API int opsgnn_csr_reduce(const OpsgnnCsrReduceDesc* desc, const void* ptr, const void* col, const void* val,
                      const void* mat, void* out, int64_t* arg, const void* plan, void* workspace,
                      int64_t workspace_bytes, void* stream);

/*
 * Device-side waits and how a launch reports one that ran out.  The bulk-copy instances of the engine wait on an
 * mbarrier for every stage of gathered rows.  Each wait is bounded (a poll limit, 2^15 polls of up to 100 us by
 * default): a warp whose wait runs out counts itself in the 64-bit status word at the head of the launch's workspace
 * (opsgnn_csr_reduce clears it before the launch), waits - bounded again - for its copies still in flight and returns
 * without writing its remaining rows.  The launch itself always ends; its output is then incomplete.  This is the
 * failure-detection contract the reference states for its device kernels (a device error surfaces as a status the
 * host reads, never as a hang); the reference has no counterpart entry point because its runtime reports through
 * aclrtSynchronizeStream.
 *
 * opsgnn_csr_reduce_status synchronises `stream`, copies the status word of `workspace` to the host and returns
 * OPSGNN_OK when it is zero, OPSGNN_ERR_TIMEOUT otherwise (*stalled_waits = the count).
 */
OPSGNN_API int opsgnn_csr_reduce_status(const void* workspace, void* stream, int64_t* stalled_waits);
/* Registers, for the current device, a second location (device-visible; mapped pinned host memory is the intended
 * use) that a stalled wait also sets to 1, so a host that must not synchronise can poll it between launches.  NULL
 * removes it.  The location must outlive every launch that was enqueued while it was registered. */
OPSGNN_API int opsgnn_set_status_sink(void* sink);
/* Poll limit of one wait for later launches (process-wide); negative restores the default.  Zero makes every
 * bulk-copy wait give up at once without touching the barrier: the diagnostic that exercises the error path on a
 * healthy GPU.  Copies in flight are still awaited with the default limit before a block exits. */
OPSGNN_API int opsgnn_set_wait_polls(int64_t polls);

/* Typed mean for integer sums (count wraps to the value dtype, truncating division, zero count gives 0):
 * out[b, r, k] /= narrow(ptr[r+1]-ptr[r]).  Follows MeanDivideRounded,
 * csrc/npu/segment_csr/op_kernel/arch35/segment_csr.cpp:282-297. */
OPSGNN_API int opsgnn_csr_integer_mean(void* out, int out_type, const void* ptr, int ptr_type, int64_t rows, int64_t feat,
                            int64_t batches, void* stream);

/* ======================================================================== */
/* SDDMM on CSR                                                              */
/* ======================================================================== */
#define OPSGNN_SDDMM_DOT 0
#define OPSGNN_SDDMM_ADD 1
#define OPSGNN_SDDMM_SUB 2
#define OPSGNN_SDDMM_MUL 3
#define OPSGNN_SDDMM_DIV 4
#define OPSGNN_SDDMM_COPY_LHS 5
#define OPSGNN_SDDMM_COPY_RHS 6
/* operand targets: which index of edge e selects the operand row */
#define OPSGNN_TARGET_ROW 0  /* "u"/"src": CSR row of e  */
#define OPSGNN_TARGET_EDGE 1 /* "e": e itself            */
#define OPSGNN_TARGET_COL 2  /* "v"/"dst": indices[e]    */

typedef struct OpsgnnSddmmDesc {
    int64_t rows;      /* CSR rows                                              */
    int64_t nnz;       /* edges                                                 */
    int64_t feat;      /* feature width of both operands (dot: reduction width) */
    int64_t lhs_rows;  /* rows of lhs (bounds the gather)                       */
    int64_t rhs_rows;  /* rows of rhs                                           */
    int32_t op;        /* OPSGNN_SDDMM_*                                        */
    int32_t lhs_target;
    int32_t rhs_target;
    int32_t index_type; /* OPSGNN_I32 / OPSGNN_I64 (indptr and indices)         */
    int32_t dtype;      /* OPSGNN_F32 / OPSGNN_F16 / OPSGNN_BF16                */
} OpsgnnSddmmDesc;

/* Bytes of scratch (the per-block row plan) for opsgnn_sddmm_csr. */
OPSGNN_API int opsgnn_sddmm_workspace_bytes(const OpsgnnSddmmDesc* desc, int64_t* bytes);
/* Replaces SddmmCsr (csrc/npu/sddmm_csr/op_kernel/arch22/sddmm_csr.cpp) as launched by
 * LaunchSddmmCsr (csrc/npu/sddmm_csr/op_host/sddmm_csr.cpp:368-411).
 * dot writes out[nnz]; the other ops write out[nnz, feat].  fp16/bf16 compute in fp32 and round once. */
OPSGNN_API int opsgnn_sddmm_csr(const OpsgnnSddmmDesc* desc, const void* indptr, const void* indices, const void* lhs,
                                const void* rhs, void* out, void* workspace, int64_t workspace_bytes, void* stream);

/*
 * opsgnn_sddmm_csr without caller-provided scratch.  It has no counterpart in the reference.
 *
 * Who needs it: a caller that is not in a position to obtain device memory at call time.  Examples are a plug-in whose
 * host application has already committed the whole GPU to its own memory pool and hands none of it to plug-ins, and a
 * latency-critical loop in which any allocator call is forbidden because cudaMalloc / cudaFree may synchronise the
 * device.  Such a caller owns its inputs and outputs but cannot produce the small row-plan scratch
 * opsgnn_sddmm_csr asks for, so this variant keeps that scratch in a fixed 256-KiB array inside the library.
 *
 * Limits and rules:
 *  - at most OPSGNN_SDDMM_STATIC_MAX_EDGES = 2^24 edges per call; a larger desc->nnz returns OPSGNN_ERR_LIMIT and
 *    launches nothing;
 *  - the array exists once per GPU that loads the library and stays until the process exits;
 *  - the first call on each device looks up the array's device address (cudaGetSymbolAddress); make that first call
 *    during start-up, before any stream capture;
 *  - every call on a device uses the same array and overwrites all of the part it reads, so nothing has to be
 *    cleared between calls, but two calls whose kernels can overlap on the GPU (different streams) race on it:
 *    serialise them;
 *  - the function calls no cudaMalloc, cudaFree or any allocating routine.
 * Arguments and results are those of opsgnn_sddmm_csr.
 */
#define OPSGNN_SDDMM_STATIC_MAX_EDGES (1LL << 24)
OPSGNN_API int opsgnn_sddmm_csr_static(const OpsgnnSddmmDesc* desc, const void* indptr, const void* indices,
                                       const void* lhs, const void* rhs, void* out, void* stream);

/* ======================================================================== */
/* Fused graph attention (no counterpart in the reference)                   */
/* ======================================================================== */
/*
 * One GAT layer over a CSR graph without materialising any per-edge tensor:
 *   logit[e, h] = leaky_relu(left[row(e), h] + right[col(e), h], negative_slope)
 *   lse[r, h]   = log sum_{e in row r} exp(logit[e, h])            (-inf for a row without edges)
 *   out[r, h, :] = sum_{e in row r} exp(logit[e, h] - lse[r, h]) * x[col(e), h, :]
 * The reference has no such entry point: it composes the layer from sddmm_csr, leaky_relu, scatter_softmax and
 * spmm / bspmm (python/ops_gnn/spmm.py:148-208, 283-289) and writes the [E, H] logits, their LeakyReLU, the softmax
 * weights (and, in the spmm fallback, the [E, H, D] messages) to memory.  Two calls: opsgnn_attention_lse reads the edge
 * list and the [N, H] halves and writes the logits [E, H] once together with lse; opsgnn_attention_aggregate (the weighted
 * bulk instance of the CSR engine) reads the logits once and forms every weight exp(logit - lse) in the gather ring.
 * fp32 only.  The aggregation needs heads * width a multiple of 256, heads a multiple of 4 and at most 21, width a
 * multiple of 4 and 16-byte aligned right / x / out; other shapes return OPSGNN_ERR_UNSUPPORTED (compose the layer
 * from the four operators instead).
 */
typedef struct OpsgnnAttentionDesc {
    int64_t rows;      /* CSR rows (destination nodes)                        */
    int64_t src_rows;  /* rows of right and x (source nodes)                  */
    int64_t heads;     /* H                                                   */
    int64_t width;     /* D: features per head                                */
    int64_t nnz;       /* edges                                               */
    float negative_slope;
    int32_t index_type; /* OPSGNN_I32 / OPSGNN_I64: ptr, col and edge_rows    */
    int32_t dtype;      /* OPSGNN_F32                                         */
} OpsgnnAttentionDesc;

OPSGNN_API int opsgnn_attention_lse_workspace_bytes(const OpsgnnAttentionDesc* desc, int64_t* bytes);
/* logits[nnz, H] and lse[rows, H] from edge_rows[nnz] (the CSR row of every edge, i.e. ptr2ind of the pointers), col[nnz],
 * left[rows, H], right[src_rows, H].  Deterministic: partial states of rows that span 128-edge chunks are folded in chunk
 * order (a row spanning more than 4 chunk boundaries by one warp, in a fixed order). */
OPSGNN_API int opsgnn_attention_lse(const OpsgnnAttentionDesc* desc, const void* edge_rows, const void* col, const float* left,
                                    const float* right, float* logits, float* lse, void* workspace, int64_t workspace_bytes,
                                    void* stream);
/* out[rows, H * D]; plan and workspace are those of opsgnn_csr_reduce for a descriptor with feat = H * D,
 * value_width = H, fp32 in and out, sum (opsgnn_csr_plan_bytes / opsgnn_csr_reduce_workspace_bytes). */
OPSGNN_API int opsgnn_attention_aggregate(const OpsgnnAttentionDesc* desc, const void* ptr, const void* col, const float* logits,
                                          const float* lse, const void* x, void* out, const void* plan, void* workspace,
                                          int64_t workspace_bytes, void* stream);

/* lse[groups, 8] = log-sum-exp per group of values[n, 8] (fp32, 16-byte aligned) under SORTED labels[n] in [0, groups):
 * the edge sweep of the fused attention layer run over given values - chunks of 128 rows, four columns per thread,
 * chunk partials folded in chunk order (deterministic).  Groups without rows get -inf.  No counterpart in the reference:
 * it is the first pass of scatter_softmax / scatter_log_softmax / scatter_logsumexp for eight-column sources (per-head
 * attention logits), whose rows are too narrow for the CSR engine's bulk ring
 * (csrc/npu/scatter_softmax/op_kernel/common/scatter_softmax_kernel_phase.h:126-279 is the reference's form). */
OPSGNN_API int opsgnn_sorted_lse8_workspace_bytes(int64_t n, int64_t* bytes);
OPSGNN_API int opsgnn_sorted_lse8(const void* labels, int index_type, const float* values, float* lse, int64_t n, int64_t groups,
                                  void* workspace, int64_t workspace_bytes, void* stream);

/* dvalue[e, w] = sum_b sum_k mat[b, col[e], k] * grad[b, row(e), k]  (w = 0 when width == 1, else k).
 * Replaces TorchSparseSpmmValueGrad (csrc/npu/torch_sparse_spmm/op_kernel/arch35/torch_sparse_spmm_kernel.h:326-395).
 * mean == 1 divides by the row's edge count.  grad and out are fp32; mat has dtype mat_type. */
OPSGNN_API int opsgnn_spmm_value_grad(const int64_t* ptr, const int64_t* col, const void* mat, int mat_type, const float* grad,
                           float* out, int64_t rows, int64_t src_rows, int64_t feat, int64_t nnz, int64_t batches,
                           int64_t width, int mean, void* stream);

/* ======================================================================== */
/* index conversions and CSR support kernels                                 */
/* ======================================================================== */
/* ptr[i] = number of ind[] entries < i, i in [0, rows]; ind sorted.  Replaces Ind2Ptr
 * (csrc/npu/ind2ptr/op_kernel/arch35/ind2ptr.cpp:146-168) and ConvertKernel with toPtr
 * (torch_sparse_spmm_kernel.h:432-456). */
OPSGNN_API int opsgnn_ind2ptr(const int64_t* ind, int64_t nnz, int64_t* ptr, int64_t rows, void* stream);
/* ind[e] = row r with ptr[r] <= e < ptr[r+1].  Replaces Ptr2Ind (csrc/npu/ptr2ind/op_kernel/arch35/ptr2ind.cpp:20-52). */
OPSGNN_API int opsgnn_ptr2ind(const int64_t* ptr, int64_t rows, int64_t* ind, int64_t nnz, void* stream);
/* status[0] = OR of: 1 ptr[0] != 0 or ptr[rows] != nnz, 2 pointer outside [0, nnz], 4 decreasing pointer,
 * 8 column outside [0, cols) (col may be NULL to skip the column check); 0 means a valid structure.
 * Replaces TorchSparseSpmmValidate (torch_sparse_spmm_kernel.h:399-430) and the device half of the CSR proof of
 * csrc/npu/common/spmm/host_proof_cache.h:243-310.  index_type selects int32/int64. */
OPSGNN_API int opsgnn_csr_validate(const void* ptr, const void* col, int index_type, int64_t rows, int64_t cols, int64_t nnz,
                        int32_t* status, void* stream);
/* out[i, :] = value[perm[i], :].  Replaces TorchSparseSpmmPermuteValues (torch_sparse_spmm.cpp:16-36). */
OPSGNN_API int opsgnn_permute_values(const int64_t* perm, const void* value, void* out, int64_t rows, int64_t width,
                          int elem_bytes, void* stream);
/* stats[0] = min(index), stats[1] = max(index), stats[2] = 1 when index is non-decreasing else 0.
 * One pass that serves the bounds checks of the grouped-softmax and scatter wrappers
 * (python/ops_gnn/_grouped_softmax.py:67-79, python/ops_gnn/scatter.py:347-361).  index_type I32/I64. */
OPSGNN_API int opsgnn_index_stats(const void* index, int index_type, int64_t n, int64_t* stats, void* stream);
/* longest[0] = rows of the largest group of a non-decreasing label vector: the longest run of equal consecutive values of
 * index[0..n) or, with perm (int64, may be NULL), of index[perm[0]], index[perm[1]], ...  Meaningless when that sequence
 * is not sorted.  Lets the grouped-softmax planner pick the single-read kernel; the reference has no sortedness
 * specialisation (scatter_softmax_kernel_phase.h:126-279 runs three atomic phases for every index). */
OPSGNN_API int opsgnn_index_longest_run(const void* index, int index_type, const int64_t* perm, int64_t n, int64_t* longest,
                                        void* stream);

/* out[i, :] = src[index[i], :] for rows of `row_bytes` bytes (a multiple of 16; src and every segment base 16-byte
 * aligned), with the output cut into `segments` (1..OPSGNN_GATHER_MAX_SEGMENTS) consecutive pieces: segment s holds
 * the next segment_rows[s] output rows and starts at segment_out[s].  The segments may live in different buffers,
 * another GPU's mapped memory included (the kernel writes with plain stores).  `segment_rows` and `segment_out` are
 * HOST arrays read during the call.  At most `max_ctas` thread blocks run (0 = no cap beyond eight per SM): the
 * kernel is the exchange step of the row-sharded SpMM, runs beside a product and is bound by NVLink, so a few dozen
 * blocks are enough.  index_type I32/I64; indices are clamped into [0, src_rows).
 * No counterpart in the reference, which is a single-device library (it has no exchange step). */
#define OPSGNN_GATHER_MAX_SEGMENTS 16
OPSGNN_API int opsgnn_gather_rows(const void* src, const void* index, int index_type, int64_t rows, int64_t src_rows,
                                  int64_t row_bytes, int segments, const int64_t* segment_rows, void* const* segment_out,
                                  int max_ctas, void* stream);

/* Batched row expansion, the inverse data movement of the segment reductions:
 *   csr == 0: out[b, i, :] = src[b, index[b, i], :]                      index is [batches, out_rows] int64
 *   csr == 1: out[b, i, :] = src[b, s, :] for ptr[b, s] <= i < ptr[b, s+1]  index is [batches, src_rows + 1] int64 pointers;
 *             output rows before ptr[b, 0] are zero.
 * src is [batches, src_rows, row_bytes], out is [batches, out_rows, row_bytes]; any element size (the copy unit is the
 * largest power of two up to 16 bytes that divides the row and both base addresses).  An index outside [0, src_rows)
 * writes zeros instead of reading out of range.  Replaces the GatherCoo launcher (csrc/npu/gather_coo/op_host/gather_coo.cpp)
 * and the GatherCsr launcher (csrc/npu/gather_csr/op_host/gather_csr.cpp:262-330). */
OPSGNN_API int opsgnn_gather_expand(const void* src, const int64_t* index, void* out, int64_t batches, int64_t src_rows,
                                    int64_t out_rows, int64_t row_bytes, int csr, void* stream);

/* ======================================================================== */
/* scatter (unsorted index)                                                  */
/* ======================================================================== */
#define OPSGNN_SCATTER_SUM 0
#define OPSGNN_SCATTER_MUL 1
#define OPSGNN_SCATTER_MEAN 2
#define OPSGNN_SCATTER_MIN 3
#define OPSGNN_SCATTER_MAX 4

typedef struct OpsgnnScatterDesc {
    int64_t before;     /* product of dims before `dim`                       */
    int64_t dim_len;    /* src.size(dim)                                      */
    int64_t after;      /* product of dims after `dim`                        */
    int64_t out_len;    /* out.size(dim)                                      */
    int64_t index_full; /* 0: index is [dim_len]; 1: index has src's shape    */
    int32_t reduce;     /* OPSGNN_SCATTER_* (codes of scatter_tiling.h:14-20) */
    int32_t dtype;      /* src/out dtype                                      */
    int32_t has_out;    /* out holds caller data that takes part in the reduce */
} OpsgnnScatterDesc;

OPSGNN_API int opsgnn_scatter_workspace_bytes(const OpsgnnScatterDesc* desc, int64_t* bytes);
/* Replaces the Scatter launcher (csrc/npu/scatter/op_kernel/arch35/scatter.cpp) called from scatter_forward
 * (csrc/npu/scatter/op_host/scatter.cpp:242-267).  out must be pre-filled by the caller exactly as the reference's
 * Python front-end does (zeros / ones / dtype extrema or the user's out); arg (int64) is required for min/max and
 * receives the largest source position among ties, dim_len where nothing was written. */
OPSGNN_API int opsgnn_scatter(const OpsgnnScatterDesc* desc, const void* src, const int64_t* index, void* out, int64_t* arg,
                   void* workspace, int64_t workspace_bytes, void* stream);

/* ======================================================================== */
/* grouped softmax family (unsorted 1-D index along `dim`)                   */
/* ======================================================================== */
#define OPSGNN_GROUPED_SOFTMAX 0
#define OPSGNN_GROUPED_LOG_SOFTMAX 1
#define OPSGNN_GROUPED_LOGSUMEXP 2

typedef struct OpsgnnGroupedDesc {
    int64_t batch;   /* product of dims before `dim`          */
    int64_t dim_len; /* src.size(dim)                         */
    int64_t after;   /* product of dims after `dim`           */
    int64_t groups;  /* dim_size                              */
    int32_t mode;    /* OPSGNN_GROUPED_*                      */
    int32_t dtype;   /* F32 / F16 / BF16                      */
    int32_t sorted;  /* 0: any order (atomic phases); 1: index is non-decreasing (log-sum-exp sweep + apply sweep);   */
                     /* OPSGNN_GROUPED_SORTED_SHORT: non-decreasing AND no group longer than                        */
                     /* OPSGNN_GROUPED_SHORT_GROUP rows: softmax / log-softmax read src once (one batch, rows of     */
                     /* whole 16-byte vectors; other shapes return OPSGNN_ERR_UNSUPPORTED, pass 1 for them)          */
    int32_t index_type; /* OPSGNN_I32 (what the reference binding passes) or OPSGNN_I64 */
} OpsgnnGroupedDesc;

#define OPSGNN_GROUPED_SORTED_SHORT 2
#define OPSGNN_GROUPED_SHORT_GROUP 1024
OPSGNN_API int opsgnn_grouped_workspace_bytes(const OpsgnnGroupedDesc* desc, int64_t* bytes);
/* Replaces ScatterSoftmaxForward / ScatterLogSoftmaxForward / ScatterLogSumExpForward
 * (csrc/npu/scatter_softmax/op_kernel/common/scatter_softmax_kernel_entry.h:218-283) as launched by
 * grouped_softmax::RunForward (csrc/npu/scatter_softmax/common/grouped_softmax_shared.h:178-208).
 * index is [dim_len] of desc->index_type. out has src's shape (softmax, log_softmax) or [batch, groups, after]
 * (logsumexp). */
OPSGNN_API int opsgnn_grouped_forward(const OpsgnnGroupedDesc* desc, const void* src, const void* index, void* out,
                                      void* workspace, int64_t workspace_bytes, void* stream);

/* Sorted labels prepared once and reused: ptr[groups + 1] (the segment pointers of the label vector) and the CSR plan
 * over them (opsgnn_csr_plan_bytes(groups, dim_len) bytes, 256-byte aligned).  opsgnn_grouped_forward_prepared is
 * opsgnn_grouped_forward for desc->sorted = 1 without the boundary scan and the plan build; the workspace is sized by
 * opsgnn_grouped_workspace_bytes as before.  No counterpart in the reference, which rescans the index in every call
 * (csrc/npu/scatter_softmax/common/grouped_softmax_shared.h:178-208). */
OPSGNN_API int opsgnn_grouped_prepare(const OpsgnnGroupedDesc* desc, const void* index, int64_t* ptr, void* plan, void* stream);
OPSGNN_API int opsgnn_grouped_forward_prepared(const OpsgnnGroupedDesc* desc, const void* src, const void* index,
                                               const int64_t* ptr, const void* plan, void* out, void* workspace,
                                               int64_t workspace_bytes, void* stream);
/* Softmax / log-softmax over an UNSORTED index through a permutation: perm[dim_len] (int64) must order the rows by group
 * (a stable argsort of index) and no group may hold more than OPSGNN_GROUPED_SHORT_GROUP rows.  Row perm[e] is read and
 * written in place of row e of the sorted sequence, so the result lands in the caller's row order with one read of src,
 * one write of out, no atomics and no fp32 scratch.  The workspace is that of the same descriptor with
 * sorted = OPSGNN_GROUPED_SORTED_SHORT.  The reference runs its three atomic phases for every index
 * (scatter_softmax_kernel_phase.h:126-279); this entry has no counterpart there.  One batch, rows of whole 16-byte
 * vectors; other shapes and log-sum-exp return OPSGNN_ERR_UNSUPPORTED. */
OPSGNN_API int opsgnn_grouped_forward_permuted(const OpsgnnGroupedDesc* desc, const void* src, const void* index,
                                               const int64_t* perm, void* out, void* workspace, int64_t workspace_bytes,
                                               void* stream);
/* Replaces the backward launches (scatter_softmax_kernel_entry.h:247-264, 293-357; RunBackward
 * grouped_softmax_shared.h:212-248).  softmax: grad = out*(g - sum_group(out*g)); log_softmax:
 * grad = g - exp(out)*sum_group(g); logsumexp: grad = exp(src - out[group]) * g[group] (src required). */
OPSGNN_API int opsgnn_grouped_backward(const OpsgnnGroupedDesc* desc, const void* src, const void* out, const void* grad_out,
                            const void* index, void* grad_src, void* workspace, int64_t workspace_bytes,
                            void* stream);

#ifdef __cplusplus
}
#endif
#endif /* OPSGNN_B200_H */
