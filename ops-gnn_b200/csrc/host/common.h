// Shared pieces of the C++ launch planners: dtype ids, current-stream lookup, status checks, scratch allocation and
// the per-graph cache of merge-path plans.  The planners validate and allocate with torch, then hand raw pointers to
// the C ABI of libopsgnn_b200.so; no planner computes on the host and none has a CPU path.
#pragma once

#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <optional>
#include <string>
#include <tuple>
#include <vector>

#include "opsgnn_b200.h"

namespace opsgnn {

inline int DtypeId(at::ScalarType t, const char* api)
{
    switch (t) {
        case at::kFloat:
            return OPSGNN_F32;
        case at::kHalf:
            return OPSGNN_F16;
        case at::kBFloat16:
            return OPSGNN_BF16;
        case at::kChar:
            return OPSGNN_I8;
        case at::kInt:
            return OPSGNN_I32;
        case at::kLong:
            return OPSGNN_I64;
        case at::kByte:
            return OPSGNN_U8;
        case at::kShort:
            return OPSGNN_I16;
        case at::kDouble:
            return OPSGNN_F64;
        default:
            TORCH_CHECK(false, api, ": unsupported dtype ", t);
    }
    return -1;
}

inline void CheckCuda(const at::Tensor& t, const char* api, const char* name)
{
    TORCH_CHECK(t.defined() && t.device().is_cuda(), api, ": ", name, " must be a CUDA tensor (there is no CPU path)");
}

inline void* CurrentStream(const at::Tensor& t)
{
    return reinterpret_cast<void*>(c10::cuda::getCurrentCUDAStream(t.device().index()).stream());
}

inline void CheckStatus(int status, const char* api)
{
    TORCH_CHECK(status == OPSGNN_OK, api, ": native launch failed: ", opsgnn_status_string(status), " (status ", status,
                ")");
}

// Byte scratch on the tensor's device; the caching allocator returns 512-byte aligned blocks.
inline at::Tensor Scratch(int64_t bytes, const at::Tensor& like)
{
    return at::empty({bytes > 0 ? bytes : 1}, like.options().dtype(at::kByte));
}

inline int64_t Product(c10::IntArrayRef sizes, int64_t from, int64_t to)
{
    int64_t p = 1;
    for (int64_t i = from; i < to; ++i) {
        p *= sizes[i];
    }
    return p;
}

// ---- when may a fact derived from a tensor's contents be reused? ---------------------------------------------------------
// The planners cache facts that depend on what an index tensor HOLDS (the merge-path plan of a pointer array, the
// validity mask of a CSR pair, whether a label vector is sorted).  A tensor's version counter sees in-place ATen
// writes, but not a write through `tensor.data`, through an independent `set_()` alias of the same storage, or by a
// kernel of this library into a caller-supplied `out=` that aliases an older input.  The reference closes that gap
// (csrc/npu/common/spmm/host_proof_cache.h:36-83, 150-200) by treating ANY ATen operation that runs between two of its
// calls as a possible write, and so does this build: a process-wide write clock advances whenever an ATen operator
// starts or ends outside a planner (a global RecordFunction callback, installed at module import) and whenever a
// planner is handed caller memory to write.  A cached fact carries the clock value it was made under and is reused
// only while the clock has not moved, no foreign operator is in flight on another thread, and the tensor's identity,
// version, address and layout are unchanged.  Back-to-back calls on one graph (a timing loop, the layers of a model
// that only calls this library) hit the caches; anything else re-derives the fact with one small kernel.
// Writes no host code can see (a raw-pointer write from another library, a peer GPU's store) remain the caller's
// business: call clear_native_caches() after them.
void StartWriteObserver();
uint64_t WriteClock();
bool WriteClockCurrent(uint64_t stamp);
void NoteCallerMemoryWritten();
// A planner about to write a caller-supplied `out`.  Every cached fact describes an INTEGER tensor (pointers, columns,
// labels), so only an integer `out` can overwrite one; floating outputs leave the clock alone (reinterpreting a float
// buffer as an index tensor of a later call is outside the contract).
inline void NoteCallerOutput(const at::Tensor& out)
{
    if (out.defined() && !out.is_floating_point()) {
        NoteCallerMemoryWritten();
    }
}

// RAII around one planner call: ATen work the planner does itself (allocations, contiguous copies, the 4-byte read of
// a validation mask) is not a foreign write.
class PlannerScope {
public:
    PlannerScope();
    ~PlannerScope();
    PlannerScope(const PlannerScope&) = delete;
    PlannerScope& operator=(const PlannerScope&) = delete;

private:
    bool could_observe_;
};

// Wraps a planner for binding: the whole call runs inside a PlannerScope.
template <class R, class... A> auto Scoped(R (*fn)(A...))
{
    return [fn](A... args) -> R {
        PlannerScope scope;
        return fn(std::forward<A>(args)...);
    };
}

// Identity of a tensor's contents as far as the host can see them (see above).  Inference tensors have no version
// counter and are never cached.
struct TensorKey {
    const c10::TensorImpl* impl = nullptr;
    const void* data = nullptr;
    int64_t version = -1;
    int64_t offset = 0;
    uint64_t clock = 0;
    std::vector<int64_t> sizes, strides;
    std::optional<c10::weak_intrusive_ptr<c10::TensorImpl>> alive;

    static std::optional<TensorKey> Of(const at::Tensor& t);
    bool Matches(const TensorKey& now) const;   // `now` = TensorKey::Of(the tensor presented by the current call)
};

// Merge-path plan of a pointer array, cached per tensor identity, version and write clock (a GNN calls the same graph
// every layer and every step).  Entries hold a weak reference, so a recycled address cannot revive a stale plan.  A plan
// built on one stream and reused on another is ordered by an event recorded after its kernel.
at::Tensor CsrPlan(const at::Tensor& ptr, int64_t rows, int64_t nnz_bound);
void ClearCsrPlanCache();

struct CsrReduceCall {
    at::Tensor ptr;                 // [rows + 1], int32/int64, contiguous
    std::optional<at::Tensor> col;  // [nnz] same dtype as ptr, or nullopt for consecutive source rows
    std::optional<at::Tensor> val;  // [nnz] or [nnz, feat], dtype of mat
    at::Tensor mat;                 // contiguous, viewed as [batches, src_rows, feat]
    at::Tensor out;                 // contiguous, viewed as [batches, rows, feat]
    std::optional<at::Tensor> arg;  // int64, shape of out (allocated internally when absent for min/max)
    int64_t rows = 0, src_rows = 0, feat = 0, nnz = 0, batches = 1, value_width = 0, arg_none = 0;
    int reduce = OPSGNN_REDUCE_SUM;
    int extremum = OPSGNN_EXTREMUM_IGNORE_NAN;
};

// Builds (or reuses) the plan, allocates carry scratch and launches the engine on the current stream.
void RunCsrReduce(CsrReduceCall& call, const char* api);

// Device-side waits that ran out (a bulk-copy wait of the reduce engine gave up; its launch left rows unwritten).  The
// kernels report into one word of mapped pinned host memory per device, registered with the C ABI on the device's first
// use, so the host can look without synchronising: every planner call looks first and raises for a stall of an EARLIER
// launch (the asynchronous-error convention of CUDA itself).  DeviceStallCount(sync = true) synchronises the device
// first, which makes the report cover everything enqueued so far.  Reading clears the word.
void RaiseIfDeviceStalled(const at::Tensor& on_device, const char* api);
int64_t DeviceStallCount(int device, bool synchronize);

// Validation facts of a CSR structure: bit mask of opsgnn_csr_validate, cached like the plans.  Costs one 4-byte
// device-to-host read on a miss.
int CsrFacts(const at::Tensor& ptr, const std::optional<at::Tensor>& col, int64_t rows, int64_t cols, int64_t nnz);
void ClearCsrFactsCache();
// What the planners know about a 1-D label vector (grouped.cpp), derived once per (tensor, version, write clock): its
// value range, whether it is non-decreasing, the rows of its largest group and - for an unsorted vector somebody asked
// to sort - the stable permutation that sorts it.  Miss: two small kernels and one 32-byte read (plus an argsort and a
// second run-length pass for the permutation).  Hit: nothing.
struct LabelFacts {
    int64_t low = 0, high = -1;
    bool sorted = false;
    int64_t longest = 0;    // rows of the largest group; valid when `measured`
    at::Tensor perm;        // int64 stable argsort; defined only when !sorted and a permutation was asked for
    bool measured = false;  // longest (and perm) were derived
};
LabelFacts LabelFactsOf(const at::Tensor& index, bool want_permutation);
void ClearSortedIndexCache();                          // grouped.cpp: the facts of label vectors
int64_t SortedIndexCacheSize();
std::tuple<int64_t, int64_t, int64_t> NativeCacheSizes();  // plans, validation facts, sortedness facts

}  // namespace opsgnn
