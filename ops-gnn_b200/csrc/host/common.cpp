#include "common.h"

#include <ATen/cuda/CUDAEvent.h>
#include <ATen/record_function.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAException.h>
#include <c10/util/intrusive_ptr.h>
#include <cuda_runtime_api.h>

#include <atomic>
#include <list>
#include <memory>
#include <mutex>

namespace opsgnn {

// ---- write clock ---------------------------------------------------------------------------------------------------------
namespace {

std::atomic<uint64_t> g_write_clock{1};
std::atomic<int64_t> g_foreign_in_flight{0};
std::atomic<bool> g_observing{false};
thread_local int t_planner_depth = 0;
thread_local bool t_observable = true;

struct ForeignOperator : at::ObserverContext {};

std::unique_ptr<at::ObserverContext> OnOperatorStart(const at::RecordFunction&)
{
    if (t_planner_depth != 0) {
        return nullptr;  // the planner's own ATen work
    }
    g_foreign_in_flight.fetch_add(1, std::memory_order_acq_rel);
    g_write_clock.fetch_add(1, std::memory_order_acq_rel);
    return std::make_unique<ForeignOperator>();
}

void OnOperatorEnd(const at::RecordFunction&, at::ObserverContext* context)
{
    if (context == nullptr) {
        return;
    }
    g_write_clock.fetch_add(1, std::memory_order_acq_rel);
    g_foreign_in_flight.fetch_sub(1, std::memory_order_acq_rel);
}

}  // namespace

void StartWriteObserver()
{
    // Once, at module import (global callbacks must not be added while operators run in parallel); kept for the life of
    // the process.
    static const auto handle = at::addGlobalCallback(at::RecordFunctionCallback(OnOperatorStart, OnOperatorEnd)
                                                         .needsInputs(false)
                                                         .needsOutputs(false)
                                                         .scopes({at::RecordScope::FUNCTION}));
    (void)handle;
    g_observing.store(true, std::memory_order_release);
}

uint64_t WriteClock() { return g_write_clock.load(std::memory_order_acquire); }

bool WriteClockCurrent(uint64_t stamp)
{
    return t_observable && g_observing.load(std::memory_order_acquire) &&
           g_foreign_in_flight.load(std::memory_order_acquire) == 0 && WriteClock() == stamp;
}

void NoteCallerMemoryWritten() { g_write_clock.fetch_add(1, std::memory_order_acq_rel); }

PlannerScope::PlannerScope() : could_observe_(t_observable)
{
    // With operator recording switched off on this thread nothing can be observed: make every cached fact stale.
    t_observable = could_observe_ && at::isRecordFunctionEnabled();
    if (!t_observable) {
        NoteCallerMemoryWritten();
    }
    ++t_planner_depth;
}

PlannerScope::~PlannerScope()
{
    --t_planner_depth;
    t_observable = could_observe_;
}

std::optional<TensorKey> TensorKey::Of(const at::Tensor& t)
{
    if (!t.defined() || t.is_inference()) {
        return std::nullopt;
    }
    TensorKey key;
    key.impl = t.unsafeGetTensorImpl();
    key.data = t.const_data_ptr();
    key.version = t._version();
    key.offset = t.storage_offset();
    key.clock = WriteClock();
    key.sizes = t.sizes().vec();
    key.strides = t.strides().vec();
    key.alive = c10::weak_intrusive_ptr<c10::TensorImpl>(t.getIntrusivePtr());
    return key;
}

bool TensorKey::Matches(const TensorKey& now) const
{
    return impl == now.impl && data == now.data && version == now.version && offset == now.offset &&
           sizes == now.sizes && strides == now.strides && alive.has_value() && !alive->expired() &&
           WriteClockCurrent(clock);
}

namespace {

struct PlanEntry {
    TensorKey ptr;
    int64_t rows, nnz;
    at::Tensor plan;
    std::shared_ptr<at::cuda::CUDAEvent> built;  // recorded after PlanKernel on the stream that built the plan
    cudaStream_t stream;
};

struct FactsEntry {
    TensorKey ptr;
    std::optional<TensorKey> col;
    int64_t rows, cols, nnz;
    int facts;
};

constexpr size_t kCacheEntries = 32;
std::mutex g_mutex;
std::list<PlanEntry> g_plans;
std::list<FactsEntry> g_facts;

}  // namespace

at::Tensor CsrPlan(const at::Tensor& ptr, int64_t rows, int64_t nnz_bound)
{
    auto key = TensorKey::Of(ptr);
    const auto current = c10::cuda::getCurrentCUDAStream(ptr.device().index());
    if (key) {
        std::lock_guard<std::mutex> lock(g_mutex);
        for (auto it = g_plans.begin(); it != g_plans.end(); ++it) {
            if (it->rows == rows && it->nnz == nnz_bound && it->ptr.Matches(*key)) {
                g_plans.splice(g_plans.begin(), g_plans, it);
                PlanEntry& hit = g_plans.front();
                if (hit.stream != current.stream()) {
                    // another stream built it: wait for its kernel, and keep the allocator from recycling the plan
                    // under this stream should the entry be evicted while this stream still reads it
                    hit.built->block(current);
                    c10::cuda::CUDACachingAllocator::recordStream(hit.plan.storage().data_ptr(), current);
                }
                return hit.plan;
            }
        }
    }
    int64_t bytes = 0;
    CheckStatus(opsgnn_csr_plan_bytes(rows, nnz_bound, &bytes), "csr_plan");
    auto plan = at::empty({bytes / 8}, ptr.options().dtype(at::kLong));
    CheckStatus(opsgnn_csr_plan_build(ptr.const_data_ptr(), DtypeId(ptr.scalar_type(), "csr_plan"), rows, nnz_bound,
                                      plan.data_ptr(), CurrentStream(ptr)),
                "csr_plan");
    if (key) {
        auto built = std::make_shared<at::cuda::CUDAEvent>();
        built->record(current);
        std::lock_guard<std::mutex> lock(g_mutex);
        g_plans.push_front(PlanEntry{*key, rows, nnz_bound, plan, built, current.stream()});
        if (g_plans.size() > kCacheEntries) {
            g_plans.pop_back();
        }
    }
    return plan;
}

void ClearCsrPlanCache()
{
    std::lock_guard<std::mutex> lock(g_mutex);
    g_plans.clear();
}

int CsrFacts(const at::Tensor& ptr, const std::optional<at::Tensor>& col, int64_t rows, int64_t cols, int64_t nnz)
{
    auto ptr_key = TensorKey::Of(ptr);
    std::optional<TensorKey> col_key;
    bool cacheable = ptr_key.has_value();
    if (col) {
        col_key = TensorKey::Of(*col);
        cacheable = cacheable && col_key.has_value();
    }
    if (cacheable) {
        std::lock_guard<std::mutex> lock(g_mutex);
        for (auto it = g_facts.begin(); it != g_facts.end(); ++it) {
            const bool same_col = col_key.has_value() == it->col.has_value() && (!col_key || it->col->Matches(*col_key));
            if (it->rows == rows && it->cols == cols && it->nnz == nnz && same_col && it->ptr.Matches(*ptr_key)) {
                g_facts.splice(g_facts.begin(), g_facts, it);
                return g_facts.front().facts;
            }
        }
    }
    auto status = at::empty({1}, ptr.options().dtype(at::kInt));
    CheckStatus(opsgnn_csr_validate(ptr.const_data_ptr(), col ? col->const_data_ptr() : nullptr,
                                    DtypeId(ptr.scalar_type(), "csr_validate"), rows, cols, nnz,
                                    status.data_ptr<int32_t>(), CurrentStream(ptr)),
                "csr_validate");
    const int facts = status.item<int32_t>();
    if (cacheable) {
        std::lock_guard<std::mutex> lock(g_mutex);
        g_facts.push_front(FactsEntry{*ptr_key, col_key, rows, cols, nnz, facts});
        if (g_facts.size() > kCacheEntries) {
            g_facts.pop_back();
        }
    }
    return facts;
}

void ClearCsrFactsCache()
{
    std::lock_guard<std::mutex> lock(g_mutex);
    g_facts.clear();
}

std::tuple<int64_t, int64_t, int64_t> NativeCacheSizes()
{
    std::lock_guard<std::mutex> lock(g_mutex);
    return {static_cast<int64_t>(g_plans.size()), static_cast<int64_t>(g_facts.size()), SortedIndexCacheSize()};
}

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_sink_mutex;
at::Tensor g_sink;               // int64[kMaxDevices] in pinned host memory: one stall word per device
bool g_sink_registered[kMaxDevices] = {false};

volatile int64_t* SinkWord(int device)
{
    if (device < 0 || device >= kMaxDevices) {
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_sink_mutex);
    if (!g_sink.defined()) {
        g_sink = at::zeros({kMaxDevices}, at::TensorOptions().dtype(at::kLong)).pin_memory();
    }
    int64_t* word = g_sink.data_ptr<int64_t>() + device;
    if (!g_sink_registered[device]) {
        // Pinned host memory is mapped into every device's address space at its host address (unified addressing).
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
        CheckStatus(opsgnn_set_status_sink(word), "status_sink");
        g_sink_registered[device] = true;
    }
    return word;
}

}  // namespace

int64_t DeviceStallCount(int device, bool synchronize)
{
    volatile int64_t* word = SinkWord(device);
    if (word == nullptr) {
        return 0;
    }
    if (synchronize) {
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
        C10_CUDA_CHECK(cudaDeviceSynchronize());
    }
    const int64_t count = *word;
    if (count != 0) {
        *word = 0;
    }
    return count;
}

void RaiseIfDeviceStalled(const at::Tensor& on_device, const char* api)
{
    const int device = on_device.device().index();
    TORCH_CHECK(DeviceStallCount(device, false) == 0, api,
                ": device wait timed out in an earlier launch on cuda:", device,
                " (a bulk-copy wait of the reduce kernel ran out of polls; that launch's output is incomplete)");
}

void RunCsrReduce(CsrReduceCall& call, const char* api)
{
    if (call.rows == 0 || call.feat == 0 || call.batches == 0) {
        return;
    }
    RaiseIfDeviceStalled(call.out, api);
    OpsgnnCsrReduceDesc desc{};
    desc.rows = call.rows;
    desc.src_rows = call.src_rows;
    desc.feat = call.feat;
    desc.nnz = call.nnz;
    desc.batches = call.batches;
    desc.value_width = call.val ? call.value_width : 0;
    desc.arg_none = call.arg_none;
    desc.reduce = call.reduce;
    desc.extremum = call.extremum;
    desc.ptr_type = DtypeId(call.ptr.scalar_type(), api);
    desc.col_type = call.col ? DtypeId(call.col->scalar_type(), api) : desc.ptr_type;
    desc.in_type = DtypeId(call.mat.scalar_type(), api);
    desc.out_type = DtypeId(call.out.scalar_type(), api);

    const bool extremum = call.reduce == OPSGNN_REDUCE_MIN || call.reduce == OPSGNN_REDUCE_MAX;
    at::Tensor arg;
    if (extremum) {
        arg = call.arg ? *call.arg : at::empty(call.out.sizes(), call.out.options().dtype(at::kLong));
    }
    at::Tensor plan = CsrPlan(call.ptr, call.rows, call.nnz);
    int64_t bytes = 0;
    CheckStatus(opsgnn_csr_reduce_workspace_bytes(&desc, &bytes), api);
    at::Tensor scratch = Scratch(bytes, call.out);
    CheckStatus(opsgnn_csr_reduce(&desc, call.ptr.const_data_ptr(), call.col ? call.col->const_data_ptr() : nullptr,
                                  call.val ? call.val->const_data_ptr() : nullptr, call.mat.const_data_ptr(),
                                  call.out.data_ptr(), extremum ? arg.data_ptr<int64_t>() : nullptr,
                                  plan.const_data_ptr(), scratch.data_ptr(), scratch.numel(), CurrentStream(call.out)),
                api);
}

}  // namespace opsgnn
