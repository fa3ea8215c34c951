// Launch planners of the SpMM family.
//
// torch_sparse_spmm::{forward, validate, value_backward, convert, permute_values, tensor_version} keep the
// contract of csrc/npu/torch_sparse_spmm/op_host/torch_sparse_spmm.cpp:72-193 of the reference;
// spmm_{sum,max,min}_csr and unified_spmm_csr keep the contract of csrc/npu/common/spmm/spmm_utils.h:58-204 and
// csrc/npu/unified_spmm/op_host/unified_spmm.cpp:116-158 (same argument checks and messages; the uint32 / UB
// capacity limits of the Ascend kernels do not exist here because every offset is 64-bit).
#include "ops.h"

namespace opsgnn {
namespace {

int SparseType(at::ScalarType t)
{
    switch (t) {
        case at::kFloat:
            return 0;
        case at::kHalf:
            return 1;
        case at::kBFloat16:
            return 2;
        case at::kChar:
            return 3;
        case at::kInt:
            return 4;
        default:
            TORCH_CHECK(false, "unsupported SpMM dtype");
    }
    return -1;
}

void SparseDevice(const at::Tensor& x) { TORCH_CHECK(x.defined() && x.device().is_cuda(), "SpMM requires CUDA tensors"); }

void SparseIndices(const at::Tensor& ptr, const at::Tensor& col)
{
    SparseDevice(ptr);
    SparseDevice(col);
    TORCH_CHECK(ptr.device() == col.device() && ptr.scalar_type() == at::kLong && col.scalar_type() == at::kLong,
                "indices must be int64 on the same GPU");
    TORCH_CHECK(ptr.dim() == 1 && ptr.numel() > 0 && col.dim() == 1, "invalid CSR shape");
}

struct SparseShape {
    int64_t m, n, k, edges, batches, width;
    int reduce;
};

SparseShape Shape(const at::Tensor& ptr, const at::Tensor& col, const at::Tensor& mat, int64_t width, int64_t reduce)
{
    SparseIndices(ptr, col);
    SparseDevice(mat);
    TORCH_CHECK(mat.device() == ptr.device() && mat.dim() >= 2, "mat must have shape [...,N,K] on the same GPU");
    TORCH_CHECK(reduce >= 0 && reduce <= 3, "unsupported reduce");
    TORCH_CHECK(SparseType(mat.scalar_type()) < 4, "int32 input is unsupported");
    return {ptr.numel() - 1, mat.size(-2), mat.size(-1), col.numel(), Product(mat.sizes(), 0, mat.dim() - 2), width,
            static_cast<int>(reduce)};
}

}  // namespace

std::tuple<at::Tensor, at::Tensor> TorchSparseSpmmForward(at::Tensor ptr, at::Tensor col,
                                                          std::optional<at::Tensor> value, at::Tensor mat,
                                                          int64_t reduce, int64_t outType)
{
    int64_t width = 1;
    if (value) {
        SparseDevice(*value);
        TORCH_CHECK(value->device() == mat.device() && value->scalar_type() == mat.scalar_type(),
                    "value dtype/device must match mat");
        TORCH_CHECK(value->dim() >= 1 && value->size(0) == col.numel(), "value length must equal E");
        width = Product(value->sizes(), 1, value->dim());
    }
    auto s = Shape(ptr, col, mat, width, reduce);
    TORCH_CHECK(width == 1 || width == s.k, "value must contain 1 or K weights per edge");
    const int input = SparseType(mat.scalar_type());
    TORCH_CHECK((input == 0 && outType == 0) || (input == 1 && (outType == 0 || outType == 1)) ||
                    (input == 2 && (outType == 0 || outType == 2)) || (input == 3 && (outType == 0 || outType == 4)),
                "unsupported input/output dtype combination");
    c10::cuda::CUDAGuard guard(mat.device());
    ptr = ptr.contiguous();
    col = col.contiguous();
    mat = mat.contiguous();
    auto sizes = mat.sizes().vec();
    sizes[sizes.size() - 2] = s.m;
    const at::ScalarType ot = outType == 0 ? at::kFloat : outType == 1 ? at::kHalf : outType == 2 ? at::kBFloat16 : at::kInt;
    auto out = at::empty(sizes, mat.options().dtype(ot));
    auto arg = at::empty(reduce >= 2 ? sizes : std::vector<int64_t>{0}, col.options());
    if (out.numel() == 0) {
        return {out, arg};
    }
    if (s.edges > 0) {
        TORCH_CHECK(s.n > 0, "mat has no rows but the CSR structure has edges");
    }
    CsrReduceCall call;
    call.ptr = ptr;
    call.col = col;
    if (value) {
        call.val = value->contiguous();
    }
    call.mat = mat;
    call.out = out;
    if (reduce >= 2) {
        call.arg = arg;
    }
    call.rows = s.m;
    call.src_rows = s.n;
    call.feat = s.k;
    call.nnz = s.edges;
    call.batches = s.batches;
    call.value_width = width;
    call.arg_none = s.edges;
    call.reduce = static_cast<int>(reduce);  // 0 sum, 1 mean, 2 min, 3 max: same codes as OPSGNN_REDUCE_*
    call.extremum = OPSGNN_EXTREMUM_IGNORE_NAN;
    const bool integer_mean = reduce == 1 && ot == at::kInt;
    // int8 rows accumulate exactly in int32; a floating mean of them divides the finished sum.
    const bool widened_mean = reduce == 1 && input == 3 && ot == at::kFloat;
    if (integer_mean || widened_mean) {
        call.reduce = OPSGNN_REDUCE_SUM;  // the division needs the complete row sum
    }
    RunCsrReduce(call, "torch_sparse_spmm");
    if (widened_mean) {
        auto degree = (ptr.slice(0, 1) - ptr.slice(0, 0, s.m)).clamp_min(1).to(at::kFloat).unsqueeze(-1);
        out.div_(degree);
    }
    if (integer_mean) {
        CheckStatus(opsgnn_csr_integer_mean(out.data_ptr(), OPSGNN_I32, ptr.const_data_ptr(), OPSGNN_I64, s.m, s.k,
                                            s.batches, CurrentStream(out)),
                    "torch_sparse_spmm");
    }
    return {out, arg};
}

at::Tensor TorchSparseSpmmValidate(at::Tensor ptr, at::Tensor col, int64_t n)
{
    SparseIndices(ptr, col);
    TORCH_CHECK(n >= 0, "N must be nonnegative");
    c10::cuda::CUDAGuard guard(ptr.device());
    ptr = ptr.contiguous();
    col = col.contiguous();
    auto flags = at::empty({1}, ptr.options().dtype(at::kInt));
    CheckStatus(opsgnn_csr_validate(ptr.const_data_ptr(), col.const_data_ptr(), OPSGNN_I64, ptr.numel() - 1, n,
                                    col.numel(), flags.data_ptr<int32_t>(), CurrentStream(ptr)),
                "torch_sparse_spmm.validate");
    // Reference status codes: 0 valid, 1 bad pointer array, 2 column out of range (the caller takes the maximum).
    auto bad_col = flags.bitwise_and(8).ne(0).to(at::kInt) * 2;
    auto bad_ptr = flags.bitwise_and(7).ne(0).to(at::kInt);
    return at::maximum(bad_col, bad_ptr);
}

at::Tensor TorchSparseSpmmValueGrad(at::Tensor ptr, at::Tensor col, at::Tensor mat, at::Tensor grad, int64_t reduce,
                                    int64_t width)
{
    auto s = Shape(ptr, col, mat, width, reduce);
    TORCH_CHECK(width == 1 || width == s.k, "value width must be 1 or K");
    TORCH_CHECK(reduce < 2 && mat.is_floating_point(), "value backward supports floating sum/mean");
    auto expected = mat.sizes().vec();
    expected[expected.size() - 2] = s.m;
    TORCH_CHECK(grad.device() == mat.device() && grad.is_floating_point() && grad.sizes().vec() == expected,
                "grad must be floating [...,M,K] on the same GPU as mat");
    c10::cuda::CUDAGuard guard(mat.device());
    grad = grad.to(at::kFloat).contiguous();
    ptr = ptr.contiguous();
    col = col.contiguous();
    mat = mat.contiguous();
    auto out = at::empty({s.edges, width}, mat.options().dtype(at::kFloat));
    if (out.numel()) {
        CheckStatus(opsgnn_spmm_value_grad(ptr.data_ptr<int64_t>(), col.data_ptr<int64_t>(), mat.const_data_ptr(),
                                           DtypeId(mat.scalar_type(), "value_backward"), grad.data_ptr<float>(),
                                           out.data_ptr<float>(), s.m, s.n, s.k, s.edges, s.batches, width,
                                           reduce == 1, CurrentStream(mat)),
                    "torch_sparse_spmm.value_backward");
    }
    return out;
}

at::Tensor TorchSparseSpmmConvert(at::Tensor src, int64_t output, bool toPtr)
{
    SparseDevice(src);
    TORCH_CHECK(src.scalar_type() == at::kLong && src.dim() == 1 && output >= 0,
                "conversion requires int64 vector and nonnegative size");
    TORCH_CHECK(toPtr || src.numel() > 0, "CSR ptr must not be empty");
    c10::cuda::CUDAGuard guard(src.device());
    src = src.contiguous();
    auto out = at::empty({output}, src.options());
    if (output) {
        if (toPtr) {
            CheckStatus(opsgnn_ind2ptr(src.data_ptr<int64_t>(), src.numel(), out.data_ptr<int64_t>(), output - 1,
                                       CurrentStream(src)),
                        "torch_sparse_spmm.convert");
        } else {
            CheckStatus(opsgnn_ptr2ind(src.data_ptr<int64_t>(), src.numel() - 1, out.data_ptr<int64_t>(), output,
                                       CurrentStream(src)),
                        "torch_sparse_spmm.convert");
        }
    }
    return out;
}

at::Tensor TorchSparseSpmmPermuteValues(at::Tensor value, at::Tensor perm)
{
    SparseDevice(value);
    SparseDevice(perm);
    TORCH_CHECK(value.device() == perm.device() && value.dim() >= 1 && perm.dim() == 1 &&
                    perm.scalar_type() == at::kLong && perm.numel() == value.size(0),
                "invalid value permutation metadata");
    TORCH_CHECK(SparseType(value.scalar_type()) < 4, "unsupported edge-value dtype");
    c10::cuda::CUDAGuard guard(value.device());
    value = value.contiguous();
    perm = perm.contiguous();
    const int64_t width = Product(value.sizes(), 1, value.dim());
    auto out = at::empty(value.sizes(), value.options());
    if (out.numel()) {
        CheckStatus(opsgnn_permute_values(perm.data_ptr<int64_t>(), value.const_data_ptr(), out.data_ptr(),
                                          value.size(0), width, static_cast<int>(value.element_size()),
                                          CurrentStream(value)),
                    "torch_sparse_spmm.permute_values");
    }
    return out;
}

std::optional<int64_t> TorchSparseSpmmTensorVersion(const at::Tensor& tensor)
{
    if (tensor.is_inference()) {
        return std::nullopt;
    }
    return tensor._version();
}

// ---- unweighted copy_lhs / copy_rhs SpMM ---------------------------------------------------------------------------
namespace {

void CheckCsrFacts(const at::Tensor& indptr, const at::Tensor& indices, int64_t rows, int64_t sources, int64_t edges,
                   const char* api, bool check_indices)
{
    const int facts = CsrFacts(indptr, check_indices ? std::optional<at::Tensor>(indices) : std::nullopt, rows, sources,
                               edges);
    TORCH_CHECK(!(facts & 1), api, ": indptr must start at zero and end at nnz");
    TORCH_CHECK(!(facts & 2), api, ": indptr values out of range");
    TORCH_CHECK(!(facts & 4), api, ": indptr must be non-decreasing");
    TORCH_CHECK(!(facts & 8), api, ": indices out of range");
}

int ReduceCode(const std::string& reduce, const char* api)
{
    if (reduce == "sum") {
        return OPSGNN_REDUCE_SUM;
    }
    if (reduce == "max") {
        return OPSGNN_REDUCE_MAX;
    }
    if (reduce == "min") {
        return OPSGNN_REDUCE_MIN;
    }
    TORCH_CHECK(false, api, ": reduce must be 'sum', 'max' or 'min'");
    return -1;
}

// x is [sources, features] or [sources, batches, features] (fp16 kernels of the reference); the middle dimension is
// folded into the feature width because every (batch, feature) column reduces independently.
at::Tensor RunCopyLhs(const at::Tensor& indptr, const at::Tensor& indices, const at::Tensor& x,
                      const std::optional<at::Tensor>& out, int reduce, const char* api)
{
    for (const auto& tensor : {indptr, indices, x}) {
        TORCH_CHECK(tensor.defined() && tensor.device().is_cuda(), api, ": inputs must be CUDA tensors");
        TORCH_CHECK(tensor.device() == x.device(), api, ": inputs must be on the same GPU");
    }
    TORCH_CHECK((x.dim() == 2 || x.dim() == 3) && x.scalar_type() == at::kHalf, api,
                ": x must be a two- or three-dimensional float16 tensor");
    TORCH_CHECK(!x.requires_grad(), api, ": autograd is not supported");
    TORCH_CHECK(indptr.dim() == 1 && indices.dim() == 1 && indptr.numel() >= 1, api,
                ": CSR tensors must be one-dimensional; indptr must be nonempty");
    TORCH_CHECK((indptr.scalar_type() == at::kInt || indptr.scalar_type() == at::kLong) &&
                    indices.scalar_type() == indptr.scalar_type(),
                api, ": CSR tensors must have the same int32/int64 dtype");
    const int64_t rows = indptr.numel() - 1, sources = x.size(0), edges = indices.numel();
    const int64_t batches = x.dim() == 3 ? x.size(1) : 1, features = x.size(-1);
    TORCH_CHECK(features > 0, api, ": dimensions exceed uint32 limits or feature_dim is zero");
    if (out) {
        TORCH_CHECK(out->defined(), api, ": out must be defined");
        bool shape_ok = out->dim() == x.dim() && out->size(0) == rows && out->size(-1) == features;
        if (x.dim() == 3) {
            shape_ok = shape_ok && out->size(1) == batches;
        }
        TORCH_CHECK(out->device() == x.device() && out->scalar_type() == at::kHalf && shape_ok, api,
                    ": out must match output shape, dtype and device");
        TORCH_CHECK(out->is_contiguous() && !out->requires_grad(), api,
                    ": out must be contiguous and must not require gradients");
        TORCH_CHECK(!out->is_alias_of(x) && !out->is_alias_of(indptr) && !out->is_alias_of(indices), api,
                    ": out must not alias any input storage");
    }
    c10::cuda::CUDAGuard guard(x.device());
    if (out) {
        NoteCallerOutput(*out);
    }
    auto ptr = indptr.contiguous();
    auto idx = indices.contiguous();
    CheckCsrFacts(ptr, idx, rows, sources, edges, api, true);
    auto sizes = x.sizes().vec();
    sizes[0] = rows;
    auto result = out ? *out : at::empty(sizes, x.options());
    if (result.numel() == 0) {
        return result;
    }
    CsrReduceCall call;
    call.ptr = ptr;
    call.col = idx;
    call.mat = x.contiguous();
    call.out = result;
    call.rows = rows;
    call.src_rows = sources;
    call.feat = batches * features;
    call.nnz = edges;
    call.arg_none = edges;
    call.reduce = reduce;
    call.extremum = OPSGNN_EXTREMUM_PROPAGATE_NAN;
    RunCsrReduce(call, api);
    return result;
}

}  // namespace

// out[i, :] = x[index[i], :]: the CSR engine run as a gather (one source row per output row, `unit_ptr` = 0..n).
// Used by the sharded SpMM to pack the rows a peer wants and to pull rows into a halo buffer; `x` may be any
// device-accessible memory (a peer's buffer mapped into this process included).  The planner's plan cache keys on
// `unit_ptr`, so a caller that keeps one pointer tensor per exchange partner pays for the plan once.
at::Tensor GatherRows(const at::Tensor& x, const at::Tensor& index, const at::Tensor& unit_ptr, const at::Tensor& out)
{
    const char* api = "gather_rows";
    for (const auto& tensor : {x, index, unit_ptr, out}) {
        TORCH_CHECK(tensor.defined() && tensor.device().is_cuda(), api, ": tensors must be CUDA tensors");
        TORCH_CHECK(tensor.device() == out.device(), api, ": tensors must be on the same GPU");
    }
    TORCH_CHECK(x.dim() == 2 && out.dim() == 2 && x.is_contiguous() && out.is_contiguous(), api,
                ": x and out must be contiguous matrices");
    TORCH_CHECK(x.scalar_type() == out.scalar_type() && x.size(1) == out.size(1), api, ": x and out must agree in dtype and width");
    TORCH_CHECK(x.scalar_type() == at::kFloat || x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16, api,
                ": dtype must be float32, float16 or bfloat16");
    TORCH_CHECK(index.dim() == 1 && unit_ptr.dim() == 1 && index.is_contiguous() && unit_ptr.is_contiguous() &&
                    (index.scalar_type() == at::kInt || index.scalar_type() == at::kLong) &&
                    unit_ptr.scalar_type() == index.scalar_type(),
                api, ": index and unit_ptr must be contiguous int32/int64 vectors of one dtype");
    const int64_t n = index.numel();
    TORCH_CHECK(out.size(0) == n && unit_ptr.numel() == n + 1, api, ": out needs one row and unit_ptr one entry more per index");
    TORCH_CHECK(!out.is_alias_of(x), api, ": out must not alias x");
    if (n == 0 || x.size(1) == 0) {
        return out;
    }
    TORCH_CHECK(x.size(0) > 0, api, ": x has no rows");
    c10::cuda::CUDAGuard guard(out.device());
    CsrReduceCall call;
    call.ptr = unit_ptr;
    call.col = index;
    call.mat = x;
    call.out = out;
    call.rows = n;
    call.src_rows = x.size(0);
    call.feat = x.size(1);
    call.nnz = n;
    call.arg_none = n;
    call.reduce = OPSGNN_REDUCE_SUM;
    RunCsrReduce(call, api);
    return out;
}

// outs[s][i, :] = x[index[start_s + i], :]: the bounded-footprint row gather behind the exchange step of the sharded SpMM.
// `outs` are contiguous [rows_s, K] matrices whose row counts add up to index.numel(); they may be views of a peer's
// symmetric-memory buffer (the kernel writes them with plain stores).  `max_ctas` caps the grid (0 = no cap).
void GatherRowsInto(const at::Tensor& x, const at::Tensor& index, const std::vector<at::Tensor>& outs, int64_t max_ctas)
{
    const char* api = "gather_rows_into";
    TORCH_CHECK(!outs.empty() && outs.size() <= OPSGNN_GATHER_MAX_SEGMENTS, api, ": between 1 and ",
                OPSGNN_GATHER_MAX_SEGMENTS, " output segments");
    TORCH_CHECK(x.defined() && x.device().is_cuda() && index.defined() && index.device() == x.device(), api,
                ": x and index must be CUDA tensors on one GPU");
    TORCH_CHECK(x.dim() == 2 && x.is_contiguous(), api, ": x must be a contiguous matrix");
    TORCH_CHECK(index.dim() == 1 && index.is_contiguous() &&
                    (index.scalar_type() == at::kInt || index.scalar_type() == at::kLong),
                api, ": index must be a contiguous int32/int64 vector");
    const int64_t row_bytes = x.size(1) * static_cast<int64_t>(x.element_size());
    TORCH_CHECK(row_bytes % 16 == 0, api, ": a row must be a multiple of 16 bytes");
    std::vector<int64_t> counts;
    std::vector<void*> bases;
    int64_t total = 0;
    for (const auto& out : outs) {
        TORCH_CHECK(out.defined() && out.device().is_cuda() && out.dim() == 2 && out.is_contiguous() &&
                        out.scalar_type() == x.scalar_type() && out.size(1) == x.size(1),
                    api, ": every output must be a contiguous CUDA matrix of x's dtype and width");
        TORCH_CHECK(!out.is_alias_of(x), api, ": an output must not alias x");
        counts.push_back(out.size(0));
        bases.push_back(out.data_ptr());
        total += out.size(0);
    }
    TORCH_CHECK(total == index.numel(), api, ": the outputs must hold one row per index");
    if (total == 0 || row_bytes == 0) {
        return;
    }
    TORCH_CHECK(x.size(0) > 0, api, ": x has no rows");
    c10::cuda::CUDAGuard guard(x.device());
    CheckStatus(opsgnn_gather_rows(x.const_data_ptr(), index.const_data_ptr(), DtypeId(index.scalar_type(), api), total,
                                   x.size(0), row_bytes, static_cast<int>(outs.size()), counts.data(), bases.data(),
                                   static_cast<int>(max_ctas), CurrentStream(x)),
                api);
}

// dst <- src with one cudaMemcpyAsync on the current stream: both contiguous, same dtype and size, `dst` in this GPU's
// memory or in a peer's block of symmetric memory.  The driver runs such a copy on a copy engine, so an exchange made
// of these takes no SM slot from a product running beside it (one call per copy; no batched-copy API is used).
void CopyRowsAsync(const at::Tensor& src, const at::Tensor& dst)
{
    const char* api = "copy_rows_async";
    TORCH_CHECK(src.defined() && dst.defined() && src.device().is_cuda() && dst.device().is_cuda(), api,
                ": src and dst must be CUDA tensors");
    TORCH_CHECK(src.is_contiguous() && dst.is_contiguous() && src.scalar_type() == dst.scalar_type() &&
                    src.numel() == dst.numel(),
                api, ": src and dst must be contiguous with one dtype and size");
    if (src.numel() == 0) {
        return;
    }
    c10::cuda::CUDAGuard guard(src.device());
    const cudaError_t status = cudaMemcpyAsync(dst.data_ptr(), src.const_data_ptr(), src.nbytes(), cudaMemcpyDeviceToDevice,
                                               static_cast<cudaStream_t>(CurrentStream(src)));
    TORCH_CHECK(status == cudaSuccess, api, ": ", cudaGetErrorString(status));
}

// out[r, :] = sum_e value[e] * x[col[e], :] written into a caller-provided `out` (a row range of a larger matrix is
// fine: any contiguous [rows, K] view).  The staged sharded SpMM produces its output stage by stage with this; the
// structure is trusted (it was validated when the shard was built), so no validation pass runs here.
at::Tensor CsrSpmmInto(const at::Tensor& ptr, const at::Tensor& col, const std::optional<at::Tensor>& value,
                       const at::Tensor& x, const at::Tensor& out)
{
    const char* api = "csr_spmm_into";
    for (const auto& tensor : {ptr, col, x, out}) {
        TORCH_CHECK(tensor.defined() && tensor.device().is_cuda(), api, ": tensors must be CUDA tensors");
        TORCH_CHECK(tensor.device() == out.device(), api, ": tensors must be on the same GPU");
    }
    TORCH_CHECK(x.dim() == 2 && out.dim() == 2 && x.is_contiguous() && out.is_contiguous(), api,
                ": x and out must be contiguous matrices");
    TORCH_CHECK(x.scalar_type() == out.scalar_type() && x.size(1) == out.size(1), api, ": x and out must agree in dtype and width");
    TORCH_CHECK(x.scalar_type() == at::kFloat || x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16, api,
                ": dtype must be float32, float16 or bfloat16");
    TORCH_CHECK(ptr.dim() == 1 && col.dim() == 1 && ptr.numel() >= 1 && ptr.is_contiguous() && col.is_contiguous() &&
                    (ptr.scalar_type() == at::kInt || ptr.scalar_type() == at::kLong) && col.scalar_type() == ptr.scalar_type(),
                api, ": ptr and col must be contiguous int32/int64 vectors of one dtype");
    const int64_t rows = ptr.numel() - 1;
    TORCH_CHECK(out.size(0) == rows, api, ": out needs one row per CSR row");
    TORCH_CHECK(!out.is_alias_of(x), api, ": out must not alias x");
    if (value) {
        TORCH_CHECK(value->defined() && value->device() == out.device() && value->scalar_type() == x.scalar_type() &&
                        value->dim() == 1 && value->numel() == col.numel() && value->is_contiguous(),
                    api, ": value must be a contiguous [E] vector of x's dtype");
    }
    if (rows == 0 || x.size(1) == 0) {
        return out;
    }
    TORCH_CHECK(col.numel() == 0 || x.size(0) > 0, api, ": x has no rows");
    c10::cuda::CUDAGuard guard(out.device());
    CsrReduceCall call;
    call.ptr = ptr;
    call.col = col;
    if (value) {
        call.val = *value;
        call.value_width = 1;
    }
    call.mat = x;
    call.out = out;
    call.rows = rows;
    call.src_rows = x.size(0);
    call.feat = x.size(1);
    call.nnz = col.numel();
    call.arg_none = col.numel();
    call.reduce = OPSGNN_REDUCE_SUM;
    RunCsrReduce(call, api);
    return out;
}

at::Tensor SpmmSumCsr(const at::Tensor& indptr, const at::Tensor& indices, const at::Tensor& x,
                      const std::optional<at::Tensor>& out)
{
    return RunCopyLhs(indptr, indices, x, out, OPSGNN_REDUCE_SUM, "spmm_sum_csr");
}

at::Tensor SpmmMaxCsr(const at::Tensor& indptr, const at::Tensor& indices, const at::Tensor& x,
                      const std::optional<at::Tensor>& out)
{
    return RunCopyLhs(indptr, indices, x, out, OPSGNN_REDUCE_MAX, "spmm_max_csr");
}

at::Tensor SpmmMinCsr(const at::Tensor& indptr, const at::Tensor& indices, const at::Tensor& x,
                      const std::optional<at::Tensor>& out)
{
    return RunCopyLhs(indptr, indices, x, out, OPSGNN_REDUCE_MIN, "spmm_min_csr");
}

at::Tensor UnifiedSpmmCsr(const at::Tensor& indptr, const at::Tensor& indices, const at::Tensor& x,
                          const std::string& op, const std::string& reduce, const std::optional<at::Tensor>& out)
{
    const char* api = "unified_spmm_csr";
    const int reduce_code = ReduceCode(reduce, api);
    TORCH_CHECK(op == "copy_lhs" || op == "copy_rhs", "unified_spmm_csr: op must be 'copy_lhs' or 'copy_rhs'");
    const bool copy_rhs = op == "copy_rhs";
    const int64_t m = indptr.defined() && indptr.dim() == 1 && indptr.numel() >= 1 ? indptr.numel() - 1 : 0;
    const int64_t n = x.defined() && x.dim() == 2 ? x.size(1) : 0;
    for (const auto& tensor : {indptr, indices, x}) {
        TORCH_CHECK(tensor.defined() && tensor.device().is_cuda(), "unified_spmm_csr: inputs must be CUDA tensors");
        TORCH_CHECK(tensor.device() == x.device(), "unified_spmm_csr: inputs must be on the same GPU");
    }
    TORCH_CHECK(x.dim() == 2 && (x.scalar_type() == at::kHalf || x.scalar_type() == at::kFloat),
                "unified_spmm_csr: x must be a two-dimensional float16/float32 tensor");
    TORCH_CHECK(!x.requires_grad(), "unified_spmm_csr: autograd is not supported");
    TORCH_CHECK(indptr.dim() == 1 && indices.dim() == 1 && indptr.numel() >= 1,
                "unified_spmm_csr: CSR tensors must be one-dimensional; indptr must be nonempty");
    TORCH_CHECK((indptr.scalar_type() == at::kInt || indptr.scalar_type() == at::kLong) &&
                    indices.scalar_type() == indptr.scalar_type(),
                "unified_spmm_csr: CSR tensors must have the same int32/int64 dtype");
    if (out) {
        TORCH_CHECK(out->defined() && out->device() == x.device() && out->scalar_type() == x.scalar_type() &&
                        out->dim() == 2 && out->size(0) == m && out->size(1) == n,
                    "unified_spmm_csr: out must match output shape, dtype and device");
        TORCH_CHECK(out->is_contiguous() && !out->requires_grad(),
                    "unified_spmm_csr: out must be contiguous and must not require gradients");
        TORCH_CHECK(!out->is_alias_of(x) && !out->is_alias_of(indptr) && !out->is_alias_of(indices),
                    "unified_spmm_csr: out must not alias any input storage");
    }
    TORCH_CHECK(!copy_rhs || x.scalar_type() == at::kFloat, "unified_spmm_csr: copy_rhs supports only float32");
    c10::cuda::CUDAGuard guard(x.device());
    if (out) {
        NoteCallerOutput(*out);
    }
    const int64_t k = x.size(0);
    const int64_t nnz = indices.numel();
    auto ptr = indptr.contiguous();
    auto idx = indices.contiguous();
    CheckCsrFacts(ptr, idx, m, k, nnz, api, !copy_rhs);
    if (copy_rhs) {
        TORCH_CHECK(k == nnz, "unified_spmm_csr: copy_rhs requires x.size(0) == indices.numel()");
    }
    TORCH_CHECK(n > 0, "unified_spmm_csr: dimensions exceed uint32 limits or feature_dim is zero");
    auto result = out ? *out : at::empty({m, n}, x.options());
    if (m == 0) {
        return result;
    }
    CsrReduceCall call;
    call.ptr = ptr;
    if (!copy_rhs) {
        call.col = idx;  // copy_rhs reduces consecutive edge rows: col(e) = e
    }
    call.mat = x.contiguous();
    call.out = result;
    call.rows = m;
    call.src_rows = k;
    call.feat = n;
    call.nnz = nnz;
    call.arg_none = nnz;
    call.reduce = reduce_code;
    call.extremum = OPSGNN_EXTREMUM_PROPAGATE_NAN;
    RunCsrReduce(call, api);
    return result;
}

// out[r, :] = reduce_e weight[e, group(k)] * x[indices[e], k] for the `mul` message of spmm / bspmm with an edge operand
// that broadcasts over trailing feature dimensions (python/ops_gnn/spmm.py:148-162 of the reference materialises the
// [E, ...] messages instead).  x is [sources, K] after flattening, weight is [E, W] with W dividing K.
at::Tensor SpmmWeightedCsr(const at::Tensor& indptr, const at::Tensor& indices, const at::Tensor& x,
                           const at::Tensor& weight, const std::string& reduce)
{
    const char* api = "spmm_weighted_csr";
    for (const auto& tensor : {indptr, indices, x, weight}) {
        TORCH_CHECK(tensor.defined() && tensor.device().is_cuda(), api, ": inputs must be CUDA tensors");
        TORCH_CHECK(tensor.device() == x.device(), api, ": inputs must be on the same GPU");
    }
    TORCH_CHECK(x.dim() == 2 && weight.dim() == 2 && weight.scalar_type() == x.scalar_type(), api,
                ": x and weight must be two-dimensional with one dtype");
    TORCH_CHECK(x.scalar_type() == at::kFloat || x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16, api,
                ": features must be float32, float16 or bfloat16");
    TORCH_CHECK(indptr.dim() == 1 && indices.dim() == 1 && indptr.numel() >= 1 &&
                    (indptr.scalar_type() == at::kInt || indptr.scalar_type() == at::kLong) &&
                    indices.scalar_type() == indptr.scalar_type(),
                api, ": CSR tensors must be one-dimensional with the same int32/int64 dtype");
    const int64_t rows = indptr.numel() - 1, sources = x.size(0), feat = x.size(1), edges = indices.numel();
    const int64_t width = weight.size(1);
    TORCH_CHECK(weight.size(0) == edges && width >= 1 && feat % width == 0, api,
                ": weight must be [E, W] with W dividing the feature width");
    int code = OPSGNN_REDUCE_SUM;
    if (reduce == "mean") {
        code = OPSGNN_REDUCE_MEAN;
    } else if (reduce == "max") {
        code = OPSGNN_REDUCE_MAX;
    } else if (reduce == "min") {
        code = OPSGNN_REDUCE_MIN;
    } else {
        TORCH_CHECK(reduce == "sum", api, ": reduce must be sum, mean, max or min");
    }
    c10::cuda::CUDAGuard guard(x.device());
    auto ptr = indptr.contiguous();
    auto idx = indices.contiguous();
    CheckCsrFacts(ptr, idx, rows, sources, edges, api, true);
    auto out = at::empty({rows, feat}, x.options());
    if (out.numel() == 0) {
        return out;
    }
    CsrReduceCall call;
    call.ptr = ptr;
    call.col = idx;
    call.val = weight.contiguous();
    call.mat = x.contiguous();
    call.out = out;
    call.rows = rows;
    call.src_rows = sources;
    call.feat = feat;
    call.nnz = edges;
    call.value_width = width;
    call.arg_none = edges;
    call.reduce = code;
    call.extremum = OPSGNN_EXTREMUM_PROPAGATE_NAN;
    RunCsrReduce(call, api);
    return out;
}

}  // namespace opsgnn
