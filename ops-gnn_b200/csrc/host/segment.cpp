// Launch planners of the segment reductions: segment_csr (csrc/npu/segment_csr/op_host/segment_csr.cpp:1663-1706 of
// the reference), segment_coo_forward (csrc/npu/segment_coo/op_host/segment_coo.cpp:1127-1175) and
// segment_logsumexp_forward (csrc/npu/segment_logsumexp/op_host/segment_logsumexp.cpp:133-168).  All three reduce
// runs of consecutive source rows, so they share the CSR reduce engine with col(e) = e; sorted COO indices are first
// turned into pointers by the boundary-scan kernel.
#include "ops.h"

namespace opsgnn {
namespace {

struct SegDims {
    int64_t dim, e1, m, k, nSeg, indptrLast;
};

SegDims CheckedDimensions(const at::Tensor& src, const at::Tensor& indptr)
{
    TORCH_CHECK(indptr.dim() >= 1, "indptr must have at least 1 dim");
    TORCH_CHECK(src.dim() >= indptr.dim(), "src.dim() must be >= indptr.dim()");
    SegDims d{};
    d.dim = indptr.dim() - 1;
    d.e1 = Product(src.sizes(), 0, d.dim);
    d.m = src.size(d.dim);
    d.indptrLast = indptr.size(d.dim);
    d.nSeg = d.indptrLast - 1;
    d.k = Product(src.sizes(), d.dim + 1, src.dim());
    TORCH_CHECK(indptr.scalar_type() == at::kLong, "indptr must be int64, got ", indptr.scalar_type());
    TORCH_CHECK(d.indptrLast >= 1, "indptr last dim must be >= 1");
    for (int64_t i = 0; i < d.dim; ++i) {
        TORCH_CHECK(indptr.size(i) == 1 || indptr.size(i) == src.size(i), "indptr leading dim ", i, " (", indptr.size(i),
                    ") must be 1 or match src (", src.size(i), ")");
    }
    TORCH_CHECK(src.device().is_cuda(), "segment_csr requires CUDA tensors, got ", src.device());
    TORCH_CHECK(indptr.device() == src.device(), "src and indptr must live on the same device");
    TORCH_CHECK(src.layout() == at::kStrided && indptr.layout() == at::kStrided,
                "src and indptr must have strided layout");
    return d;
}

struct Reduction {
    int code;
    bool mean;
    bool extremum;
};

Reduction ParseReduction(const std::string& reduce)
{
    if (reduce == "sum" || reduce == "add") {
        return {OPSGNN_REDUCE_SUM, false, false};
    }
    if (reduce == "mean") {
        return {OPSGNN_REDUCE_MEAN, true, false};
    }
    if (reduce == "min") {
        return {OPSGNN_REDUCE_MIN, false, true};
    }
    TORCH_CHECK(reduce == "max", "reduce value '", reduce, "' is not valid (use sum, add, mean, min or max)");
    return {OPSGNN_REDUCE_MAX, false, true};
}

bool SupportedSegmentDtype(at::ScalarType t)
{
    switch (t) {
        case at::kFloat:
        case at::kHalf:
        case at::kBFloat16:
        case at::kChar:
        case at::kByte:
        case at::kInt:
        case at::kLong:
        case at::kShort:
        case at::kDouble:
            return true;
        default:
            return false;
    }
}

// One engine launch over [batches, length, k] -> [batches, segments, k] with a shared pointer array.
void ReduceShared(const at::Tensor& src, const at::Tensor& ptr, at::Tensor& out, at::Tensor arg, int64_t batches,
                  int64_t length, int64_t segments, int64_t k, const Reduction& reduction, int extremum,
                  const char* api)
{
    const bool integer = !src.is_floating_point();
    CsrReduceCall call;
    call.ptr = ptr;
    call.mat = src;
    call.out = out;
    if (arg.defined()) {
        call.arg = arg;
    }
    call.rows = segments;
    call.src_rows = length;
    call.feat = k;
    call.nnz = length;
    call.batches = batches;
    call.arg_none = length;
    call.reduce = (reduction.mean && integer) ? OPSGNN_REDUCE_SUM : reduction.code;
    call.extremum = extremum;
    RunCsrReduce(call, api);
    if (reduction.mean && integer) {
        CheckStatus(opsgnn_csr_integer_mean(out.data_ptr(), DtypeId(out.scalar_type(), api), ptr.const_data_ptr(),
                                            DtypeId(ptr.scalar_type(), api), segments, k, batches, CurrentStream(out)),
                    api);
    }
}

}  // namespace

std::vector<at::Tensor> segment_csr(at::Tensor src, at::Tensor indptr, std::optional<at::Tensor> outOpt,
                                    const std::string& reduce, bool returnArg)
{
    const auto reduction = ParseReduction(reduce);
    const SegDims dims = CheckedDimensions(src, indptr);
    TORCH_CHECK(SupportedSegmentDtype(src.scalar_type()), "segment_csr unsupported dtype: ", src.scalar_type());
    c10::cuda::CUDAGuard guard(src.device());
    at::Tensor srcC = src.contiguous();
    bool shared = true;
    for (int64_t i = 0; i < dims.dim; ++i) {
        shared = shared && indptr.size(i) == 1;
    }
    at::Tensor ptr = indptr.contiguous();
    if (!shared) {
        std::vector<int64_t> shape(src.sizes().begin(), src.sizes().begin() + dims.dim);
        shape.push_back(dims.indptrLast);
        ptr = ptr.expand(shape).contiguous();
    }
    std::vector<int64_t> outShape(src.sizes().begin(), src.sizes().end());
    outShape[dims.dim] = dims.nSeg;
    const bool has_out = outOpt.has_value() && outOpt->defined();
    at::Tensor out;
    if (has_out) {
        NoteCallerOutput(*outOpt);
        TORCH_CHECK(outOpt->scalar_type() == src.scalar_type(), "out dtype (", outOpt->scalar_type(),
                    ") must match src (", src.scalar_type(), ")");
        TORCH_CHECK(outOpt->sizes() == c10::IntArrayRef(outShape), "out shape ", outOpt->sizes(), " must be ",
                    c10::IntArrayRef(outShape));
        TORCH_CHECK(outOpt->device() == src.device(), "out must live on src's device");
        const bool aliases = outOpt->is_alias_of(src) || outOpt->is_alias_of(indptr);
        out = (outOpt->is_contiguous() && !aliases) ? *outOpt : at::empty(outShape, src.options());
    } else {
        out = at::empty(outShape, src.options());
    }
    at::Tensor argOut;
    if (reduction.extremum && returnArg) {
        argOut = at::empty(outShape, src.options().dtype(at::kLong));
    }
    if (src.numel() == 0) {
        if (!has_out) {
            out.zero_();
        }
        if (argOut.defined()) {
            argOut.fill_(dims.m);
        }
        if (has_out) {
            out = *outOpt;
        }
        return argOut.defined() ? std::vector<at::Tensor>{out, argOut} : std::vector<at::Tensor>{out};
    }
    if (out.numel() > 0) {
        if (shared) {
            ReduceShared(srcC, ptr.reshape({dims.indptrLast}), out, argOut, dims.e1, dims.m, dims.nSeg, dims.k,
                         reduction, OPSGNN_EXTREMUM_PROPAGATE_NAN, "segment_csr");
        } else {
            // Every batch row has its own pointers: one launch per row over views of the packed tensors.
            auto src3 = srcC.reshape({dims.e1, dims.m, dims.k});
            auto out3 = out.reshape({dims.e1, dims.nSeg, dims.k});
            auto arg3 = argOut.defined() ? argOut.reshape({dims.e1, dims.nSeg, dims.k}) : at::Tensor();
            auto ptr2 = ptr.reshape({dims.e1, dims.indptrLast});
            for (int64_t b = 0; b < dims.e1; ++b) {
                at::Tensor out_b = out3[b];
                ReduceShared(src3[b], ptr2[b], out_b, arg3.defined() ? arg3[b] : at::Tensor(), 1, dims.m, dims.nSeg,
                             dims.k, reduction, OPSGNN_EXTREMUM_PROPAGATE_NAN, "segment_csr");
            }
        }
    }
    if (has_out && out.data_ptr() != outOpt->data_ptr()) {
        outOpt->copy_(out);
        out = *outOpt;
    }
    return argOut.defined() ? std::vector<at::Tensor>{out, argOut} : std::vector<at::Tensor>{out};
}

std::tuple<at::Tensor, at::Tensor> segment_coo_forward(at::Tensor src, at::Tensor index,
                                                       std::optional<at::Tensor> optional_out,
                                                       std::optional<int64_t> dim_size, int64_t reduce,
                                                       bool return_arg)
{
    TORCH_CHECK(src.device().is_cuda(), "src must be a CUDA tensor");
    TORCH_CHECK(index.device() == src.device(), "index and src must be on the same GPU");
    TORCH_CHECK(index.scalar_type() == at::kLong, "index must be int64");
    TORCH_CHECK(src.dim() >= 1 && src.dim() <= 8 && index.dim() >= 1 && index.dim() <= src.dim(), "invalid rank");
    TORCH_CHECK(src.layout() == at::kStrided && index.layout() == at::kStrided, "src and index must be strided tensors");
    TORCH_CHECK(reduce >= SEGMENT_COO_SUM && reduce <= SEGMENT_COO_MAX, "invalid reduction");
    TORCH_CHECK(SupportedSegmentDtype(src.scalar_type()), "unsupported src dtype");
    c10::cuda::CUDAGuard guard(src.device());

    const int64_t dim = index.dim() - 1;
    const int64_t length = src.size(dim);
    int64_t before = 1;
    bool shared = true;
    std::vector<int64_t> index_shape;
    for (int64_t d = 0; d < dim; ++d) {
        TORCH_CHECK(index.size(d) == 1 || index.size(d) == src.size(d), "index broadcast mismatch");
        before *= src.size(d);
        index_shape.push_back(src.size(d));
        shared = shared && index.size(d) == 1;
    }
    TORCH_CHECK(index.size(dim) == length, "index length must match reduction dimension");
    index_shape.push_back(length);
    const int64_t after = Product(src.sizes(), dim + 1, src.dim());
    if (!shared) {
        index = index.expand(index_shape);
    }
    index = index.contiguous();
    src = src.contiguous();

    int64_t segments = 0;
    const bool has_out = optional_out.has_value();
    if (has_out) {
        const auto& out = *optional_out;
        NoteCallerOutput(out);
        TORCH_CHECK(out.device() == src.device() && out.scalar_type() == src.scalar_type(),
                    "out device and dtype must match src");
        TORCH_CHECK(out.dim() == src.dim(), "out rank mismatch");
        for (int64_t d = 0; d < src.dim(); ++d) {
            if (d != dim) {
                TORCH_CHECK(out.size(d) == src.size(d), "out shape mismatch");
            }
        }
        segments = out.size(dim);
    } else if (dim_size.has_value()) {
        segments = *dim_size;
    } else if (index.numel() > 0) {
        segments = index.select(dim, length - 1).max().item<int64_t>() + 1;
    }
    TORCH_CHECK(segments >= 0, "dim_size must be non-negative");
    auto shape = src.sizes().vec();
    shape[dim] = segments;
    const bool extremum = reduce >= SEGMENT_COO_MIN;
    at::Tensor fresh = at::empty(shape, src.options());
    at::Tensor arg = extremum && return_arg ? at::empty(shape, src.options().dtype(at::kLong)) : at::Tensor();
    if (fresh.numel() == 0) {
        return {has_out ? *optional_out : fresh, arg};
    }
    Reduction reduction{static_cast<int>(reduce), reduce == SEGMENT_COO_MEAN, extremum};
    // With a caller-provided out the golden semantics seed every reduction from it; the engine reduces from the
    // neutral element and the seed is merged afterwards, so min/max always need the positions.
    at::Tensor arg_work = arg;
    if (extremum && has_out && !arg_work.defined()) {
        arg_work = at::empty(shape, src.options().dtype(at::kLong));
    }
    if (has_out && reduction.mean) {
        reduction.code = OPSGNN_REDUCE_SUM;
        reduction.mean = false;
    }
    const int rule = has_out ? OPSGNN_EXTREMUM_IGNORE_NAN : OPSGNN_EXTREMUM_SEEDED;
    at::Tensor counts;  // [index batches, segments], only for the seeded mean
    const int64_t index_batches = shared ? 1 : before;
    auto index2 = index.reshape({index_batches, length});
    auto ptr_all = at::empty({index_batches, segments + 1}, index.options());
    for (int64_t b = 0; b < index_batches; ++b) {
        CheckStatus(opsgnn_ind2ptr(index2[b].data_ptr<int64_t>(), length, ptr_all[b].data_ptr<int64_t>(), segments,
                                   CurrentStream(src)),
                    "segment_coo");
    }
    if (shared) {
        ReduceShared(src, ptr_all[0], fresh, arg_work, before, length, segments, after, reduction, rule, "segment_coo");
    } else {
        auto src3 = src.reshape({before, length, after});
        auto out3 = fresh.reshape({before, segments, after});
        auto arg3 = arg_work.defined() ? arg_work.reshape({before, segments, after}) : at::Tensor();
        for (int64_t b = 0; b < before; ++b) {
            at::Tensor out_b = out3[b];
            ReduceShared(src3[b], ptr_all[b], out_b, arg3.defined() ? arg3[b] : at::Tensor(), 1, length, segments, after,
                         reduction, rule, "segment_coo");
        }
    }
    if (!has_out) {
        return {fresh, arg};
    }
    // Merge the caller's out as the seed of every segment that received at least one element
    // (test/segment_coo/arch35/golden.py:125-148 of the reference); other segments keep their contents.
    at::Tensor out = *optional_out;
    std::vector<int64_t> count_shape(src.dim(), 1);
    for (int64_t d = 0; d <= dim; ++d) {
        count_shape[d] = d < dim ? (shared ? 1 : src.size(d)) : segments;
    }
    auto count = (ptr_all.slice(1, 1) - ptr_all.slice(1, 0, segments)).reshape(count_shape);
    auto touched = count.gt(0);
    if (reduce == SEGMENT_COO_SUM) {
        out.copy_(at::where(touched, out + fresh, out));
    } else if (reduce == SEGMENT_COO_MEAN) {
        auto total = out + fresh;
        at::Tensor mean;
        if (src.is_floating_point()) {
            mean = total / count.to(src.scalar_type());
        } else {
            auto divisor = count.to(src.scalar_type());
            mean = at::where(divisor.ne(0), at::div(total, at::where(divisor.ne(0), divisor, at::ones_like(divisor)), "trunc"),
                             at::zeros_like(total));
        }
        out.copy_(at::where(touched, mean, out));
    } else {
        auto found = arg_work.ne(length);
        auto better = reduce == SEGMENT_COO_MIN ? fresh.lt(out) : fresh.gt(out);
        auto take = touched.logical_and(found).logical_and(better);
        out.copy_(at::where(take, fresh, out));
        if (arg.defined()) {
            arg.copy_(at::where(take, arg_work, at::full_like(arg_work, length)));
        }
    }
    return {out, arg};
}

at::Tensor segment_logsumexp_forward(const at::Tensor& src, const at::Tensor& indptr)
{
    TORCH_CHECK(src.defined() && src.device().is_cuda(), "segment_logsumexp: src must be a CUDA tensor");
    TORCH_CHECK(indptr.defined() && indptr.device() == src.device(), "segment_logsumexp: indptr must be on src's device");
    TORCH_CHECK(src.dim() >= 1, "segment_logsumexp: src must have at least one dimension");
    TORCH_CHECK(indptr.dim() == 1 && indptr.numel() >= 1, "segment_logsumexp: indptr must be 1-D and nonempty");
    TORCH_CHECK(indptr.scalar_type() == at::kInt || indptr.scalar_type() == at::kLong,
                "segment_logsumexp: indptr must be int32 or int64");
    TORCH_CHECK(src.scalar_type() == at::kFloat || src.scalar_type() == at::kHalf || src.scalar_type() == at::kBFloat16,
                "segment_logsumexp: src must be float16, float32 or bfloat16");
    TORCH_CHECK(src.is_contiguous() && indptr.is_contiguous(), "segment_logsumexp: inputs must be contiguous");
    c10::cuda::CUDAGuard guard(src.device());
    std::vector<int64_t> sizes(src.sizes().begin(), src.sizes().end());
    sizes[0] = indptr.numel() - 1;
    at::Tensor out = at::empty(sizes, src.options());
    if (out.numel() == 0) {
        return out;
    }
    if (src.size(0) == 0) {
        return out.fill_(-std::numeric_limits<float>::infinity());
    }
    CsrReduceCall call;
    call.ptr = indptr;
    call.mat = src;
    call.out = out;
    call.rows = sizes[0];
    call.src_rows = src.size(0);
    call.feat = Product(src.sizes(), 1, src.dim());
    call.nnz = src.size(0);
    call.arg_none = src.size(0);
    call.reduce = OPSGNN_REDUCE_LOGSUMEXP;
    RunCsrReduce(call, "segment_logsumexp");
    return out;
}

}  // namespace opsgnn
