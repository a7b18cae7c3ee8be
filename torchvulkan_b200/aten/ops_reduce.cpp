// Reductions, arg-reductions, sort and top-k for the "vulkan" device.
//
// Counterparts in the reference: sum_dim_vulkan / mean_dim_vulkan / reduce_dims_vulkan
// (src/api/ops/reduce.cpp:207-376), argreduce (reduce.cpp:424-502), sort / topk
// (src/api/ops/sort.cpp:19-140). Half and bfloat16 inputs accumulate in fp32 and are rounded
// once at the end (reduce.cpp:266-274). The reference issues one dispatch per reduced dim
// (reduce.cpp:258-261); here every run of adjacent reduced dims is one launch.
#include "common.h"

#include <ATen/WrapDimUtilsMulti.h>
#include <ATen/native/ReduceOpsUtils.h>

namespace tvk_aten {
namespace {

struct Run { int64_t first, last; };  // inclusive range of adjacent reduced dims

std::vector<Run> runs_of(const std::vector<bool>& reduced) {
    std::vector<Run> runs;
    const int64_t nd = (int64_t)reduced.size();
    for (int64_t d = 0; d < nd;) {
        if (!reduced[d]) { ++d; continue; }
        int64_t e = d;
        while (e + 1 < nd && reduced[e + 1]) ++e;
        runs.push_back({d, e});
        d = e + 1;
    }
    return runs;
}

at::Tensor reduce_run(int op, const at::Tensor& x, int64_t first, int64_t last, at::ScalarType out_dtype) {
    int64_t outer = 1, red = 1, inner = 1;
    std::vector<int64_t> oshape;
    for (int64_t d = 0; d < x.dim(); ++d) {
        if (d < first) { outer *= x.size(d); oshape.push_back(x.size(d)); }
        else if (d <= last) red *= x.size(d);
        else { inner *= x.size(d); oshape.push_back(x.size(d)); }
    }
    at::Tensor out = empty_vulkan(oshape, out_dtype, x.device());
    if (out.numel() == 0) return out;
    DeviceScope scope(x);
    uint64_t ws_bytes = 0;
    TVK_CALL(tvk_reduce_workspace_size(outer, red, inner, &ws_bytes));
    Workspace ws(scope.device, ws_bytes);
    TVK_CALL(tvk_reduce(op, to_tvk_dtype(x.scalar_type()), to_tvk_dtype(out_dtype), out.data_ptr(), x.data_ptr(), outer, red, inner, ws.ptr,
                        ws.bytes, scope.stream));
    return out;
}

at::Tensor reduce_dims(int op, const at::Tensor& self, at::OptionalIntArrayRef dims, bool keepdim, c10::optional<at::ScalarType> dtype,
                       const char* name) {
    at::ScalarType in_st = self.scalar_type();
    at::ScalarType out_st = dtype.value_or(in_st);
    at::Tensor x = self;
    if (c10::isIntegralType(in_st, true) && (op == TVK_R_SUM)) {
        if (!(dtype.has_value() && is_hot_float(*dtype))) {
            // Integer (and boolean) sums promote to int64 in ATen and must be exact: the reduced dimensions are moved last and
            // folded into one, scanned by the 64-bit cumulative sum, and the last column is the result. Counts and index
            // bookkeeping, not a hot path.
            TORCH_CHECK(!dtype.has_value() || c10::isIntegralType(*dtype, false), "torchvulkan [NOT IMPLEMENTED]: ", name, " of ", in_st, " into ", *dtype);
            const int64_t nd = self.dim();
            std::vector<bool> red(nd, false);
            if (!dims.has_value() || dims->empty()) std::fill(red.begin(), red.end(), true);
            else for (int64_t d : *dims) red[at::maybe_wrap_dim(d, nd)] = true;
            std::vector<int64_t> perm, kept_shape, keep_shape;
            int64_t count = 1;
            for (int64_t d = 0; d < nd; ++d) {
                keep_shape.push_back(red[d] ? 1 : self.size(d));
                if (!red[d]) { perm.push_back(d); kept_shape.push_back(self.size(d)); }
            }
            for (int64_t d = 0; d < nd; ++d)
                if (red[d]) { perm.push_back(d); count *= self.size(d); }
            at::Tensor result;
            if (nd == 0) result = self.to(at::kLong);
            else if (count == 0) result = at::zeros(kept_shape, self.options().dtype(at::kLong));
            else {
                std::vector<int64_t> folded(kept_shape);
                folded.push_back(count);
                at::Tensor y = contiguous_vulkan(self.to(at::kLong).permute(perm)).reshape(folded);
                result = at::cumsum(y, -1).select(-1, count - 1);
            }
            result = result.to(dtype.value_or(at::kLong));
            return (keepdim && nd > 0) ? result.reshape(keep_shape) : result;
        }
        x = self.to(*dtype);
        in_st = *dtype;
    }
    if (!is_hot_float(in_st) || !is_hot_float(out_st)) TVK_NOT_IMPLEMENTED(name, " for dtype ", in_st, " -> ", out_st, " on the vulkan device");
    x = contiguous_vulkan(x);
    const int64_t nd = x.dim();
    std::vector<bool> reduced(nd, false);
    if (!dims.has_value() || dims->empty()) {
        std::fill(reduced.begin(), reduced.end(), true);
    } else {
        for (int64_t d : *dims) reduced[at::maybe_wrap_dim(d, nd)] = true;
    }
    std::vector<int64_t> keep_shape;
    for (int64_t d = 0; d < nd; ++d) keep_shape.push_back(reduced[d] ? 1 : x.size(d));

    if (nd == 0) {  // a scalar: the reduction is a copy (mean/sum/amax of one element)
        at::Tensor out = x.to(out_st).clone();
        return out;
    }
    const auto runs = runs_of(reduced);
    if (runs.empty()) return x.to(out_st).clone();
    int64_t count = 1;
    for (int64_t d = 0; d < nd; ++d) if (reduced[d]) count *= x.size(d);
    if (op == TVK_R_AMAX || op == TVK_R_AMIN)
        TORCH_CHECK(count > 0, name, "(): Expected reduction dim to be specified for input.numel() == 0. Specify the reduction dim with the 'dim' argument.");

    // Runs are folded from the innermost outwards; intermediates stay in fp32.
    at::Tensor cur = x;
    const bool multi = runs.size() > 1;
    for (size_t r = runs.size(); r-- > 0;) {
        const bool final_run = r == 0;
        const int step_op = (op == TVK_R_MEAN && multi) ? TVK_R_SUM : op;
        cur = reduce_run(step_op, cur, runs[r].first, runs[r].last, final_run && !(op == TVK_R_MEAN && multi) ? out_st : at::kFloat);
    }
    if (op == TVK_R_MEAN && multi) {
        cur = at::mul(cur, at::Scalar(count > 0 ? 1.0 / (double)count : std::numeric_limits<double>::quiet_NaN())).to(out_st);
    }
    if (keepdim) return cur.view(keep_shape);
    return cur;
}

at::Tensor sum_dim(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, c10::optional<at::ScalarType> dtype) {
    return reduce_dims(TVK_R_SUM, self, dim, keepdim, dtype, "sum");
}
at::Tensor mean_dim(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, c10::optional<at::ScalarType> dtype) {
    TORCH_CHECK(at::isFloatingType(dtype.value_or(self.scalar_type())), "mean(): could not infer output dtype. Input dtype must be either a floating point or complex dtype. Got: ",
                self.scalar_type());
    return reduce_dims(TVK_R_MEAN, self, dim, keepdim, dtype, "mean");
}
at::Tensor amax(const at::Tensor& self, at::IntArrayRef dim, bool keepdim) { return reduce_dims(TVK_R_AMAX, self, dim, keepdim, c10::nullopt, "amax"); }
at::Tensor amin(const at::Tensor& self, at::IntArrayRef dim, bool keepdim) { return reduce_dims(TVK_R_AMIN, self, dim, keepdim, c10::nullopt, "amin"); }

at::Tensor& into(at::Tensor& out, const at::Tensor& r) {
    if (out.sizes() != r.sizes()) out.resize_(r.sizes());
    out.copy_(r);
    return out;
}
at::Tensor& sum_out(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, c10::optional<at::ScalarType> dtype, at::Tensor& out) {
    return into(out, sum_dim(self, dim, keepdim, dtype.has_value() ? dtype : c10::optional<at::ScalarType>(out.scalar_type())));
}
at::Tensor& mean_out(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, c10::optional<at::ScalarType> dtype, at::Tensor& out) {
    return into(out, mean_dim(self, dim, keepdim, dtype.has_value() ? dtype : c10::optional<at::ScalarType>(out.scalar_type())));
}
at::Tensor& amax_out(const at::Tensor& self, at::IntArrayRef dim, bool keepdim, at::Tensor& out) { return into(out, (amax)(self, dim, keepdim)); }
at::Tensor& amin_out(const at::Tensor& self, at::IntArrayRef dim, bool keepdim, at::Tensor& out) { return into(out, (amin)(self, dim, keepdim)); }

at::Tensor argreduce(bool is_max, const at::Tensor& self, c10::optional<int64_t> dim, bool keepdim) {
    if (!is_hot_float(self.scalar_type())) TVK_NOT_IMPLEMENTED(is_max ? "argmax" : "argmin", " for dtype ", self.scalar_type(), " on the vulkan device");
    at::Tensor x = contiguous_vulkan(self);
    int64_t outer = 1, red = 1, inner = 1;
    std::vector<int64_t> oshape, keep_shape;
    if (!dim.has_value()) {
        red = x.numel();
        keep_shape.assign(x.dim(), 1);
    } else {
        const int64_t d0 = at::maybe_wrap_dim(*dim, std::max<int64_t>(x.dim(), 1));
        for (int64_t d = 0; d < x.dim(); ++d) {
            if (d < d0) { outer *= x.size(d); oshape.push_back(x.size(d)); keep_shape.push_back(x.size(d)); }
            else if (d == d0) { red = x.size(d); keep_shape.push_back(1); }
            else { inner *= x.size(d); oshape.push_back(x.size(d)); keep_shape.push_back(x.size(d)); }
        }
    }
    TORCH_CHECK(red > 0, is_max ? "argmax" : "argmin", "(): Expected reduction dim to be specified for input.numel() == 0. Specify the reduction dim with the 'dim' argument.");
    at::Tensor out = empty_vulkan(oshape, at::kLong, x.device());
    if (out.numel()) {
        DeviceScope scope(x);
        uint64_t ws_bytes = 0;
        TVK_CALL(tvk_reduce_workspace_size(outer, red, inner, &ws_bytes));
        Workspace ws(scope.device, ws_bytes);
        TVK_CALL(tvk_argreduce(is_max ? 1 : 0, to_tvk_dtype(x.scalar_type()), (int64_t*)out.data_ptr(), x.data_ptr(), outer, red, inner, ws.ptr,
                               ws.bytes, scope.stream));
    }
    return keepdim ? out.view(keep_shape) : out;
}
at::Tensor argmax(const at::Tensor& self, c10::optional<int64_t> dim, bool keepdim) { return argreduce(true, self, dim, keepdim); }
at::Tensor argmin(const at::Tensor& self, c10::optional<int64_t> dim, bool keepdim) { return argreduce(false, self, dim, keepdim); }
at::Tensor& argmax_out(const at::Tensor& self, c10::optional<int64_t> dim, bool keepdim, at::Tensor& out) { return into(out, (argmax)(self, dim, keepdim)); }
at::Tensor& argmin_out(const at::Tensor& self, c10::optional<int64_t> dim, bool keepdim, at::Tensor& out) { return into(out, (argmin)(self, dim, keepdim)); }

// Stable sort along `dim`, first k entries (src/api/ops/sort.cpp:118-140: topk = sort + narrow).
std::tuple<at::Tensor, at::Tensor> sort_take(const at::Tensor& self, int64_t k, int64_t dim, bool descending, const char* name) {
    if (!is_hot_float(self.scalar_type())) TVK_NOT_IMPLEMENTED(name, " for dtype ", self.scalar_type(), " on the vulkan device");
    const int64_t nd = std::max<int64_t>(self.dim(), 1);
    dim = at::maybe_wrap_dim(dim, nd);
    at::Tensor x = self.dim() == 0 ? self.reshape({1}) : self;
    const int64_t n = x.size(dim);
    TORCH_CHECK(k >= 0 && k <= n, "selected index k out of range");
    at::Tensor moved = contiguous_vulkan(x.transpose(dim, -1));
    std::vector<int64_t> oshape(moved.sizes().begin(), moved.sizes().end());
    oshape.back() = k;
    at::Tensor values = empty_vulkan(oshape, x.scalar_type(), x.device());
    at::Tensor indices = empty_vulkan(oshape, at::kLong, x.device());
    const int64_t lines = n ? moved.numel() / n : 0;
    if (values.numel()) {
        DeviceScope scope(x);
        const int dt = to_tvk_dtype(x.scalar_type());
        // the kernel takes up to 65535 lines per launch
        for (int64_t l0 = 0; l0 < lines; l0 += 65535) {
            const int64_t nl = std::min<int64_t>(65535, lines - l0);
            uint64_t ws_bytes = 0;
            TVK_CALL(tvk_sort_workspace_size(dt, nl, n, &ws_bytes));
            Workspace ws(scope.device, ws_bytes);
            TVK_CALL(tvk_topk(dt, (char*)values.data_ptr() + l0 * k * values.itemsize(), (int64_t*)indices.data_ptr() + l0 * k,
                              (const char*)moved.data_ptr() + l0 * n * moved.itemsize(), nl, n, k, descending ? 1 : 0, ws.ptr, ws.bytes,
                              scope.stream));
        }
    }
    values = values.transpose(dim, -1);
    indices = indices.transpose(dim, -1);
    if (self.dim() == 0) return {values.reshape({}), indices.reshape({})};
    return {values, indices};
}

std::tuple<at::Tensor, at::Tensor> topk(const at::Tensor& self, c10::SymInt k, int64_t dim, bool largest, bool) {
    return sort_take(self, k.guard_int(__FILE__, __LINE__), dim, largest, "topk");
}
std::tuple<at::Tensor&, at::Tensor&> topk_out(const at::Tensor& self, c10::SymInt k, int64_t dim, bool largest, bool sorted, at::Tensor& values,
                                              at::Tensor& indices) {
    auto r = (topk)(self, k, dim, largest, sorted);
    into(values, std::get<0>(r));
    into(indices, std::get<1>(r));
    return {values, indices};
}
std::tuple<at::Tensor, at::Tensor> sort_stable(const at::Tensor& self, c10::optional<bool>, int64_t dim, bool descending) {
    const int64_t d = at::maybe_wrap_dim(dim, std::max<int64_t>(self.dim(), 1));
    auto r = sort_take(self, self.dim() ? self.size(d) : 1, dim, descending, "sort");
    return {std::get<0>(r).contiguous(), std::get<1>(r).contiguous()};
}
std::tuple<at::Tensor, at::Tensor> sort_plain(const at::Tensor& self, int64_t dim, bool descending) { return sort_stable(self, false, dim, descending); }
std::tuple<at::Tensor&, at::Tensor&> sort_values_stable(const at::Tensor& self, c10::optional<bool> stable, int64_t dim, bool descending,
                                                        at::Tensor& values, at::Tensor& indices) {
    auto r = sort_stable(self, stable, dim, descending);
    into(values, std::get<0>(r));
    into(indices, std::get<1>(r));
    return {values, indices};
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("sum.dim_IntList", &sum_dim);
    m.impl("sum.IntList_out", &sum_out);
    m.impl("mean.dim", &mean_dim);
    m.impl("mean.out", &mean_out);
    m.impl("amax", &amax);
    m.impl("amax.out", &amax_out);
    m.impl("amin", &amin);
    m.impl("amin.out", &amin_out);
    m.impl("argmax", &argmax);
    m.impl("argmax.out", &argmax_out);
    m.impl("argmin", &argmin);
    m.impl("argmin.out", &argmin_out);
    m.impl("topk", &topk);
    m.impl("topk.values", &topk_out);
    m.impl("sort", &sort_plain);
    m.impl("sort.stable", &sort_stable);
    m.impl("sort.values_stable", &sort_values_stable);
}

}  // namespace tvk_aten
