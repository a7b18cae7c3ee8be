// LayerNorm, GroupNorm and the cumulative scans on the "vulkan" device.
//
// Replaces native_layer_norm_vulkan / native_layer_norm_backward (src/api/decompositions.cpp:775-812 with
// layer_norm_shader / layer_norm_backward_shader, src/api/ops/norm.cpp:264-325), native_group_norm and cumsum_out_vulkan /
// cumprod_out_vulkan / logcumsumexp_vulkan (src/api/ops/scan.cpp:104-126). The kernels are tvk_layernorm_*,
// tvk_groupnorm_* and tvk_scan of the C-ABI; floating types other than fp32 / fp16 / bf16 raise (no CPU fallback).
#include "common.h"

#include <ATen/native/Resize.h>

namespace {

using namespace tvk_aten;

void require_hot(const at::Tensor& t, const char* op) {
    if (!is_hot_float(t.scalar_type())) TVK_NOT_IMPLEMENTED(op, " for dtype ", t.scalar_type());
}

at::Tensor opt_param(const c10::optional<at::Tensor>& p, at::ScalarType dtype) {
    if (p.has_value() && p->defined()) return contiguous_vulkan(p->to(dtype));
    return at::Tensor();
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> native_layer_norm(const at::Tensor& input, c10::SymIntArrayRef normalized_shape,
                                                                 const c10::optional<at::Tensor>& weight, const c10::optional<at::Tensor>& bias, double eps) {
    require_hot(input, "native_layer_norm");
    const std::vector<int64_t> shape = C10_AS_INTARRAYREF_SLOW(normalized_shape).vec();
    const int64_t nnorm = (int64_t)shape.size(), ndim = input.dim();
    TORCH_CHECK(nnorm >= 1, "Expected normalized_shape to be at least 1-dimensional, i.e., containing at least one element, but got normalized_shape = ",
                at::IntArrayRef(shape));
    TORCH_CHECK(ndim >= nnorm && input.sizes().slice(ndim - nnorm).equals(shape), "Given normalized_shape=", at::IntArrayRef(shape),
                ", expected input with shape [*, ...], but got input of size", input.sizes());
    TORCH_CHECK(!weight.has_value() || !weight->defined() || weight->sizes().equals(shape), "Expected weight to be of same shape as normalized_shape");
    TORCH_CHECK(!bias.has_value() || !bias->defined() || bias->sizes().equals(shape), "Expected bias to be of same shape as normalized_shape");
    int64_t cols = 1;
    for (int64_t s : shape) cols *= s;
    at::Tensor x = contiguous_vulkan(input);
    const int64_t rows = cols ? x.numel() / cols : 0;
    at::Tensor w = opt_param(weight, input.scalar_type()), b = opt_param(bias, input.scalar_type());
    at::Tensor y = empty_like_contig(x);
    std::vector<int64_t> stat_shape(input.sizes().begin(), input.sizes().end() - nnorm);
    for (int64_t i = 0; i < nnorm; ++i) stat_shape.push_back(1);
    at::Tensor mean = empty_vulkan(stat_shape, at::kFloat, input.device()), rstd = empty_vulkan(stat_shape, at::kFloat, input.device());
    if (x.numel()) {
        DeviceScope scope(input);
        TVK_CALL(tvk_layernorm_forward(to_tvk_dtype(input.scalar_type()), y.data_ptr(), (float*)mean.data_ptr(), (float*)rstd.data_ptr(), x.data_ptr(),
                                       w.defined() ? w.data_ptr() : nullptr, b.defined() ? b.data_ptr() : nullptr, rows, cols, eps, scope.stream));
    }
    return {y, mean, rstd};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> native_layer_norm_backward(const at::Tensor& grad_out, const at::Tensor& input,
                                                                          c10::SymIntArrayRef normalized_shape, const at::Tensor& mean,
                                                                          const at::Tensor& rstd, const c10::optional<at::Tensor>& weight,
                                                                          const c10::optional<at::Tensor>& bias, std::array<bool, 3> mask) {
    require_hot(input, "native_layer_norm_backward");
    const std::vector<int64_t> shape = C10_AS_INTARRAYREF_SLOW(normalized_shape).vec();
    int64_t cols = 1;
    for (int64_t s : shape) cols *= s;
    at::Tensor x = contiguous_vulkan(input), g = contiguous_vulkan(grad_out.to(input.scalar_type()));
    at::Tensor mu = contiguous_vulkan(mean.to(at::kFloat)), rs = contiguous_vulkan(rstd.to(at::kFloat));
    at::Tensor w = opt_param(weight, input.scalar_type());
    const int64_t rows = cols ? x.numel() / cols : 0;
    at::Tensor gx, gw, gb;
    if (mask[0]) gx = empty_like_contig(x);
    const bool want_w = mask[1] && weight.has_value() && weight->defined();
    const bool want_b = mask[2] && bias.has_value() && bias->defined();
    if (want_w) gw = empty_vulkan(shape, input.scalar_type(), input.device());
    if (want_b) gb = empty_vulkan(shape, input.scalar_type(), input.device());
    if (cols) {
        DeviceScope scope(input);
        uint64_t ws_bytes = 0;
        TVK_CALL(tvk_layernorm_backward_workspace_size(rows, cols, &ws_bytes));
        Workspace ws(scope.device, (want_w || want_b) ? ws_bytes : 0);
        TVK_CALL(tvk_layernorm_backward(to_tvk_dtype(input.scalar_type()), mask[0] ? gx.data_ptr() : nullptr, want_w ? gw.data_ptr() : nullptr,
                                        want_b ? gb.data_ptr() : nullptr, g.data_ptr(), x.data_ptr(), w.defined() ? w.data_ptr() : nullptr,
                                        (const float*)mu.data_ptr(), (const float*)rs.data_ptr(), rows, cols, ws.ptr, ws.bytes, scope.stream));
    }
    return {gx, gw, gb};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> native_group_norm(const at::Tensor& input, const c10::optional<at::Tensor>& weight,
                                                                 const c10::optional<at::Tensor>& bias, c10::SymInt N, c10::SymInt C, c10::SymInt HxW,
                                                                 int64_t group, double eps) {
    require_hot(input, "native_group_norm");
    const int64_t n = N.expect_int(), c = C.expect_int(), hw = HxW.expect_int();
    TORCH_CHECK(group > 0 && c % group == 0, "Expected number of channels in input to be divisible by num_groups, but got input of shape ", input.sizes(),
                " and num_groups=", group);
    at::Tensor x = contiguous_vulkan(input);
    at::Tensor w = opt_param(weight, input.scalar_type()), b = opt_param(bias, input.scalar_type());
    at::Tensor y = empty_like_contig(x);
    at::Tensor mean = empty_vulkan({n, group}, at::kFloat, input.device()), rstd = empty_vulkan({n, group}, at::kFloat, input.device());
    if (x.numel()) {
        DeviceScope scope(input);
        TVK_CALL(tvk_groupnorm_forward(to_tvk_dtype(input.scalar_type()), y.data_ptr(), (float*)mean.data_ptr(), (float*)rstd.data_ptr(), x.data_ptr(),
                                       w.defined() ? w.data_ptr() : nullptr, b.defined() ? b.data_ptr() : nullptr, n, c, hw, group, eps, scope.stream));
    }
    return {y, mean, rstd};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> native_group_norm_backward(const at::Tensor& grad_out, const at::Tensor& input, const at::Tensor& mean,
                                                                          const at::Tensor& rstd, const c10::optional<at::Tensor>& weight, c10::SymInt N,
                                                                          c10::SymInt C, c10::SymInt HxW, int64_t group, std::array<bool, 3> mask) {
    require_hot(input, "native_group_norm_backward");
    const int64_t n = N.expect_int(), c = C.expect_int(), hw = HxW.expect_int();
    at::Tensor x = contiguous_vulkan(input), g = contiguous_vulkan(grad_out.to(input.scalar_type()));
    at::Tensor mu = contiguous_vulkan(mean.to(at::kFloat)), rs = contiguous_vulkan(rstd.to(at::kFloat));
    at::Tensor w = opt_param(weight, input.scalar_type());
    at::Tensor gx, gw, gb;
    if (mask[0]) gx = empty_like_contig(x);
    if (mask[1]) gw = empty_vulkan({c}, input.scalar_type(), input.device());
    if (mask[2]) gb = empty_vulkan({c}, input.scalar_type(), input.device());
    if (c) {
        DeviceScope scope(input);
        TVK_CALL(tvk_groupnorm_backward(to_tvk_dtype(input.scalar_type()), mask[0] ? gx.data_ptr() : nullptr, mask[1] ? gw.data_ptr() : nullptr,
                                        mask[2] ? gb.data_ptr() : nullptr, g.data_ptr(), x.data_ptr(), w.defined() ? w.data_ptr() : nullptr,
                                        (const float*)mu.data_ptr(), (const float*)rs.data_ptr(), n, c, hw, group, scope.stream));
    }
    return {gx, gw, gb};
}

// ---- scans ------------------------------------------------------------------------------------------------------------
at::Tensor scan_impl(const at::Tensor& self, int64_t dim, c10::optional<at::ScalarType> dtype, int op, const char* name) {
    at::ScalarType out_dtype = dtype.value_or(at::isIntegralType(self.scalar_type(), true) ? at::kLong : self.scalar_type());
    at::Tensor x = self.scalar_type() == out_dtype ? self : self.to(out_dtype);
    if (!(is_hot_float(out_dtype) || (out_dtype == at::kLong && op != TVK_SCAN_LOGADDEXP))) TVK_NOT_IMPLEMENTED(name, " for dtype ", out_dtype);
    x = contiguous_vulkan(x);
    at::Tensor out = empty_like_contig(x);
    if (x.dim() == 0) {
        out.copy_(x);
        return out;
    }
    dim = at::maybe_wrap_dim(dim, x.dim());
    int64_t outer = 1, inner = 1;
    for (int64_t d = 0; d < dim; ++d) outer *= x.size(d);
    for (int64_t d = dim + 1; d < x.dim(); ++d) inner *= x.size(d);
    if (x.numel()) {
        DeviceScope scope(self);
        TVK_CALL(tvk_scan(op, to_tvk_dtype(out_dtype), out.data_ptr(), x.data_ptr(), outer, x.size(dim), inner, scope.stream));
    }
    return out;
}

at::Tensor& cumsum_out(const at::Tensor& self, int64_t dim, c10::optional<at::ScalarType> dtype, at::Tensor& out) {
    at::Tensor r = scan_impl(self, dim, dtype, TVK_SCAN_SUM, "cumsum");
    at::native::resize_output(out, r.sizes());
    out.copy_(r);
    return out;
}
at::Tensor& cumprod_out(const at::Tensor& self, int64_t dim, c10::optional<at::ScalarType> dtype, at::Tensor& out) {
    at::Tensor r = scan_impl(self, dim, dtype, TVK_SCAN_PROD, "cumprod");
    at::native::resize_output(out, r.sizes());
    out.copy_(r);
    return out;
}
at::Tensor logcumsumexp(const at::Tensor& self, int64_t dim) { return scan_impl(self, dim, c10::nullopt, TVK_SCAN_LOGADDEXP, "logcumsumexp"); }
at::Tensor& logcumsumexp_out(const at::Tensor& self, int64_t dim, at::Tensor& out) {
    at::Tensor r = scan_impl(self, dim, c10::nullopt, TVK_SCAN_LOGADDEXP, "logcumsumexp");
    at::native::resize_output(out, r.sizes());
    out.copy_(r);
    return out;
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("native_layer_norm", &native_layer_norm);
    m.impl("native_layer_norm_backward", &native_layer_norm_backward);
    m.impl("native_group_norm", &native_group_norm);
    m.impl("native_group_norm_backward", &native_group_norm_backward);
    m.impl("cumsum.out", &cumsum_out);
    m.impl("cumprod.out", &cumprod_out);
    m.impl("logcumsumexp", &logcumsumexp);
    m.impl("logcumsumexp.out", &logcumsumexp_out);
}
