// Elementwise operators of the "vulkan" device: unary, binary (with broadcasting, type promotion
// and scalar operands), comparisons, addcmul/addcdiv/lerp/where, fill.
//
// Counterparts in the reference: unary_op_vulkan (src/api/ops/unary.cpp:76-135 and its 98
// registrations), dispatch_binary_shader (src/api/ops/binary.cpp:60-131), dispatch_addc_shader
// (binary.cpp:711-771), compare.cpp, fill.cpp. As there, type promotion happens on the host
// (binary.cpp:72-73), same-shape dense operands take the flat kernel and everything else the
// strided/broadcast kernel. Unsupported dtypes raise; nothing falls back to the CPU.
#include "common.h"

#include <limits>

namespace tvk_aten {
namespace {

void require_float(const at::Tensor& t, const char* op) {
    if (!is_hot_float(t.scalar_type())) TVK_NOT_IMPLEMENTED(op, " for dtype ", t.scalar_type(), " on the vulkan device");
}

// Same sizes and same dense strides: the flat kernel can walk the storage in memory order.
bool same_dense_layout(const at::Tensor& a, const at::Tensor& b) {
    return a.sizes() == b.sizes() && a.strides() == b.strides() && a.is_non_overlapping_and_dense();
}

at::Tensor alloc_like(const at::Tensor& t, at::ScalarType dtype) {
    if (t.is_non_overlapping_and_dense()) return at::empty_strided(t.sizes(), t.strides(), t.options().dtype(dtype));
    return empty_vulkan(t.sizes(), dtype, t.device());
}

at::Tensor to_dtype(const at::Tensor& t, at::ScalarType dtype) { return t.scalar_type() == dtype ? t : t.to(dtype); }

// A 0-dim CPU tensor (a wrapped Python number or a scalar tensor) used as an operand.
bool is_cpu_scalar(const at::Tensor& t) { return t.device().is_cpu() && t.dim() == 0; }

at::Tensor on_device(const at::Tensor& t, const at::Tensor& like, at::ScalarType dtype) {
    if (is_vulkan(t)) return to_dtype(t, dtype);
    TORCH_CHECK(is_cpu_scalar(t), "Expected all tensors to be on the same device, but found at least two devices, ", like.device(), " and ",
                t.device(), "!");
    return t.to(like.options().dtype(dtype));
}

// ---- unary ------------------------------------------------------------------------------
void unary_into(int op, const at::Tensor& self, at::Tensor& out, const char* name) {
    require_float(self, name);
    TORCH_CHECK(out.scalar_type() == self.scalar_type(), "torchvulkan [ERROR]: ", name, ": out dtype must match the input");
    if (self.numel() == 0) return;
    DeviceScope scope(self);
    const int dt = to_tvk_dtype(self.scalar_type());
    if (same_dense_layout(self, out)) {
        TVK_CALL(tvk_unary(op, dt, out.data_ptr(), self.data_ptr(), self.numel(), scope.stream));
    } else {
        tvk_iter it;
        make_iter(&it, out, {&self});
        TVK_CALL(tvk_unary_strided(op, dt, out.data_ptr(), self.data_ptr(), &it, scope.stream));
    }
}

at::Tensor binary_impl(int op, const at::Tensor& a_in, const at::Tensor& b_in, double alpha, at::Tensor out, const char* name, bool integer_ok = false);
at::Tensor scalar_tensor_like(const at::Scalar& s, const at::Tensor& like);
// neg and abs of integer tensors ride the exact integer kernels: -x = x * -1, |x| = max(x, -x)
template <int OP> at::Tensor unary_fn(const at::Tensor& self);
template <int OP> bool integer_unary(const at::Tensor& self, at::Tensor* result) {
    const at::ScalarType st = self.scalar_type();
    // float64 tensors (torch.amp.GradScaler forms its inverse scale as scale.double().reciprocal().float()) are stored in
    // full width but computed in fp32: this device's kernels compute in fp32, fp16 and bf16
    if (st == at::kDouble) {
        *result = unary_fn<OP>(self.to(at::kFloat)).to(at::kDouble);
        return true;
    }
    if (!(st == at::kLong || st == at::kInt) || !(OP == TVK_U_NEG || OP == TVK_U_ABS)) return false;
    at::Tensor negated = binary_impl(TVK_B_MUL, self, scalar_tensor_like(-1, self), 1.0, {}, "neg", true);
    *result = OP == TVK_U_NEG ? negated : binary_impl(TVK_B_MAXIMUM, self, negated, 1.0, {}, "abs", true);
    return true;
}
template <int OP> at::Tensor unary_fn(const at::Tensor& self) {
    at::Tensor r;
    if (integer_unary<OP>(self, &r)) return r;
    at::Tensor out = alloc_like(self, self.scalar_type());
    unary_into(OP, self, out, "unary op");
    return out;
}
template <int OP> at::Tensor& unary_fn_(at::Tensor& self) {
    at::Tensor r;
    if (integer_unary<OP>(self, &r)) { self.copy_(r); return self; }
    unary_into(OP, self, self, "unary op");
    return self;
}
template <int OP> at::Tensor& unary_out(const at::Tensor& self, at::Tensor& out) {
    if (out.sizes() != self.sizes()) out.resize_(self.sizes());
    at::Tensor r;
    if (integer_unary<OP>(self, &r)) { out.copy_(r); return out; }
    unary_into(OP, self, out, "unary op");
    return out;
}

// true for approximate='tanh', false for 'none' (src/api/ops/unary.cpp:229-230)
bool gelu_is_tanh(c10::string_view approximate) {
    if (approximate != "none" && approximate != "tanh") TVK_NOT_IMPLEMENTED("gelu(approximate='", approximate, "')");
    return approximate == "tanh";
}
at::Tensor gelu(const at::Tensor& self, c10::string_view approximate) {
    return gelu_is_tanh(approximate) ? unary_fn<TVK_U_GELU_TANH>(self) : unary_fn<TVK_U_GELU>(self);
}
at::Tensor& gelu_(at::Tensor& self, c10::string_view approximate) {
    return gelu_is_tanh(approximate) ? unary_fn_<TVK_U_GELU_TANH>(self) : unary_fn_<TVK_U_GELU>(self);
}
at::Tensor& gelu_out(const at::Tensor& self, c10::string_view approximate, at::Tensor& out) {
    return gelu_is_tanh(approximate) ? unary_out<TVK_U_GELU_TANH>(self, out) : unary_out<TVK_U_GELU>(self, out);
}

// ---- binary -----------------------------------------------------------------------------
// out = op(a, b) with alpha. `out` may be undefined (allocate), or an existing tensor (in-place / out=).
at::Tensor binary_impl(int op, const at::Tensor& a_in, const at::Tensor& b_in, double alpha, at::Tensor out, const char* name, bool integer_ok) {
    const at::Tensor& anchor = is_vulkan(a_in) ? a_in : b_in;
    at::ScalarType st = at::result_type(a_in, b_in);
    if (op == TVK_B_DIV && c10::isIntegralType(st, true)) st = c10::typeMetaToScalarType(at::get_default_dtype());
    const bool is_int = st == at::kLong || st == at::kInt;
    if (!(is_hot_float(st) || (integer_ok && is_int))) TVK_NOT_IMPLEMENTED(name, " for dtype ", st, " on the vulkan device");
    const int dt = to_tvk_dtype(st);
    // scalar * tensor (what `t.mul_(2.0)` turns into: mul.out(wrapped 2.0, t, out=t)) is tensor * scalar
    const bool commutes = op == TVK_B_MUL || op == TVK_B_MAXIMUM || op == TVK_B_MINIMUM || (op == TVK_B_ADD && alpha == 1.0);
    if (commutes && is_cpu_scalar(a_in) && is_vulkan(b_in)) return binary_impl(op, b_in, a_in, alpha, out, name, integer_ok);
    DeviceScope scope(anchor);

    // A CPU scalar second operand uses the scalar-operand kernel (binary.cpp scalar variants).
    if (is_vulkan(a_in) && is_cpu_scalar(b_in)) {
        at::Tensor a = to_dtype(a_in, st);
        if (!out.defined()) out = alloc_like(a, st);
        TORCH_CHECK(out.sizes() == a.sizes(), "torchvulkan [ERROR]: ", name, ": output shape mismatch");
        if (a.numel() == 0) return out;
        at::Tensor target = out.scalar_type() == st ? out : alloc_like(a, st);
        if (same_dense_layout(a, target)) {
            TVK_CALL(tvk_binary(op, dt, target.data_ptr(), a.data_ptr(), nullptr, b_in.item<double>(), alpha, a.numel(), scope.stream));
            if (!target.is_same(out)) out.copy_(target);
            return out;
        }
    }
    at::Tensor a = on_device(a_in, anchor, st), b = on_device(b_in, anchor, st);
    const auto shape = at::infer_size(a.sizes(), b.sizes());
    if (!out.defined()) {
        out = (a.sizes() == shape && same_dense_layout(a, b)) ? alloc_like(a, st) : empty_vulkan(shape, st, anchor.device());
    } else if (out.sizes() != at::IntArrayRef(shape)) {
        TORCH_CHECK(out.numel() == 0 || !out.is_same(a_in), "output with shape ", out.sizes(), " doesn't match the broadcast shape ", at::IntArrayRef(shape));
        out.resize_(shape);
    }
    if (out.numel() == 0) return out;
    at::Tensor target = out.scalar_type() == st ? out : empty_vulkan(shape, st, anchor.device());
    if (same_dense_layout(a, b) && same_dense_layout(a, target)) {
        TVK_CALL(tvk_binary(op, dt, target.data_ptr(), a.data_ptr(), b.data_ptr(), 0.0, alpha, a.numel(), scope.stream));
    } else {
        tvk_iter it;
        make_iter(&it, target, {&a, &b});
        TVK_CALL(tvk_binary_strided(op, dt, target.data_ptr(), a.data_ptr(), b.data_ptr(), alpha, &it, scope.stream));
    }
    if (!target.is_same(out)) out.copy_(target);
    return out;
}

at::Tensor add(const at::Tensor& a, const at::Tensor& b, const at::Scalar& alpha) { return binary_impl(TVK_B_ADD, a, b, alpha.toDouble(), {}, "add", true); }
at::Tensor& add_(at::Tensor& a, const at::Tensor& b, const at::Scalar& alpha) { binary_impl(TVK_B_ADD, a, b, alpha.toDouble(), a, "add_", true); return a; }
at::Tensor& add_out(const at::Tensor& a, const at::Tensor& b, const at::Scalar& alpha, at::Tensor& out) { binary_impl(TVK_B_ADD, a, b, alpha.toDouble(), out, "add.out", true); return out; }
// _add_relu: the reference composes relu(add(...)) (src/api/ops/binary.cpp:655-673); one kernel here
at::Tensor add_relu(const at::Tensor& a, const at::Tensor& b, const at::Scalar& alpha) { return binary_impl(TVK_B_ADD_RELU, a, b, alpha.toDouble(), {}, "_add_relu", false); }
at::Tensor& add_relu_(at::Tensor& a, const at::Tensor& b, const at::Scalar& alpha) { binary_impl(TVK_B_ADD_RELU, a, b, alpha.toDouble(), a, "_add_relu_", false); return a; }
at::Tensor& add_relu_out(const at::Tensor& a, const at::Tensor& b, const at::Scalar& alpha, at::Tensor& out) { binary_impl(TVK_B_ADD_RELU, a, b, alpha.toDouble(), out, "_add_relu.out", false); return out; }
at::Tensor sub(const at::Tensor& a, const at::Tensor& b, const at::Scalar& alpha) { return binary_impl(TVK_B_SUB, a, b, alpha.toDouble(), {}, "sub", true); }
at::Tensor& sub_(at::Tensor& a, const at::Tensor& b, const at::Scalar& alpha) { binary_impl(TVK_B_SUB, a, b, alpha.toDouble(), a, "sub_", true); return a; }
at::Tensor& sub_out(const at::Tensor& a, const at::Tensor& b, const at::Scalar& alpha, at::Tensor& out) { binary_impl(TVK_B_SUB, a, b, alpha.toDouble(), out, "sub.out", true); return out; }

template <int OP, bool INT_OK> at::Tensor bin_fn(const at::Tensor& a, const at::Tensor& b) { return binary_impl(OP, a, b, 1.0, {}, "binary op", INT_OK); }
template <int OP, bool INT_OK> at::Tensor& bin_fn_(at::Tensor& a, const at::Tensor& b) { binary_impl(OP, a, b, 1.0, a, "binary op", INT_OK); return a; }
template <int OP, bool INT_OK> at::Tensor& bin_out(const at::Tensor& a, const at::Tensor& b, at::Tensor& out) { binary_impl(OP, a, b, 1.0, out, "binary op", INT_OK); return out; }

at::Tensor scalar_tensor_like(const at::Scalar& s, const at::Tensor& like) {
    // a wrapped number: participates in type promotion as a Python scalar does
    at::Tensor t = at::scalar_tensor(s, at::TensorOptions().dtype(s.isFloatingPoint() ? at::kDouble : at::kLong).device(at::kCPU));
    t.unsafeGetTensorImpl()->set_wrapped_number(true);
    (void)like;
    return t;
}

at::Tensor pow_tensor_scalar(const at::Tensor& self, const at::Scalar& exponent) {
    if (exponent.toDouble() == 2.0) return unary_fn<TVK_U_SQUARE>(self);
    return binary_impl(TVK_B_POW, self, scalar_tensor_like(exponent, self), 1.0, {}, "pow");
}
at::Tensor& pow_tensor_scalar_out(const at::Tensor& self, const at::Scalar& exponent, at::Tensor& out) {
    if (exponent.toDouble() == 2.0) return unary_out<TVK_U_SQUARE>(self, out);
    binary_impl(TVK_B_POW, self, scalar_tensor_like(exponent, self), 1.0, out, "pow.out");
    return out;
}

// grad-style binaries: (grad, saved) -> grad_input, all in grad's dtype
at::Tensor gelu_backward(const at::Tensor& grad, const at::Tensor& self, c10::string_view approximate) {
    return binary_impl(gelu_is_tanh(approximate) ? TVK_B_GELU_TANH_BACKWARD : TVK_B_GELU_BACKWARD, grad, self, 1.0, {}, "gelu_backward");
}
at::Tensor& gelu_backward_out(const at::Tensor& grad, const at::Tensor& self, c10::string_view approximate, at::Tensor& out) {
    binary_impl(gelu_is_tanh(approximate) ? TVK_B_GELU_TANH_BACKWARD : TVK_B_GELU_BACKWARD, grad, self, 1.0, out, "gelu_backward");
    return out;
}
at::Tensor threshold_backward(const at::Tensor& grad, const at::Tensor& self, const at::Scalar& threshold) {
    return binary_impl(TVK_B_THRESHOLD_BACKWARD, grad, self, threshold.toDouble(), {}, "threshold_backward");
}
at::Tensor& threshold_backward_out(const at::Tensor& grad, const at::Tensor& self, const at::Scalar& threshold, at::Tensor& out) {
    binary_impl(TVK_B_THRESHOLD_BACKWARD, grad, self, threshold.toDouble(), out, "threshold_backward");
    return out;
}

// ---- comparisons ------------------------------------------------------------------------
at::Tensor compare_impl(int op, const at::Tensor& a_in, const at::Tensor& b_in, at::Tensor out, const char* name) {
    const at::Tensor& anchor = is_vulkan(a_in) ? a_in : b_in;
    const at::ScalarType st = at::result_type(a_in, b_in);
    const bool is_int = st == at::kLong || st == at::kInt || st == at::kBool || st == at::kByte;     // compared exactly, as 64-bit integers
    if (!is_hot_float(st) && !is_int) TVK_NOT_IMPLEMENTED(name, " for dtype ", st, " on the vulkan device");
    const int dt = to_tvk_dtype(st);
    DeviceScope scope(anchor);
    if (is_vulkan(a_in) && is_cpu_scalar(b_in) && a_in.is_contiguous()) {
        at::Tensor a = to_dtype(a_in, st);
        if (!out.defined()) out = empty_vulkan(a.sizes(), at::kBool, a.device());
        if (out.sizes() != a.sizes()) out.resize_(a.sizes());
        if (a.numel() && out.is_contiguous() && out.scalar_type() == at::kBool) {
            TVK_CALL(tvk_compare(op, dt, (uint8_t*)out.data_ptr(), a.data_ptr(), nullptr, b_in.item<double>(), a.numel(), scope.stream));
            return out;
        }
        if (!a.numel()) return out;
    }
    at::Tensor a = on_device(a_in, anchor, st), b = on_device(b_in, anchor, st);
    const auto shape = at::infer_size(a.sizes(), b.sizes());
    if (!out.defined()) out = empty_vulkan(shape, at::kBool, anchor.device());
    if (out.sizes() != at::IntArrayRef(shape)) out.resize_(shape);
    if (out.numel() == 0) return out;
    at::Tensor target = out.scalar_type() == at::kBool ? out : empty_vulkan(shape, at::kBool, anchor.device());
    tvk_iter it;
    make_iter(&it, target, {&a, &b});
    TVK_CALL(tvk_compare_strided(op, dt, (uint8_t*)target.data_ptr(), a.data_ptr(), b.data_ptr(), &it, scope.stream));
    if (!target.is_same(out)) out.copy_(target);
    return out;
}
template <int OP> at::Tensor cmp_tensor(const at::Tensor& a, const at::Tensor& b) { return compare_impl(OP, a, b, {}, "comparison"); }
template <int OP> at::Tensor& cmp_tensor_out(const at::Tensor& a, const at::Tensor& b, at::Tensor& out) { compare_impl(OP, a, b, out, "comparison"); return out; }
template <int OP> at::Tensor cmp_scalar(const at::Tensor& a, const at::Scalar& b) { return compare_impl(OP, a, scalar_tensor_like(b, a), {}, "comparison"); }
template <int OP> at::Tensor& cmp_scalar_out(const at::Tensor& a, const at::Scalar& b, at::Tensor& out) { compare_impl(OP, a, scalar_tensor_like(b, a), out, "comparison"); return out; }

// ---- one tensor and two scalar parameters (clamp, hardtanh, leaky_relu, elu, softplus) ----------------------------
// The kernels are the binary family's scalar-operand form (b == NULL): b_scalar and alpha carry the parameters.
at::Tensor scalar_binary(int op, const at::Tensor& self, double bs, double alpha, at::Tensor out, const char* name) {
    require_float(self, name);
    at::Tensor a = self.is_non_overlapping_and_dense() ? self : contiguous_vulkan(self);
    const bool direct = out.defined() && out.scalar_type() == a.scalar_type() && same_dense_layout(a, out);
    at::Tensor target = direct ? out : alloc_like(a, a.scalar_type());
    if (a.numel()) {
        DeviceScope scope(a);
        TVK_CALL(tvk_binary(op, to_tvk_dtype(a.scalar_type()), target.data_ptr(), a.data_ptr(), nullptr, bs, alpha, a.numel(), scope.stream));
    }
    if (out.defined() && !direct) {
        if (out.sizes() != a.sizes()) out.resize_(a.sizes());
        out.copy_(target);
        return out;
    }
    return target;
}
at::Tensor clamp_impl(const at::Tensor& self, const c10::optional<at::Scalar>& lo, const c10::optional<at::Scalar>& hi, at::Tensor out) {
    TORCH_CHECK(lo.has_value() || hi.has_value(), "torch.clamp: At least one of 'min' or 'max' must not be None");
    if (self.scalar_type() == at::kLong || self.scalar_type() == at::kInt) {        // exact: maximum then minimum with integer bounds
        TORCH_CHECK((!lo.has_value() || lo->isIntegral(false)) && (!hi.has_value() || hi->isIntegral(false)), "torchvulkan [NOT IMPLEMENTED]: clamp of an integer tensor to floating bounds");
        at::Tensor r = self;
        if (lo.has_value()) r = binary_impl(TVK_B_MAXIMUM, r, scalar_tensor_like(*lo, self), 1.0, {}, "clamp", true);
        if (hi.has_value()) r = binary_impl(TVK_B_MINIMUM, r, scalar_tensor_like(*hi, self), 1.0, {}, "clamp", true);
        if (out.defined()) { if (out.sizes() != r.sizes()) out.resize_(r.sizes()); out.copy_(r); return out; }
        return r;
    }
    return scalar_binary(TVK_B_CLAMP, self, hi.has_value() ? hi->toDouble() : std::numeric_limits<double>::infinity(),
                         lo.has_value() ? lo->toDouble() : -std::numeric_limits<double>::infinity(), out, "clamp");
}
at::Tensor clamp(const at::Tensor& self, const c10::optional<at::Scalar>& lo, const c10::optional<at::Scalar>& hi) { return clamp_impl(self, lo, hi, {}); }
at::Tensor& clamp_(at::Tensor& self, const c10::optional<at::Scalar>& lo, const c10::optional<at::Scalar>& hi) { clamp_impl(self, lo, hi, self); return self; }
at::Tensor& clamp_out(const at::Tensor& self, const c10::optional<at::Scalar>& lo, const c10::optional<at::Scalar>& hi, at::Tensor& out) { clamp_impl(self, lo, hi, out); return out; }
at::Tensor clamp_min(const at::Tensor& self, const at::Scalar& lo) { return clamp_impl(self, lo, c10::nullopt, {}); }
at::Tensor& clamp_min_(at::Tensor& self, const at::Scalar& lo) { clamp_impl(self, lo, c10::nullopt, self); return self; }
at::Tensor& clamp_min_out(const at::Tensor& self, const at::Scalar& lo, at::Tensor& out) { clamp_impl(self, lo, c10::nullopt, out); return out; }
at::Tensor clamp_max(const at::Tensor& self, const at::Scalar& hi) { return clamp_impl(self, c10::nullopt, hi, {}); }
at::Tensor& clamp_max_(at::Tensor& self, const at::Scalar& hi) { clamp_impl(self, c10::nullopt, hi, self); return self; }
at::Tensor& clamp_max_out(const at::Tensor& self, const at::Scalar& hi, at::Tensor& out) { clamp_impl(self, c10::nullopt, hi, out); return out; }
at::Tensor hardtanh(const at::Tensor& self, const at::Scalar& lo, const at::Scalar& hi) { return clamp_impl(self, lo, hi, {}); }
at::Tensor& hardtanh_(at::Tensor& self, const at::Scalar& lo, const at::Scalar& hi) { clamp_impl(self, lo, hi, self); return self; }
at::Tensor& hardtanh_out(const at::Tensor& self, const at::Scalar& lo, const at::Scalar& hi, at::Tensor& out) { clamp_impl(self, lo, hi, out); return out; }
// grad where lo < x < hi, else 0 (hardtanh_backward of ATen)
at::Tensor hardtanh_backward(const at::Tensor& grad, const at::Tensor& self, const at::Scalar& lo, const at::Scalar& hi) {
    return at::where(at::logical_and(at::gt(self, lo), at::lt(self, hi)), grad, at::zeros({}, grad.options()));
}
at::Tensor leaky_relu(const at::Tensor& self, const at::Scalar& slope) { return scalar_binary(TVK_B_LEAKY_RELU, self, slope.toDouble(), 1.0, {}, "leaky_relu"); }
at::Tensor& leaky_relu_(at::Tensor& self, const at::Scalar& slope) { scalar_binary(TVK_B_LEAKY_RELU, self, slope.toDouble(), 1.0, self, "leaky_relu_"); return self; }
at::Tensor& leaky_relu_out(const at::Tensor& self, const at::Scalar& slope, at::Tensor& out) { scalar_binary(TVK_B_LEAKY_RELU, self, slope.toDouble(), 1.0, out, "leaky_relu.out"); return out; }
at::Tensor leaky_relu_backward(const at::Tensor& grad, const at::Tensor& self, const at::Scalar& slope, bool self_is_result) {
    // with a positive slope the sign of the result is the sign of the input, so the same test serves both
    TORCH_CHECK(!self_is_result || slope.toDouble() > 0.0, "In-place leakyReLu backward calculation is triggered with a negative slope which is not supported.");
    return binary_impl(TVK_B_LEAKY_RELU_BACKWARD, grad, self, slope.toDouble(), {}, "leaky_relu_backward");
}
// elu(x) = scale * (x > 0 ? x : alpha * (exp(input_scale * x) - 1)). The kernel covers scale = input_scale = 1 (elu); selu and
// celu, which set the other two, are composed from where / expm1.
bool plain_elu(const at::Scalar& scale, const at::Scalar& input_scale) { return scale.toDouble() == 1.0 && input_scale.toDouble() == 1.0; }
at::Tensor elu_general(const at::Tensor& self, const at::Scalar& alpha, const at::Scalar& scale, const at::Scalar& input_scale) {
    return at::where(at::gt(self, 0), self * scale, at::expm1(self * input_scale) * (alpha.toDouble() * scale.toDouble()));
}
at::Tensor elu(const at::Tensor& self, const at::Scalar& alpha, const at::Scalar& scale, const at::Scalar& input_scale) {
    if (!plain_elu(scale, input_scale)) return elu_general(self, alpha, scale, input_scale);
    return scalar_binary(TVK_B_ELU, self, 0.0, alpha.toDouble(), {}, "elu");
}
at::Tensor& elu_(at::Tensor& self, const at::Scalar& alpha, const at::Scalar& scale, const at::Scalar& input_scale) {
    if (!plain_elu(scale, input_scale)) { self.copy_(elu_general(self, alpha, scale, input_scale)); return self; }
    scalar_binary(TVK_B_ELU, self, 0.0, alpha.toDouble(), self, "elu_");
    return self;
}
at::Tensor& elu_out(const at::Tensor& self, const at::Scalar& alpha, const at::Scalar& scale, const at::Scalar& input_scale, at::Tensor& out) {
    if (!plain_elu(scale, input_scale)) {
        at::Tensor r = elu_general(self, alpha, scale, input_scale);
        if (out.sizes() != r.sizes()) out.resize_(r.sizes());
        out.copy_(r);
        return out;
    }
    scalar_binary(TVK_B_ELU, self, 0.0, alpha.toDouble(), out, "elu.out");
    return out;
}
at::Tensor elu_backward(const at::Tensor& grad, const at::Scalar& alpha, const at::Scalar& scale, const at::Scalar& input_scale, bool is_result,
                        const at::Tensor& self_or_result) {
    const double a = alpha.toDouble(), sc = scale.toDouble(), is = input_scale.toDouble();
    // from the result y = scale * alpha * (exp(is * x) - 1) for x <= 0: dy/dx = is * (y + scale * alpha)
    if (is_result) return at::where(at::gt(self_or_result, 0), grad * sc, grad * (self_or_result + a * sc) * is);
    if (!plain_elu(scale, input_scale)) return at::where(at::gt(self_or_result, 0), grad * sc, grad * at::exp(self_or_result * is) * (a * sc * is));
    return binary_impl(TVK_B_ELU_BACKWARD, grad, self_or_result, a, {}, "elu_backward");
}
at::Tensor softplus(const at::Tensor& self, const at::Scalar& beta, const at::Scalar& threshold) {
    return scalar_binary(TVK_B_SOFTPLUS, self, threshold.toDouble(), beta.toDouble(), {}, "softplus");
}
at::Tensor& softplus_out(const at::Tensor& self, const at::Scalar& beta, const at::Scalar& threshold, at::Tensor& out) {
    scalar_binary(TVK_B_SOFTPLUS, self, threshold.toDouble(), beta.toDouble(), out, "softplus.out");
    return out;
}
at::Tensor softplus_backward(const at::Tensor& grad, const at::Tensor& self, const at::Scalar& beta, const at::Scalar& threshold) {
    if (threshold.toDouble() != 20.0) TVK_NOT_IMPLEMENTED("softplus backward with a threshold other than 20");
    return binary_impl(TVK_B_SOFTPLUS_BACKWARD, grad, self, beta.toDouble(), {}, "softplus_backward");
}
template <int OP> at::Tensor grad_x_fn(const at::Tensor& grad, const at::Tensor& self) { return binary_impl(OP, grad, self, 1.0, {}, "activation backward"); }
std::tuple<at::Tensor, at::Tensor> log_sigmoid_forward(const at::Tensor& self) {
    return {unary_fn<TVK_U_LOGSIGMOID>(self), at::empty({0}, self.options())};      // (the buffer is a CPU-kernel detail; unused here)
}
at::Tensor log_sigmoid_backward(const at::Tensor& grad, const at::Tensor& self, const at::Tensor&) {
    return binary_impl(TVK_B_LOGSIGMOID_BACKWARD, grad, self, 1.0, {}, "log_sigmoid_backward");
}

// clamp to tensor bounds: maximum then minimum (NaN in self or a bound propagates, as in ATen)
at::Tensor clamp_tensor(const at::Tensor& self, const c10::optional<at::Tensor>& lo, const c10::optional<at::Tensor>& hi) {
    TORCH_CHECK((lo.has_value() && lo->defined()) || (hi.has_value() && hi->defined()), "torch.clamp: At least one of 'min' or 'max' must not be None");
    at::Tensor r = self;
    if (lo.has_value() && lo->defined()) r = binary_impl(TVK_B_MAXIMUM, r, *lo, 1.0, {}, "clamp", true);
    if (hi.has_value() && hi->defined()) r = binary_impl(TVK_B_MINIMUM, r, *hi, 1.0, {}, "clamp", true);
    return r;
}
at::Tensor& clamp_tensor_out(const at::Tensor& self, const c10::optional<at::Tensor>& lo, const c10::optional<at::Tensor>& hi, at::Tensor& out) {
    at::Tensor r = clamp_tensor(self, lo, hi);
    if (out.sizes() != r.sizes()) out.resize_(r.sizes());
    out.copy_(r);
    return out;
}
at::Tensor clamp_min_tensor(const at::Tensor& self, const at::Tensor& lo) { return binary_impl(TVK_B_MAXIMUM, self, lo, 1.0, {}, "clamp_min", true); }
at::Tensor& clamp_min_tensor_out(const at::Tensor& self, const at::Tensor& lo, at::Tensor& out) { binary_impl(TVK_B_MAXIMUM, self, lo, 1.0, out, "clamp_min", true); return out; }
at::Tensor clamp_max_tensor(const at::Tensor& self, const at::Tensor& hi) { return binary_impl(TVK_B_MINIMUM, self, hi, 1.0, {}, "clamp_max", true); }
at::Tensor& clamp_max_tensor_out(const at::Tensor& self, const at::Tensor& hi, at::Tensor& out) { binary_impl(TVK_B_MINIMUM, self, hi, 1.0, out, "clamp_max", true); return out; }
// threshold(x, t, v) = x > t ? x : v;  hardshrink(x, l) = |x| > l ? x : 0
at::Tensor vk_threshold(const at::Tensor& self, const at::Scalar& t, const at::Scalar& value) {
    return at::where(at::gt(self, t), self, at::full({}, value, self.options()));
}
at::Tensor& threshold_(at::Tensor& self, const at::Scalar& t, const at::Scalar& value) { self.copy_(vk_threshold(self, t, value)); return self; }
at::Tensor& threshold_out(const at::Tensor& self, const at::Scalar& t, const at::Scalar& value, at::Tensor& out) {
    at::Tensor r = vk_threshold(self, t, value);
    if (out.sizes() != r.sizes()) out.resize_(r.sizes());
    out.copy_(r);
    return out;
}
at::Tensor hardshrink(const at::Tensor& self, const at::Scalar& lambd) { return at::where(at::gt(at::abs(self), lambd), self, at::zeros({}, self.options())); }
at::Tensor hardshrink_backward(const at::Tensor& grad, const at::Tensor& self, const at::Scalar& lambd) {
    return at::where(at::gt(at::abs(self), lambd), grad, at::zeros({}, grad.options()));
}

// ---- logical ops on boolean tensors ------------------------------------------------------
// any dtype in (x != 0 is true), Bool out; the operands are broadcast and made contiguous first (masks are small next to
// the tensors they select from)
at::Tensor as_bool(const at::Tensor& t) {
    if (t.scalar_type() == at::kBool) return t;
    return at::ne(t, 0);
}
at::Tensor logical_impl(int op, const at::Tensor& a_in, const at::Tensor* b_in, at::Tensor out) {
    const at::Tensor& anchor = (b_in && !is_vulkan(a_in)) ? *b_in : a_in;
    auto bring = [&](const at::Tensor& t) { return is_vulkan(t) ? as_bool(t) : t.to(at::kBool).to(anchor.device()); };
    at::Tensor a = bring(a_in), b;
    std::vector<int64_t> shape(a.sizes().begin(), a.sizes().end());
    if (b_in) {
        b = bring(*b_in);
        shape = at::infer_size(a.sizes(), b.sizes());
        b = contiguous_vulkan(b.expand(shape));
    }
    a = contiguous_vulkan(a.expand(shape));
    at::Tensor target = (out.defined() && out.scalar_type() == at::kBool && out.is_contiguous() && out.sizes() == at::IntArrayRef(shape)) ? out
                                                                                                                                       : empty_vulkan(shape, at::kBool, anchor.device());
    if (target.numel()) {
        DeviceScope scope(anchor);
        TVK_CALL(tvk_logical(op, (uint8_t*)target.data_ptr(), (const uint8_t*)a.data_ptr(), b_in ? (const uint8_t*)b.data_ptr() : nullptr, target.numel(), scope.stream));
    }
    if (out.defined() && !target.is_same(out)) {
        if (out.sizes() != at::IntArrayRef(shape)) out.resize_(shape);
        out.copy_(target);
        return out;
    }
    return target;
}
template <int OP> at::Tensor logical_fn(const at::Tensor& a, const at::Tensor& b) { return logical_impl(OP, a, &b, {}); }
template <int OP> at::Tensor& logical_out(const at::Tensor& a, const at::Tensor& b, at::Tensor& out) { logical_impl(OP, a, &b, out); return out; }
template <int OP> at::Tensor& logical_fn_(at::Tensor& a, const at::Tensor& b) { logical_impl(OP, a, &b, a); return a; }
at::Tensor logical_not(const at::Tensor& a) { return logical_impl(TVK_L_NOT, a, nullptr, {}); }
at::Tensor& logical_not_out(const at::Tensor& a, at::Tensor& out) { logical_impl(TVK_L_NOT, a, nullptr, out); return out; }
// bitwise ops: on Bool tensors they are the logical ops (masks); integer tensors are not handled
void require_bool(const at::Tensor& a, const char* name) {
    if (a.scalar_type() != at::kBool) TVK_NOT_IMPLEMENTED(name, " for dtype ", a.scalar_type(), " (Bool masks are supported)");
}
template <int OP> at::Tensor bitwise_fn(const at::Tensor& a, const at::Tensor& b) { require_bool(a, "bitwise op"); require_bool(b, "bitwise op"); return logical_impl(OP, a, &b, {}); }
template <int OP> at::Tensor& bitwise_out(const at::Tensor& a, const at::Tensor& b, at::Tensor& out) { require_bool(a, "bitwise op"); require_bool(b, "bitwise op"); logical_impl(OP, a, &b, out); return out; }
at::Tensor bitwise_not(const at::Tensor& a) { require_bool(a, "bitwise_not"); return logical_impl(TVK_L_NOT, a, nullptr, {}); }
at::Tensor& bitwise_not_out(const at::Tensor& a, at::Tensor& out) { require_bool(a, "bitwise_not"); logical_impl(TVK_L_NOT, a, nullptr, out); return out; }

// the product of two masks is their conjunction
at::Tensor mul_tensor(const at::Tensor& a, const at::Tensor& b) {
    if (a.scalar_type() == at::kBool && b.scalar_type() == at::kBool) return logical_impl(TVK_L_AND, a, &b, {});
    return binary_impl(TVK_B_MUL, a, b, 1.0, {}, "binary op", true);
}

// isnan / isposinf / isneginf as comparisons
at::Tensor isnan(const at::Tensor& self) { return compare_impl(TVK_C_NE, self, self, {}, "isnan"); }
at::Tensor& isposinf_out(const at::Tensor& self, at::Tensor& out) { compare_impl(TVK_C_EQ, self, scalar_tensor_like(std::numeric_limits<double>::infinity(), self), out, "isposinf"); return out; }
at::Tensor& isneginf_out(const at::Tensor& self, at::Tensor& out) { compare_impl(TVK_C_EQ, self, scalar_tensor_like(-std::numeric_limits<double>::infinity(), self), out, "isneginf"); return out; }

// ---- ternary ----------------------------------------------------------------------------
at::Tensor ternary_impl(int op, const at::Tensor& a_in, const at::Tensor& b_in, const at::Tensor* c_in, double value, at::Tensor out, const char* name) {
    at::ScalarType st = at::result_type(a_in, b_in);
    if (c_in) st = c10::promoteTypes(st, c_in->scalar_type());
    if (!is_hot_float(st)) TVK_NOT_IMPLEMENTED(name, " for dtype ", st, " on the vulkan device");
    const int dt = to_tvk_dtype(st);
    DeviceScope scope(a_in);
    at::Tensor a = on_device(a_in, a_in, st), b = on_device(b_in, a_in, st), c;
    if (c_in) c = on_device(*c_in, a_in, st);
    auto shape = at::infer_size(a.sizes(), b.sizes());
    if (c_in) shape = at::infer_size(shape, c.sizes());
    if (!out.defined()) out = (a.sizes() == at::IntArrayRef(shape)) ? alloc_like(a, st) : empty_vulkan(shape, st, a.device());
    TORCH_CHECK(out.sizes() == at::IntArrayRef(shape), "torchvulkan [ERROR]: ", name, ": output shape mismatch");
    if (out.numel() == 0) return out;
    at::Tensor target = out.scalar_type() == st ? out : empty_vulkan(shape, st, a.device());
    const bool flat = same_dense_layout(a, b) && same_dense_layout(a, target) && (!c_in || same_dense_layout(a, c));
    if (flat) {
        TVK_CALL(tvk_ternary(op, dt, target.data_ptr(), a.data_ptr(), b.data_ptr(), c_in ? c.data_ptr() : nullptr, value, a.numel(), scope.stream));
    } else if (c_in) {
        tvk_iter it;
        make_iter(&it, target, {&a, &b, &c});
        TVK_CALL(tvk_ternary_strided(op, dt, target.data_ptr(), a.data_ptr(), b.data_ptr(), c.data_ptr(), value, &it, scope.stream));
    } else {
        tvk_iter it;
        make_iter(&it, target, {&a, &b});
        TVK_CALL(tvk_ternary_strided(op, dt, target.data_ptr(), a.data_ptr(), b.data_ptr(), nullptr, value, &it, scope.stream));
    }
    if (!target.is_same(out)) out.copy_(target);
    return out;
}
at::Tensor addcmul(const at::Tensor& s, const at::Tensor& t1, const at::Tensor& t2, const at::Scalar& v) { return ternary_impl(TVK_T_ADDCMUL, s, t1, &t2, v.toDouble(), {}, "addcmul"); }
at::Tensor& addcmul_(at::Tensor& s, const at::Tensor& t1, const at::Tensor& t2, const at::Scalar& v) { ternary_impl(TVK_T_ADDCMUL, s, t1, &t2, v.toDouble(), s, "addcmul_"); return s; }
at::Tensor& addcmul_out(const at::Tensor& s, const at::Tensor& t1, const at::Tensor& t2, const at::Scalar& v, at::Tensor& out) { ternary_impl(TVK_T_ADDCMUL, s, t1, &t2, v.toDouble(), out, "addcmul.out"); return out; }
at::Tensor addcdiv(const at::Tensor& s, const at::Tensor& t1, const at::Tensor& t2, const at::Scalar& v) { return ternary_impl(TVK_T_ADDCDIV, s, t1, &t2, v.toDouble(), {}, "addcdiv"); }
at::Tensor& addcdiv_(at::Tensor& s, const at::Tensor& t1, const at::Tensor& t2, const at::Scalar& v) { ternary_impl(TVK_T_ADDCDIV, s, t1, &t2, v.toDouble(), s, "addcdiv_"); return s; }
at::Tensor& addcdiv_out(const at::Tensor& s, const at::Tensor& t1, const at::Tensor& t2, const at::Scalar& v, at::Tensor& out) { ternary_impl(TVK_T_ADDCDIV, s, t1, &t2, v.toDouble(), out, "addcdiv.out"); return out; }
at::Tensor lerp_scalar(const at::Tensor& s, const at::Tensor& e, const at::Scalar& w) { return ternary_impl(TVK_T_LERP, s, e, nullptr, w.toDouble(), {}, "lerp"); }
at::Tensor& lerp_scalar_(at::Tensor& s, const at::Tensor& e, const at::Scalar& w) { ternary_impl(TVK_T_LERP, s, e, nullptr, w.toDouble(), s, "lerp_"); return s; }
at::Tensor& lerp_scalar_out(const at::Tensor& s, const at::Tensor& e, const at::Scalar& w, at::Tensor& out) { ternary_impl(TVK_T_LERP, s, e, nullptr, w.toDouble(), out, "lerp.out"); return out; }
// lerp with a tensor weight: start + weight * (end - start)
at::Tensor lerp_tensor(const at::Tensor& s0, const at::Tensor& e, const at::Tensor& w) {
    at::Tensor d = at::sub(e, s0);
    return ternary_impl(TVK_T_ADDCMUL, s0, w, &d, 1.0, {}, "lerp");
}
at::Tensor& lerp_tensor_(at::Tensor& s0, const at::Tensor& e, const at::Tensor& w) { s0.copy_(lerp_tensor(s0, e, w)); return s0; }
at::Tensor& lerp_tensor_out(const at::Tensor& s0, const at::Tensor& e, const at::Tensor& w, at::Tensor& out) {
    at::Tensor r = lerp_tensor(s0, e, w);
    if (out.sizes() != r.sizes()) out.resize_(r.sizes());
    out.copy_(r);
    return out;
}

at::Tensor where_self(const at::Tensor& cond, const at::Tensor& a_in, const at::Tensor& b_in) {
    TORCH_CHECK(cond.scalar_type() == at::kBool, "where expected condition to be a boolean tensor, but got a tensor with dtype ", cond.scalar_type());
    const at::ScalarType st = at::result_type(a_in, b_in);
    const int dt = to_tvk_dtype(st);
    TORCH_CHECK(dt >= 0, "torchvulkan [NOT IMPLEMENTED]: where for dtype ", st);
    DeviceScope scope(cond);
    at::Tensor a = on_device(a_in, cond, st), b = on_device(b_in, cond, st);
    auto shape = at::infer_size(at::infer_size(a.sizes(), b.sizes()), cond.sizes());
    at::Tensor out = empty_vulkan(shape, st, cond.device());
    if (out.numel() == 0) return out;
    tvk_iter it;
    make_iter(&it, out, {&a, &b, &cond});
    TVK_CALL(tvk_ternary_strided(TVK_T_WHERE, dt, out.data_ptr(), a.data_ptr(), b.data_ptr(), cond.data_ptr(), 0.0, &it, scope.stream));
    return out;
}

// ---- fill -------------------------------------------------------------------------------
at::Tensor& fill_scalar_(at::Tensor& self, const at::Scalar& value) {
    if (self.numel() == 0) return self;
    const int dt = to_tvk_dtype(self.scalar_type());
    TORCH_CHECK(dt >= 0, "torchvulkan [NOT IMPLEMENTED]: fill_ for dtype ", self.scalar_type());
    const double v = self.scalar_type() == at::kBool ? (value.toBool() ? 1.0 : 0.0) : value.toDouble();
    if (self.is_non_overlapping_and_dense()) {
        DeviceScope scope(self);
        TVK_CALL(tvk_fill(dt, self.data_ptr(), v, self.numel(), scope.stream));
    } else {
        at::Tensor tmp = empty_vulkan(self.sizes(), self.scalar_type(), self.device());
        {
            DeviceScope scope(self);
            TVK_CALL(tvk_fill(dt, tmp.data_ptr(), v, tmp.numel(), scope.stream));
        }
        self.copy_(tmp);
    }
    return self;
}
at::Tensor& fill_tensor_(at::Tensor& self, const at::Tensor& value) {
    TORCH_CHECK(value.dim() == 0, "fill_ only supports 0-dimension value tensor but got tensor with ", value.dim(), " dimensions.");
    return fill_scalar_(self, value.item());
}
at::Tensor& zero_(at::Tensor& self) { return fill_scalar_(self, 0); }

}  // namespace

#define REG_UNARY(m, name, OP)                              \
    m.impl(name, &unary_fn<OP>);                            \
    m.impl(name "_", &unary_fn_<OP>);                       \
    m.impl(name ".out", &unary_out<OP>)

#define REG_BINARY(m, name, OP, INT_OK)                     \
    m.impl(name, &bin_fn<OP, INT_OK>);                      \
    m.impl(name "_", &bin_fn_<OP, INT_OK>);                 \
    m.impl(name ".out", &bin_out<OP, INT_OK>)

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    REG_UNARY(m, "neg", TVK_U_NEG);
    REG_UNARY(m, "exp", TVK_U_EXP);
    REG_UNARY(m, "log", TVK_U_LOG);
    REG_UNARY(m, "sqrt", TVK_U_SQRT);
    REG_UNARY(m, "rsqrt", TVK_U_RSQRT);
    REG_UNARY(m, "sigmoid", TVK_U_SIGMOID);
    REG_UNARY(m, "relu", TVK_U_RELU);
    REG_UNARY(m, "tanh", TVK_U_TANH);
    REG_UNARY(m, "abs", TVK_U_ABS);
    REG_UNARY(m, "silu", TVK_U_SILU);
    REG_UNARY(m, "reciprocal", TVK_U_RECIPROCAL);
    REG_UNARY(m, "sin", TVK_U_SIN);
    REG_UNARY(m, "cos", TVK_U_COS);
    m.impl("gelu", &gelu);
    m.impl("gelu_", &gelu_);
    m.impl("gelu.out", &gelu_out);

    m.impl("add.Tensor", &add);
    m.impl("add_.Tensor", &add_);
    m.impl("add.out", &add_out);
    m.impl("_add_relu.Tensor", &add_relu);
    m.impl("_add_relu_.Tensor", &add_relu_);
    m.impl("_add_relu.out", &add_relu_out);
    m.impl("sub.Tensor", &sub);
    m.impl("sub_.Tensor", &sub_);
    m.impl("sub.out", &sub_out);
    m.impl("mul.Tensor", &mul_tensor);
    m.impl("mul_.Tensor", &bin_fn_<TVK_B_MUL, true>);
    m.impl("mul.out", &bin_out<TVK_B_MUL, true>);
    m.impl("div.Tensor", &bin_fn<TVK_B_DIV, false>);
    m.impl("div_.Tensor", &bin_fn_<TVK_B_DIV, false>);
    m.impl("div.out", &bin_out<TVK_B_DIV, false>);
    m.impl("maximum", &bin_fn<TVK_B_MAXIMUM, true>);
    m.impl("maximum.out", &bin_out<TVK_B_MAXIMUM, true>);
    m.impl("minimum", &bin_fn<TVK_B_MINIMUM, true>);
    m.impl("minimum.out", &bin_out<TVK_B_MINIMUM, true>);
    m.impl("pow.Tensor_Tensor", &bin_fn<TVK_B_POW, false>);
    m.impl("pow_.Tensor", &bin_fn_<TVK_B_POW, false>);
    m.impl("pow.Tensor_Tensor_out", &bin_out<TVK_B_POW, false>);
    m.impl("pow.Tensor_Scalar", &pow_tensor_scalar);
    m.impl("pow.Tensor_Scalar_out", &pow_tensor_scalar_out);

    m.impl("gelu_backward", &gelu_backward);
    m.impl("gelu_backward.grad_input", &gelu_backward_out);
    m.impl("threshold_backward", &threshold_backward);
    m.impl("threshold_backward.grad_input", &threshold_backward_out);
    m.impl("silu_backward", &bin_fn<TVK_B_SILU_BACKWARD, false>);
    m.impl("silu_backward.grad_input", &bin_out<TVK_B_SILU_BACKWARD, false>);
    m.impl("sigmoid_backward", &bin_fn<TVK_B_SIGMOID_BACKWARD, false>);
    m.impl("sigmoid_backward.grad_input", &bin_out<TVK_B_SIGMOID_BACKWARD, false>);
    m.impl("tanh_backward", &bin_fn<TVK_B_TANH_BACKWARD, false>);
    m.impl("tanh_backward.grad_input", &bin_out<TVK_B_TANH_BACKWARD, false>);

    REG_UNARY(m, "floor", TVK_U_FLOOR);
    REG_UNARY(m, "ceil", TVK_U_CEIL);
    REG_UNARY(m, "round", TVK_U_ROUND);
    REG_UNARY(m, "trunc", TVK_U_TRUNC);
    REG_UNARY(m, "sign", TVK_U_SIGN);
    REG_UNARY(m, "sgn", TVK_U_SIGN);           // real tensors: sgn is sign (the gradient of abs)
    REG_UNARY(m, "log2", TVK_U_LOG2);
    REG_UNARY(m, "log10", TVK_U_LOG10);
    REG_UNARY(m, "log1p", TVK_U_LOG1P);
    REG_UNARY(m, "expm1", TVK_U_EXPM1);
    REG_UNARY(m, "exp2", TVK_U_EXP2);
    REG_UNARY(m, "tan", TVK_U_TAN);
    REG_UNARY(m, "sinh", TVK_U_SINH);
    REG_UNARY(m, "cosh", TVK_U_COSH);
    REG_UNARY(m, "asin", TVK_U_ASIN);
    REG_UNARY(m, "acos", TVK_U_ACOS);
    REG_UNARY(m, "atan", TVK_U_ATAN);
    REG_UNARY(m, "erf", TVK_U_ERF);
    REG_UNARY(m, "erfc", TVK_U_ERFC);
    REG_UNARY(m, "hardsigmoid", TVK_U_HARDSIGMOID);
    REG_UNARY(m, "hardswish", TVK_U_HARDSWISH);
    REG_UNARY(m, "mish", TVK_U_MISH);
    REG_UNARY(m, "asinh", TVK_U_ASINH);
    REG_UNARY(m, "acosh", TVK_U_ACOSH);
    REG_UNARY(m, "atanh", TVK_U_ATANH);
    REG_UNARY(m, "erfinv", TVK_U_ERFINV);
    REG_UNARY(m, "lgamma", TVK_U_LGAMMA);
    REG_UNARY(m, "frac", TVK_U_FRAC);
    REG_UNARY(m, "sinc", TVK_U_SINC);
    REG_BINARY(m, "hypot", TVK_B_HYPOT, false);
    REG_BINARY(m, "logaddexp", TVK_B_LOGADDEXP, false);
    REG_BINARY(m, "logaddexp2", TVK_B_LOGADDEXP2, false);
    REG_BINARY(m, "fmax", TVK_B_FMAX, false);
    REG_BINARY(m, "fmin", TVK_B_FMIN, false);
    REG_BINARY(m, "heaviside", TVK_B_HEAVISIDE, false);
    m.impl("copysign.Tensor", &bin_fn<TVK_B_COPYSIGN, false>);
    m.impl("copysign_.Tensor", &bin_fn_<TVK_B_COPYSIGN, false>);
    m.impl("copysign.out", &bin_out<TVK_B_COPYSIGN, false>);
    m.impl("fmod.Tensor", &bin_fn<TVK_B_FMOD, true>);
    m.impl("fmod_.Tensor", &bin_fn_<TVK_B_FMOD, true>);
    m.impl("fmod.Tensor_out", &bin_out<TVK_B_FMOD, true>);
    m.impl("remainder.Tensor", &bin_fn<TVK_B_REMAINDER, true>);
    m.impl("remainder_.Tensor", &bin_fn_<TVK_B_REMAINDER, true>);
    m.impl("remainder.Tensor_out", &bin_out<TVK_B_REMAINDER, true>);
    m.impl("atan2", &bin_fn<TVK_B_ATAN2, false>);
    m.impl("atan2_", &bin_fn_<TVK_B_ATAN2, false>);
    m.impl("atan2.out", &bin_out<TVK_B_ATAN2, false>);
    m.impl("floor_divide", &bin_fn<TVK_B_FLOOR_DIVIDE, true>);
    m.impl("floor_divide_.Tensor", &bin_fn_<TVK_B_FLOOR_DIVIDE, true>);
    m.impl("floor_divide.out", &bin_out<TVK_B_FLOOR_DIVIDE, true>);
    m.impl("clamp", &clamp);
    m.impl("clamp_", &clamp_);
    m.impl("clamp.out", &clamp_out);
    m.impl("clamp_min", &clamp_min);
    m.impl("clamp_min_", &clamp_min_);
    m.impl("clamp_min.out", &clamp_min_out);
    m.impl("clamp_max", &clamp_max);
    m.impl("clamp_max_", &clamp_max_);
    m.impl("clamp_max.out", &clamp_max_out);
    m.impl("clamp.Tensor", &clamp_tensor);
    m.impl("clamp.Tensor_out", &clamp_tensor_out);
    m.impl("clamp_min.Tensor", &clamp_min_tensor);
    m.impl("clamp_min.Tensor_out", &clamp_min_tensor_out);
    m.impl("clamp_max.Tensor", &clamp_max_tensor);
    m.impl("clamp_max.Tensor_out", &clamp_max_tensor_out);
    m.impl("threshold", &vk_threshold);
    m.impl("threshold_", &threshold_);
    m.impl("threshold.out", &threshold_out);
    m.impl("hardshrink", &hardshrink);
    m.impl("hardshrink_backward", &hardshrink_backward);
    m.impl("hardtanh", &hardtanh);
    m.impl("hardtanh_", &hardtanh_);
    m.impl("hardtanh.out", &hardtanh_out);
    m.impl("hardtanh_backward", &hardtanh_backward);
    m.impl("leaky_relu", &leaky_relu);
    m.impl("leaky_relu_", &leaky_relu_);
    m.impl("leaky_relu.out", &leaky_relu_out);
    m.impl("leaky_relu_backward", &leaky_relu_backward);
    m.impl("elu", &elu);
    m.impl("elu_", &elu_);
    m.impl("elu.out", &elu_out);
    m.impl("elu_backward", &elu_backward);
    m.impl("softplus", &softplus);
    m.impl("softplus.out", &softplus_out);
    m.impl("softplus_backward", &softplus_backward);
    m.impl("hardswish_backward", &grad_x_fn<TVK_B_HARDSWISH_BACKWARD>);
    m.impl("hardsigmoid_backward", &grad_x_fn<TVK_B_HARDSIGMOID_BACKWARD>);
    m.impl("mish_backward", &grad_x_fn<TVK_B_MISH_BACKWARD>);
    m.impl("log_sigmoid_forward", &log_sigmoid_forward);
    m.impl("log_sigmoid_backward", &log_sigmoid_backward);
    m.impl("logical_and", &logical_fn<TVK_L_AND>);
    m.impl("logical_and_", &logical_fn_<TVK_L_AND>);
    m.impl("logical_and.out", &logical_out<TVK_L_AND>);
    m.impl("logical_or", &logical_fn<TVK_L_OR>);
    m.impl("logical_or_", &logical_fn_<TVK_L_OR>);
    m.impl("logical_or.out", &logical_out<TVK_L_OR>);
    m.impl("logical_xor", &logical_fn<TVK_L_XOR>);
    m.impl("logical_xor.out", &logical_out<TVK_L_XOR>);
    m.impl("logical_not", &logical_not);
    m.impl("logical_not.out", &logical_not_out);
    m.impl("bitwise_and.Tensor", &bitwise_fn<TVK_L_AND>);
    m.impl("bitwise_and.Tensor_out", &bitwise_out<TVK_L_AND>);
    m.impl("bitwise_or.Tensor", &bitwise_fn<TVK_L_OR>);
    m.impl("bitwise_or.Tensor_out", &bitwise_out<TVK_L_OR>);
    m.impl("bitwise_xor.Tensor", &bitwise_fn<TVK_L_XOR>);
    m.impl("bitwise_xor.Tensor_out", &bitwise_out<TVK_L_XOR>);
    m.impl("bitwise_not", &bitwise_not);
    m.impl("bitwise_not.out", &bitwise_not_out);
    m.impl("isnan", &isnan);
    m.impl("isposinf.out", &isposinf_out);
    m.impl("isneginf.out", &isneginf_out);

#define REG_CMP(name, OP)                                   \
    m.impl(name ".Tensor", &cmp_tensor<OP>);                \
    m.impl(name ".Tensor_out", &cmp_tensor_out<OP>);        \
    m.impl(name ".Scalar", &cmp_scalar<OP>);                \
    m.impl(name ".Scalar_out", &cmp_scalar_out<OP>)
    REG_CMP("eq", TVK_C_EQ);
    REG_CMP("ne", TVK_C_NE);
    REG_CMP("lt", TVK_C_LT);
    REG_CMP("le", TVK_C_LE);
    REG_CMP("gt", TVK_C_GT);
    REG_CMP("ge", TVK_C_GE);
#undef REG_CMP

    m.impl("lerp.Tensor", &lerp_tensor);
    m.impl("lerp_.Tensor", &lerp_tensor_);
    m.impl("lerp.Tensor_out", &lerp_tensor_out);
    m.impl("addcmul", &addcmul);
    m.impl("addcmul_", &addcmul_);
    m.impl("addcmul.out", &addcmul_out);
    m.impl("addcdiv", &addcdiv);
    m.impl("addcdiv_", &addcdiv_);
    m.impl("addcdiv.out", &addcdiv_out);
    m.impl("lerp.Scalar", &lerp_scalar);
    m.impl("lerp_.Scalar", &lerp_scalar_);
    m.impl("lerp.Scalar_out", &lerp_scalar_out);
    m.impl("where.self", &where_self);

    m.impl("fill_.Scalar", &fill_scalar_);
    m.impl("fill_.Tensor", &fill_tensor_);
    m.impl("zero_", &zero_);
}

}  // namespace tvk_aten
