// aten::mm / addmm / bmm / baddbmm / addbmm / addmv / dot / _addmm_activation / _scaled_mm (+ .out) for the "vulkan" device.
//
// Counterparts in the reference: mm_vulkan ... addmm_activation_vulkan and their .out wrappers
// (src/api/ops/matmul.cpp:598-763). The checks and their messages follow ATen's CPU ops as the
// reference's do (matmul.cpp:598-606, 622-630); operands are handed to tvk_gemm with their
// strides so transposed views are consumed in place (matmul.cpp:342-353), the bias is passed
// with broadcast strides (matmul.cpp:49-53), and the result is a fresh contiguous tensor.
// There is no CPU fallback: dtypes outside fp32/fp16/bf16 raise.
#include "common.h"

namespace tvk_aten {
namespace {

void check_matrix_product(const char* name, const at::Tensor& mat1, const at::Tensor& mat2) {
    TORCH_CHECK(mat1.dim() == 2, name, ": self must be a matrix, got ", mat1.dim(), "-D tensor");
    TORCH_CHECK(mat2.dim() == 2, name, ": mat2 must be a matrix, got ", mat2.dim(), "-D tensor");
    TORCH_CHECK(mat1.size(1) == mat2.size(0), name, ": mat1 and mat2 shapes cannot be multiplied (", mat1.size(0), "x", mat1.size(1),
                " and ", mat2.size(0), "x", mat2.size(1), ")");
}

void check_same(const at::Tensor& a, const at::Tensor& b) {
    TORCH_CHECK(a.device() == b.device(), "Expected all tensors to be on the same device, but found at least two devices, ", a.device(), " and ",
                b.device(), "!");
    TORCH_CHECK(a.scalar_type() == b.scalar_type(), "expected scalar type ", a.scalar_type(), " but found ", b.scalar_type());
}

// An operand the kernels can address: one unit stride (or a degenerate dim). Anything else is
// copied once (the reference does the same with .contiguous(), matmul.cpp:41-42).
at::Tensor addressable(const at::Tensor& t) {
    const int64_t r = t.dim() - 2, c = t.dim() - 1;
    const bool ok = t.stride(c) == 1 || t.stride(r) == 1 || t.size(r) == 1 || t.size(c) == 1;
    bool nonneg = true;
    for (int64_t d = 0; d < t.dim(); ++d) nonneg = nonneg && t.stride(d) >= 0;
    return (ok && nonneg) ? t : contiguous_vulkan(t);
}

// out[B?, m, n] = act(alpha * a @ b + beta * bias)
at::Tensor run_gemm(const at::Tensor& a_in, const at::Tensor& b_in, const c10::optional<at::Tensor>& bias_in, double alpha, double beta,
                    int activation) {
    const at::ScalarType st = a_in.scalar_type();
    if (!is_hot_float(st)) TVK_NOT_IMPLEMENTED("matmul for dtype ", st, " on the vulkan device");
    check_same(a_in, b_in);
    const bool batched = a_in.dim() == 3;
    at::Tensor a = addressable(a_in), b = addressable(b_in);
    const int64_t batch = batched ? a.size(0) : 1;
    const int64_t m = a.size(-2), k = a.size(-1), n = b.size(-1);
    std::vector<int64_t> shape = batched ? std::vector<int64_t>{batch, m, n} : std::vector<int64_t>{m, n};
    at::Tensor out = empty_vulkan(shape, st, a.device());
    if (out.numel() == 0) return out;

    tvk_gemm_desc d = {};
    d.dtype = to_tvk_dtype(st);
    d.activation = activation;
    d.batch = batch; d.m = m; d.n = n; d.k = k;
    d.a = a.data_ptr(); d.a_rs = a.stride(-2); d.a_cs = a.stride(-1); d.a_bs = batched && batch > 1 ? a.stride(0) : 0;
    d.b = b.data_ptr(); d.b_rs = b.stride(-2); d.b_cs = b.stride(-1); d.b_bs = batched && batch > 1 ? b.stride(0) : 0;
    d.c = out.data_ptr(); d.c_rs = n; d.c_bs = m * n;
    d.alpha = (float)alpha; d.beta = (float)beta;
    at::Tensor bias;
    if (bias_in.has_value() && bias_in->defined() && beta != 0.0) {
        check_same(a_in, *bias_in);
        bias = bias_in->expand(shape);  // broadcast as strides of zero (matmul.cpp:49-53)
        d.bias = bias.data_ptr();
        d.bias_rs = bias.stride(-2); d.bias_cs = bias.stride(-1); d.bias_bs = batched ? bias.stride(0) : 0;
    }
    DeviceScope scope(a);
    uint64_t ws_bytes = 0;
    TVK_CALL(tvk_gemm_workspace_size(&d, &ws_bytes));
    Workspace ws(scope.device, ws_bytes);
    TVK_CALL(tvk_gemm(&d, ws.ptr, ws.bytes, scope.stream));
    return out;
}

at::Tensor& fill_out(at::Tensor& out, const at::Tensor& result) {
    TORCH_CHECK(out.device() == result.device(), "Expected out tensor to be on the same device as the inputs");
    if (out.sizes() != result.sizes()) out.resize_(result.sizes());
    out.copy_(result);
    return out;
}

at::Tensor mm(const at::Tensor& self, const at::Tensor& other) {
    check_matrix_product("mm", self, other);
    return run_gemm(self, other, c10::nullopt, 1.0, 0.0, TVK_ACT_NONE);
}

void check_bmm(const at::Tensor& self, const at::Tensor& other) {
    TORCH_CHECK(self.dim() == 3, "batch1 must be a 3D tensor");
    TORCH_CHECK(other.dim() == 3, "batch2 must be a 3D tensor");
    TORCH_CHECK(other.size(0) == self.size(0) && other.size(1) == self.size(2), "Expected size for first two dimensions of batch2 tensor to be: [",
                self.size(0), ", ", self.size(2), "] but got: [", other.size(0), ", ", other.size(1), "].");
}

at::Tensor bmm(const at::Tensor& self, const at::Tensor& other) {
    check_bmm(self, other);
    return run_gemm(self, other, c10::nullopt, 1.0, 0.0, TVK_ACT_NONE);
}

at::Tensor addmm(const at::Tensor& input, const at::Tensor& mat1, const at::Tensor& mat2, const at::Scalar& beta, const at::Scalar& alpha) {
    check_matrix_product("addmm", mat1, mat2);
    return run_gemm(mat1, mat2, input, alpha.toDouble(), beta.toDouble(), TVK_ACT_NONE);
}

at::Tensor baddbmm(const at::Tensor& input, const at::Tensor& b1, const at::Tensor& b2, const at::Scalar& beta, const at::Scalar& alpha) {
    TORCH_CHECK(input.scalar_type() == b1.scalar_type() && b1.scalar_type() == b2.scalar_type(), "Input dtypes must be the same, got: input ",
                input.dtype().name(), ", batch1: ", b1.dtype().name(), ", batch2: ", b2.dtype().name());
    check_bmm(b1, b2);
    return run_gemm(b1, b2, input, alpha.toDouble(), beta.toDouble(), TVK_ACT_NONE);
}

at::Tensor addmm_activation(const at::Tensor& input, const at::Tensor& mat1, const at::Tensor& mat2, const at::Scalar& beta,
                            const at::Scalar& alpha, bool use_gelu) {
    check_matrix_product("addmm", mat1, mat2);
    return run_gemm(mat1, mat2, input, alpha.toDouble(), beta.toDouble(), use_gelu ? TVK_ACT_GELU : TVK_ACT_RELU);
}

// addbmm: beta * self + alpha * sum over the batches of batch1[b] @ batch2[b]. The sum over b is folded into the contraction
// (addbmm_vulkan, src/api/decompositions.cpp:1114-1129): batch1 as one [n, b*k] matrix (a copy: the batch index is not a
// plain stride of a matrix column), batch2 as [b*k, p] in place, and ONE product with the whole epilogue (alpha, beta * self).
at::Tensor addbmm(const at::Tensor& self, const at::Tensor& batch1, const at::Tensor& batch2, const at::Scalar& beta, const at::Scalar& alpha) {
    TORCH_CHECK(batch1.dim() == 3 && batch2.dim() == 3, "batch1 and batch2 must be 3D tensors");
    TORCH_CHECK(batch1.size(0) == batch2.size(0), "batch1 and batch2 must have same number of batches, got ", batch1.size(0), " and ", batch2.size(0));
    TORCH_CHECK(batch1.size(2) == batch2.size(1), "Incompatible matrix sizes for bmm (", batch1.size(1), "x", batch1.size(2), " and ", batch2.size(1), "x",
                batch2.size(2), ")");
    const int64_t b = batch1.size(0), n = batch1.size(1), k = batch1.size(2), p = batch2.size(2);
    if (!is_hot_float(self.scalar_type())) TVK_NOT_IMPLEMENTED("addbmm for dtype ", self.scalar_type(), " on the vulkan device");
    if (b == 0 || k == 0) return at::mul(self.expand({n, p}), beta).contiguous();
    at::Tensor a2 = batch1.permute({1, 0, 2}).reshape({n, b * k});
    at::Tensor b2 = batch2.is_contiguous() ? batch2.view({b * k, p}) : batch2.reshape({b * k, p});
    return run_gemm(a2, b2, self, alpha.toDouble(), beta.toDouble(), TVK_ACT_NONE);
}
at::Tensor& addbmm_out(const at::Tensor& self, const at::Tensor& b1, const at::Tensor& b2, const at::Scalar& beta, const at::Scalar& alpha, at::Tensor& out) {
    return fill_out(out, (addbmm)(self, b1, b2, beta, alpha));
}
at::Tensor& addbmm_(at::Tensor& self, const at::Tensor& b1, const at::Tensor& b2, const at::Scalar& beta, const at::Scalar& alpha) {
    return fill_out(self, (addbmm)(self, b1, b2, beta, alpha));
}

// addmv / mv: a product with one output column (addmv_out_vulkan, src/api/decompositions.cpp:109-124); the vector and the
// result are addressed as [k, 1] and [m, 1] views, so nothing is copied.
at::Tensor& addmv_out(const at::Tensor& self, const at::Tensor& mat, const at::Tensor& vec, const at::Scalar& beta, const at::Scalar& alpha,
                      at::Tensor& out) {
    TORCH_CHECK(mat.dim() == 2 && vec.dim() == 1, "vector + matrix @ vector expected, got ", self.dim(), ", ", mat.dim(), ", ", vec.dim());
    TORCH_CHECK(mat.size(1) == vec.size(0), "size mismatch, got input (", self.size(0), "), mat (", mat.size(0), "x", mat.size(1), "), vec (", vec.size(0), ")");
    TORCH_CHECK(out.scalar_type() == mat.scalar_type(), "Expected out tensor to have dtype ", mat.scalar_type(), ", but got ", out.scalar_type(), " instead");
    if (!is_hot_float(mat.scalar_type())) TVK_NOT_IMPLEMENTED("addmv for dtype ", mat.scalar_type(), " on the vulkan device");
    const bool use_self = beta.toDouble() != 0.0;
    at::Tensor bias = use_self ? self.expand({mat.size(0)}).unsqueeze(1) : at::Tensor();
    at::Tensor r = mat.size(1) == 0 ? (use_self ? at::mul(self.expand({mat.size(0)}), beta).contiguous() : at::zeros({mat.size(0)}, mat.options()))
                                    : run_gemm(mat, vec.unsqueeze(1), use_self ? c10::optional<at::Tensor>(bias) : c10::nullopt, alpha.toDouble(),
                                               beta.toDouble(), TVK_ACT_NONE).squeeze(1);
    return fill_out(out, r);
}

// dot: the reference multiplies and sums in fp32 (dot_vulkan, src/api/decompositions.cpp:46-58); as a [1, k] x [k, 1]
// product the accumulation is fp32 too and nothing is materialised.
at::Tensor dot(const at::Tensor& self, const at::Tensor& other) {
    TORCH_CHECK(self.dim() == 1 && other.dim() == 1, "1D tensors expected, but got ", self.dim(), "D and ", other.dim(), "D tensors");
    TORCH_CHECK(self.scalar_type() == other.scalar_type(), "dot : expected both vectors to have same dtype, but found ", self.scalar_type(), " and ",
                other.scalar_type());
    TORCH_CHECK(self.numel() == other.numel(), "inconsistent tensor size, expected tensor [", self.numel(), "] and src [", other.numel(),
                "] to have the same number of elements, but got ", self.numel(), " and ", other.numel(), " elements respectively");
    if (!is_hot_float(self.scalar_type())) TVK_NOT_IMPLEMENTED("dot for dtype ", self.scalar_type(), " on the vulkan device");
    if (self.numel() == 0) return at::zeros({}, self.options());
    return run_gemm(self.unsqueeze(0), other.unsqueeze(1), c10::nullopt, 1.0, 0.0, TVK_ACT_NONE).reshape({});
}

at::Tensor& mm_out(const at::Tensor& self, const at::Tensor& other, at::Tensor& out) { return fill_out(out, (mm)(self, other)); }
at::Tensor& bmm_out(const at::Tensor& self, const at::Tensor& other, at::Tensor& out) { return fill_out(out, (bmm)(self, other)); }
at::Tensor& addmm_out(const at::Tensor& input, const at::Tensor& m1, const at::Tensor& m2, const at::Scalar& beta, const at::Scalar& alpha,
                      at::Tensor& out) {
    return fill_out(out, (addmm)(input, m1, m2, beta, alpha));
}
at::Tensor& addmm_(at::Tensor& self, const at::Tensor& m1, const at::Tensor& m2, const at::Scalar& beta, const at::Scalar& alpha) {
    return fill_out(self, (addmm)(self, m1, m2, beta, alpha));
}
at::Tensor& baddbmm_out(const at::Tensor& input, const at::Tensor& b1, const at::Tensor& b2, const at::Scalar& beta, const at::Scalar& alpha,
                        at::Tensor& out) {
    return fill_out(out, (baddbmm)(input, b1, b2, beta, alpha));
}
at::Tensor& baddbmm_(at::Tensor& self, const at::Tensor& b1, const at::Tensor& b2, const at::Scalar& beta, const at::Scalar& alpha) {
    return fill_out(self, (baddbmm)(self, b1, b2, beta, alpha));
}
at::Tensor& addmm_activation_out(const at::Tensor& input, const at::Tensor& m1, const at::Tensor& m2, const at::Scalar& beta,
                                 const at::Scalar& alpha, bool use_gelu, at::Tensor& out) {
    return fill_out(out, (addmm_activation)(input, m1, m2, beta, alpha, use_gelu));
}

// ---- _scaled_mm (src/api/ops/matmul.cpp:706-747): the same checks and messages, then tvk_scaled_mm -------------------
int scaled_out_kind(at::ScalarType st) {
    switch (st) {
        case at::kFloat: return TVK_SCALED_OUT_F32;
        case at::kHalf: return TVK_SCALED_OUT_F16;
        case at::kBFloat16: return TVK_SCALED_OUT_BF16;
        case at::kFloat8_e4m3fn: return TVK_SCALED_OUT_E4M3;
        case at::kFloat8_e5m2: return TVK_SCALED_OUT_E5M2;
        default: return -1;
    }
}
int f8_kind(at::ScalarType st) { return st == at::kFloat8_e5m2 ? TVK_F8_E5M2 : TVK_F8_E4M3; }

at::Tensor& scaled_mm_out(const at::Tensor& mat1, const at::Tensor& mat2, const at::Tensor& scale_a, const at::Tensor& scale_b,
                          const std::optional<at::Tensor>& bias, const std::optional<at::Tensor>& scale_result, std::optional<at::ScalarType> out_dtype,
                          bool /*use_fast_accum*/, at::Tensor& out) {
    TORCH_CHECK_VALUE(!out_dtype || *out_dtype == out.scalar_type(), "out_dtype must match output matrix type");
    TORCH_CHECK(mat1.dim() == 2, "mat1 must be a matrix");
    TORCH_CHECK(mat2.dim() == 2, "mat2 must be a matrix");
    TORCH_CHECK(mat1.size(1) == mat2.size(0), "mat_a and mat_b shapes cannot be multiplied (", mat1.size(0), "x", mat1.size(1), " and ", mat2.size(0), "x",
                mat2.size(1), ")");
    const auto is_f8 = [](at::ScalarType st) { return st == at::kFloat8_e4m3fn || st == at::kFloat8_e5m2; };
    TORCH_CHECK_VALUE(at::isFloat8Type(mat1.scalar_type()) && at::isFloat8Type(mat2.scalar_type()), "mat1 and mat2 must be fp8 types, got: ", mat1.scalar_type(),
                      mat2.scalar_type());
    if (!is_f8(mat1.scalar_type()) || !is_f8(mat2.scalar_type())) TVK_NOT_IMPLEMENTED("_scaled_mm for ", mat1.scalar_type(), " and ", mat2.scalar_type(), " (e4m3fn and e5m2 are supported)");
    const bool tensorwise = scale_a.numel() == 1 && scale_b.numel() == 1;
    const bool rowwise = scale_a.dim() == 2 && scale_b.dim() == 2 && scale_a.size(0) == mat1.size(0) && scale_a.size(1) == 1 && scale_b.size(0) == 1 &&
                         scale_b.size(1) == mat2.size(1);
    TORCH_CHECK_VALUE(tensorwise || rowwise, "Invalid scaling configuration");
    TORCH_CHECK_VALUE(scale_a.scalar_type() == at::kFloat, "scale_a must have Float elements");
    TORCH_CHECK_VALUE(scale_b.scalar_type() == at::kFloat, "scale_b must have Float elements");
    TORCH_CHECK(!scale_result || (scale_result->numel() == 1 && scale_result->scalar_type() == at::kFloat), "scale_result must be a float scalar");
    TORCH_CHECK(!bias || bias->numel() == mat2.size(1), "Bias must be size ", mat2.size(1), " but got ", bias->numel());
    for (const at::Tensor* t : {&mat2, &scale_a, &scale_b})
        TORCH_CHECK(t->device() == mat1.device(), "Expected all tensors to be on the same device, but found at least two devices, ", mat1.device(), " and ", t->device(), "!");
    const int kind = scaled_out_kind(out.scalar_type());
    if (kind < 0) TVK_NOT_IMPLEMENTED("_scaled_mm with output dtype ", out.scalar_type());

    const int64_t m = mat1.size(0), k = mat1.size(1), n = mat2.size(1);
    const bool direct = out.is_contiguous() && out.dim() == 2 && out.size(0) == m && out.size(1) == n;
    at::Tensor dst = out;
    if (!direct) {
        if (out.sizes() != at::IntArrayRef({m, n})) out.resize_({m, n});
        dst = out.is_contiguous() ? out : empty_vulkan({m, n}, out.scalar_type(), out.device());
    }
    if (m > 0 && n > 0) {
        at::Tensor sa = contiguous_vulkan(scale_a), sb = contiguous_vulkan(scale_b), bs, sr;
        tvk_scaled_mm_desc d = {};
        d.a_kind = f8_kind(mat1.scalar_type()); d.b_kind = f8_kind(mat2.scalar_type()); d.out_kind = kind;
        d.m = m; d.n = n; d.k = k;
        d.a = mat1.data_ptr(); d.a_rs = mat1.stride(0); d.a_cs = mat1.stride(1);
        d.b = mat2.data_ptr(); d.b_rs = mat2.stride(0); d.b_cs = mat2.stride(1);
        d.out = dst.data_ptr();
        d.scale_a = sa.data_ptr<float>(); d.sa_stride = tensorwise ? 0 : 1;
        d.scale_b = sb.data_ptr<float>(); d.sb_stride = tensorwise ? 0 : 1;
        if (bias && bias->defined()) {
            bs = contiguous_vulkan(*bias);
            if (!is_hot_float(bs.scalar_type())) TVK_NOT_IMPLEMENTED("_scaled_mm with a bias of dtype ", bs.scalar_type());
            d.bias = bs.data_ptr(); d.bias_dtype = to_tvk_dtype(bs.scalar_type());
        }
        if (scale_result && scale_result->defined()) {
            sr = contiguous_vulkan(*scale_result);
            d.scale_result = sr.data_ptr<float>();
        }
        DeviceScope scope(mat1);
        uint64_t ws_bytes = 0;
        TVK_CALL(tvk_scaled_mm_workspace_size(&d, &ws_bytes));
        Workspace ws(scope.device, ws_bytes);
        TVK_CALL(tvk_scaled_mm(&d, ws.ptr, ws.bytes, scope.stream));
    }
    if (!dst.is_same(out)) out.copy_(dst);
    return out;
}

at::Tensor scaled_mm(const at::Tensor& mat1, const at::Tensor& mat2, const at::Tensor& scale_a, const at::Tensor& scale_b, const std::optional<at::Tensor>& bias,
                     const std::optional<at::Tensor>& scale_result, std::optional<at::ScalarType> out_dtype, bool use_fast_accum) {
    // as the reference: without out_dtype the result has mat1's (float8) type
    at::Tensor out = empty_vulkan({mat1.dim() == 2 ? mat1.size(0) : 0, mat2.dim() == 2 ? mat2.size(1) : 0}, out_dtype.value_or(mat1.scalar_type()), mat1.device());
    return scaled_mm_out(mat1, mat2, scale_a, scale_b, bias, scale_result, out_dtype, use_fast_accum, out);
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("mm", &mm);
    m.impl("mm.out", &mm_out);
    m.impl("bmm", &bmm);
    m.impl("bmm.out", &bmm_out);
    m.impl("addmm", &addmm);
    m.impl("addmm.out", &addmm_out);
    m.impl("addmm_", &addmm_);
    m.impl("baddbmm", &baddbmm);
    m.impl("baddbmm.out", &baddbmm_out);
    m.impl("baddbmm_", &baddbmm_);
    m.impl("addbmm", &addbmm);
    m.impl("addbmm.out", &addbmm_out);
    m.impl("addbmm_", &addbmm_);
    m.impl("addmv.out", &addmv_out);
    m.impl("dot", &dot);
    m.impl("_addmm_activation", &addmm_activation);
    m.impl("_addmm_activation.out", &addmm_activation_out);
    m.impl("_scaled_mm", &scaled_mm);
    m.impl("_scaled_mm.out", &scaled_mm_out);
}

}  // namespace tvk_aten
