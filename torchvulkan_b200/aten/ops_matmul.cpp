// aten::mm / addmm / bmm / baddbmm / _addmm_activation (+ .out) for the "vulkan" device.
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
}

}  // namespace tvk_aten
