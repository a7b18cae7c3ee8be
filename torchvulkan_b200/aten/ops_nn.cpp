// Softmax family, nll_loss, RMSNorm, BatchNorm, embedding, cat and the fused optimizer steps for
// the "vulkan" device.
//
// Counterparts in the reference: softmax_vulkan / log_softmax_vulkan and their backward
// (src/api/decompositions.cpp:506-571), nll_loss_forward/backward_vulkan (src/api/ops/nllloss.cpp:79-211),
// fused_rms_norm_vulkan (+backward) and the batch-norm entry points (src/api/ops/norm.cpp:169-433,
// src/api/ops/nn.cpp:44-291), embedding_vulkan / embedding_dense_backward_vulkan
// (src/api/ops/indexing.cpp:299-345), cat (decompositions.cpp:355-414), fused_adam(w) / fused_sgd
// (src/api/ops/optim.cpp:46-277). Each op is one or two launches of the tvk kernels; half types
// compute in fp32 and round once, as the reference does.
#include "common.h"

namespace tvk_aten {
namespace {

void require_float(const at::Tensor& t, const char* op) {
    if (!is_hot_float(t.scalar_type())) TVK_NOT_IMPLEMENTED(op, " for dtype ", t.scalar_type(), " on the vulkan device");
}

// ---- softmax ----------------------------------------------------------------------------
at::Tensor softmax_impl(bool log, const at::Tensor& self, int64_t dim, bool half_to_float) {
    require_float(self, log ? "_log_softmax" : "_softmax");
    const int64_t nd = std::max<int64_t>(self.dim(), 1);
    dim = at::maybe_wrap_dim(dim, nd);
    const at::ScalarType out_st = half_to_float ? at::kFloat : self.scalar_type();
    at::Tensor x = self.dim() == 0 ? self.reshape({1}) : self;
    const bool last = dim == nd - 1;
    at::Tensor xc = contiguous_vulkan(last ? x : x.transpose(dim, -1));
    at::Tensor out = empty_vulkan(xc.sizes(), out_st, self.device());
    const int64_t cols = xc.size(-1), rows = cols ? xc.numel() / cols : 0;
    if (out.numel()) {
        DeviceScope scope(self);
        TVK_CALL(tvk_softmax_forward(log, to_tvk_dtype(self.scalar_type()), to_tvk_dtype(out_st), out.data_ptr(), xc.data_ptr(), rows, cols,
                                     scope.stream));
    }
    if (!last) out = contiguous_vulkan(out.transpose(dim, -1));
    return self.dim() == 0 ? out.reshape({}) : out;
}
at::Tensor softmax_bwd_impl(bool log, const at::Tensor& grad, const at::Tensor& output, int64_t dim, at::ScalarType input_dtype) {
    require_float(grad, log ? "_log_softmax_backward_data" : "_softmax_backward_data");
    const int64_t nd = std::max<int64_t>(grad.dim(), 1);
    dim = at::maybe_wrap_dim(dim, nd);
    at::Tensor g = grad.dim() == 0 ? grad.reshape({1}) : grad, y = output.dim() == 0 ? output.reshape({1}) : output;
    const at::ScalarType st = g.scalar_type();
    if (y.scalar_type() != st) y = y.to(st);
    const bool last = dim == nd - 1;
    at::Tensor gc = contiguous_vulkan(last ? g : g.transpose(dim, -1)), yc = contiguous_vulkan(last ? y : y.transpose(dim, -1));
    at::Tensor out = empty_vulkan(gc.sizes(), st, grad.device());
    const int64_t cols = gc.size(-1), rows = cols ? gc.numel() / cols : 0;
    if (out.numel()) {
        DeviceScope scope(grad);
        TVK_CALL(tvk_softmax_backward(log, to_tvk_dtype(st), out.data_ptr(), gc.data_ptr(), yc.data_ptr(), rows, cols, scope.stream));
    }
    if (!last) out = contiguous_vulkan(out.transpose(dim, -1));
    if (out.scalar_type() != input_dtype) out = out.to(input_dtype);
    return grad.dim() == 0 ? out.reshape({}) : out;
}
at::Tensor log_softmax(const at::Tensor& self, int64_t dim, bool h2f) { return softmax_impl(true, self, dim, h2f); }
at::Tensor softmax(const at::Tensor& self, int64_t dim, bool h2f) { return softmax_impl(false, self, dim, h2f); }
at::Tensor log_softmax_bwd(const at::Tensor& g, const at::Tensor& o, int64_t dim, at::ScalarType dt) { return softmax_bwd_impl(true, g, o, dim, dt); }
at::Tensor softmax_bwd(const at::Tensor& g, const at::Tensor& o, int64_t dim, at::ScalarType dt) { return softmax_bwd_impl(false, g, o, dim, dt); }
at::Tensor& copy_into(at::Tensor& out, const at::Tensor& r) {
    if (out.sizes() != r.sizes()) out.resize_(r.sizes());
    out.copy_(r);
    return out;
}
at::Tensor& log_softmax_out(const at::Tensor& s, int64_t d, bool h, at::Tensor& out) { return copy_into(out, (log_softmax)(s, d, h)); }
at::Tensor& softmax_out(const at::Tensor& s, int64_t d, bool h, at::Tensor& out) { return copy_into(out, (softmax)(s, d, h)); }
at::Tensor& log_softmax_bwd_out(const at::Tensor& g, const at::Tensor& o, int64_t d, at::ScalarType dt, at::Tensor& out) { return copy_into(out, (log_softmax_bwd)(g, o, d, dt)); }
at::Tensor& softmax_bwd_out(const at::Tensor& g, const at::Tensor& o, int64_t d, at::ScalarType dt, at::Tensor& out) { return copy_into(out, (softmax_bwd)(g, o, d, dt)); }

// ---- nll_loss ---------------------------------------------------------------------------
std::tuple<at::Tensor, at::Tensor> nll_loss_forward(const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight,
                                                    int64_t reduction, c10::SymInt ignore_index) {
    require_float(self, "nll_loss_forward");
    TORCH_CHECK(self.dim() >= 1 && self.dim() <= 2, "input tensor should be 1D or 2D");
    TORCH_CHECK(target.dim() <= 1, "0D or 1D target tensor expected, multi-target not supported");
    TORCH_CHECK(target.scalar_type() == at::kLong, "expected scalar type Long but found ", target.scalar_type());
    at::Tensor x = contiguous_vulkan(self.dim() == 1 ? self.unsqueeze(0) : self);
    at::Tensor t = contiguous_vulkan(target.dim() == 0 ? target.unsqueeze(0) : target);
    const int64_t n = x.size(0), c = x.size(1);
    TORCH_CHECK(t.size(0) == n, "Expected input batch_size (", n, ") to match target batch_size (", t.size(0), ").");
    at::Tensor w;
    if (weight.has_value() && weight->defined()) {
        TORCH_CHECK(weight->numel() == c, "weight tensor should be defined either for all ", c, " classes or no classes but got weight tensor of shape: ", weight->sizes());
        w = contiguous_vulkan(weight->to(self.scalar_type()));
    }
    const bool none = reduction == at::Reduction::None;
    at::Tensor out = empty_vulkan(none ? (self.dim() == 1 ? std::vector<int64_t>{} : std::vector<int64_t>{n}) : std::vector<int64_t>{}, self.scalar_type(), self.device());
    at::Tensor total = empty_vulkan({}, self.scalar_type(), self.device());
    DeviceScope scope(self);
    const int red = none ? 0 : (reduction == at::Reduction::Mean ? 1 : 2);
    TVK_CALL(tvk_nll_loss_forward(to_tvk_dtype(self.scalar_type()), out.data_ptr(), total.data_ptr(), x.data_ptr(), (const int64_t*)t.data_ptr(),
                                  w.defined() ? w.data_ptr() : nullptr, n, c, red, ignore_index.guard_int(__FILE__, __LINE__), scope.stream));
    return {out, total};
}

at::Tensor nll_loss_backward(const at::Tensor& grad_output, const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight,
                             int64_t reduction, c10::SymInt ignore_index, const at::Tensor& total_weight) {
    require_float(self, "nll_loss_backward");
    const bool one_d = self.dim() == 1;
    const int64_t n = one_d ? 1 : self.size(0), c = one_d ? self.size(0) : self.size(1);
    at::Tensor t = contiguous_vulkan(target.dim() == 0 ? target.unsqueeze(0) : target);
    at::Tensor g = contiguous_vulkan(grad_output.to(self.scalar_type()));
    at::Tensor tw = total_weight.to(self.scalar_type());
    at::Tensor w;
    if (weight.has_value() && weight->defined()) w = contiguous_vulkan(weight->to(self.scalar_type()));
    at::Tensor gin = empty_vulkan(self.sizes(), self.scalar_type(), self.device());
    if (gin.numel() == 0) return gin;
    const bool none = reduction == at::Reduction::None;
    const int red = none ? 0 : (reduction == at::Reduction::Mean ? 1 : 2);
    DeviceScope scope(self);
    TVK_CALL(tvk_nll_loss_backward(to_tvk_dtype(self.scalar_type()), gin.data_ptr(), g.data_ptr(), (const int64_t*)t.data_ptr(),
                                   w.defined() ? w.data_ptr() : nullptr, tw.data_ptr(), n, c, red, ignore_index.guard_int(__FILE__, __LINE__),
                                   scope.stream));
    return gin;
}

// ---- RMSNorm ----------------------------------------------------------------------------
std::tuple<at::Tensor, at::Tensor> fused_rms_norm(const at::Tensor& input, at::IntArrayRef normalized_shape, const c10::optional<at::Tensor>& weight,
                                                  c10::optional<double> eps) {
    require_float(input, "_fused_rms_norm");
    int64_t cols = 1;
    for (int64_t s : normalized_shape) cols *= s;
    TORCH_CHECK(cols > 0 && input.numel() % cols == 0, "torchvulkan [ERROR]: rms_norm: normalized_shape does not match the input");
    at::Tensor x = contiguous_vulkan(input);
    const int64_t rows = x.numel() / cols;
    at::Tensor w;
    if (weight.has_value() && weight->defined()) w = contiguous_vulkan(weight->to(input.scalar_type()));
    at::Tensor y = empty_like_contig(x);
    std::vector<int64_t> stat_shape(input.sizes().begin(), input.sizes().end() - normalized_shape.size());
    for (size_t i = 0; i < normalized_shape.size(); ++i) stat_shape.push_back(1);
    at::Tensor rstd = empty_vulkan(stat_shape, at::kFloat, input.device());   // fp32 statistics (norm.cpp:198-200)
    if (x.numel()) {
        DeviceScope scope(input);
        const double e = eps.value_or((double)std::numeric_limits<float>::epsilon());   // norm.cpp:177
        TVK_CALL(tvk_rmsnorm_forward(to_tvk_dtype(input.scalar_type()), y.data_ptr(), (float*)rstd.data_ptr(), x.data_ptr(),
                                     w.defined() ? w.data_ptr() : nullptr, rows, cols, e, scope.stream));
    }
    return {y, rstd};
}

std::tuple<at::Tensor, at::Tensor> fused_rms_norm_backward(const at::Tensor& grad_out, const at::Tensor& input, at::IntArrayRef normalized_shape,
                                                           const at::Tensor& rstd, const c10::optional<at::Tensor>& weight,
                                                           std::array<bool, 2> output_mask) {
    require_float(input, "_fused_rms_norm_backward");
    int64_t cols = 1;
    for (int64_t s : normalized_shape) cols *= s;
    at::Tensor x = contiguous_vulkan(input), g = contiguous_vulkan(grad_out.to(input.scalar_type()));
    at::Tensor rs = contiguous_vulkan(rstd.to(at::kFloat));
    const int64_t rows = cols ? x.numel() / cols : 0;
    at::Tensor w;
    if (weight.has_value() && weight->defined()) w = contiguous_vulkan(weight->to(input.scalar_type()));
    at::Tensor gx = empty_like_contig(x), gw;
    const bool want_w = output_mask[1] && w.defined();
    if (want_w) gw = empty_vulkan(w.sizes(), input.scalar_type(), input.device());
    if (x.numel()) {
        DeviceScope scope(input);
        uint64_t ws_bytes = 0;
        TVK_CALL(tvk_rmsnorm_backward_workspace_size(rows, cols, &ws_bytes));
        Workspace ws(scope.device, want_w ? ws_bytes : 0);
        TVK_CALL(tvk_rmsnorm_backward(to_tvk_dtype(input.scalar_type()), gx.data_ptr(), want_w ? gw.data_ptr() : nullptr, g.data_ptr(), x.data_ptr(),
                                      w.defined() ? w.data_ptr() : nullptr, (const float*)rs.data_ptr(), rows, cols, ws.ptr, ws.bytes, scope.stream));
    }
    return {output_mask[0] ? gx : at::Tensor(), gw};
}

// ---- BatchNorm (training) ---------------------------------------------------------------
// A 4-D tensor in channels-last memory whose channel count the channels-last kernels accept.
bool bn_channels_last(const at::Tensor& t) {
    if (t.dim() != 4 || t.is_contiguous() || !t.is_contiguous(at::MemoryFormat::ChannelsLast)) return false;
    const int64_t packet = 16 / (int64_t)t.element_size();
    return t.size(1) % packet == 0 && (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> batch_norm_train(const at::Tensor& input, const c10::optional<at::Tensor>& weight,
                                                                const c10::optional<at::Tensor>& bias, at::Tensor* running_mean,
                                                                at::Tensor* running_var, bool training, double momentum, double eps) {
    require_float(input, "native_batch_norm");
    TORCH_CHECK(input.dim() >= 2, "torchvulkan [ERROR]: batch_norm expects at least a 2-D input");
    if (!training) {
        // evaluation mode: one pass with the running statistics; the input's memory format is kept
        TORCH_CHECK(running_mean && running_mean->defined() && running_var && running_var->defined(),
                    "torchvulkan [ERROR]: batch_norm in evaluation mode needs running_mean and running_var");
        TORCH_CHECK(running_mean->is_contiguous() && running_var->is_contiguous() && running_mean->scalar_type() == running_var->scalar_type(),
                    "torchvulkan [ERROR]: running statistics must be contiguous and of one dtype");
        const bool cl = input.dim() == 4 && !input.is_contiguous() && input.is_contiguous(at::MemoryFormat::ChannelsLast);
        at::Tensor x = cl ? input : contiguous_vulkan(input);
        const at::ScalarType st = input.scalar_type();
        at::Tensor w, b;
        if (weight.has_value() && weight->defined()) w = contiguous_vulkan(weight->to(st));
        if (bias.has_value() && bias->defined()) b = contiguous_vulkan(bias->to(st));
        at::Tensor y = cl ? at::empty_strided(input.sizes(), input.strides(), input.options()) : empty_like_contig(x);
        const int64_t n = x.size(0), c = x.size(1), hw = (n * c) ? x.numel() / (n * c) : 0;
        if (x.numel()) {
            DeviceScope scope(input);
            TVK_CALL(tvk_batchnorm_inference(to_tvk_dtype(st), y.data_ptr(), x.data_ptr(), w.defined() ? w.data_ptr() : nullptr,
                                             b.defined() ? b.data_ptr() : nullptr, to_tvk_dtype(running_mean->scalar_type()), running_mean->data_ptr(),
                                             running_var->data_ptr(), n, c, hw, cl ? 1 : 0, eps, scope.stream));
        }
        return {y, empty_vulkan({0}, at::kFloat, input.device()), empty_vulkan({0}, at::kFloat, input.device())};
    }
    if (bn_channels_last(input) && input.numel()) {
        // channels-last in, channels-last out: no layout copies (the reference keeps the input's format too)
        const int64_t c = input.size(1), rows = input.numel() / c;
        const at::ScalarType st = input.scalar_type();
        at::Tensor w, b;
        if (weight.has_value() && weight->defined()) w = contiguous_vulkan(weight->to(st));
        if (bias.has_value() && bias->defined()) b = contiguous_vulkan(bias->to(st));
        at::Tensor y = at::empty_strided(input.sizes(), input.strides(), input.options());
        at::Tensor mean = empty_vulkan({c}, at::kFloat, input.device()), invstd = empty_vulkan({c}, at::kFloat, input.device());
        DeviceScope scope(input);
        uint64_t ws_bytes = 0;
        TVK_CALL(tvk_batchnorm_cl_workspace_size(rows, c, &ws_bytes));
        Workspace ws(scope.device, ws_bytes);
        const bool stats = running_mean && running_mean->defined() && running_var && running_var->defined();
        if (stats) TORCH_CHECK(running_mean->is_contiguous() && running_var->is_contiguous() && running_mean->scalar_type() == running_var->scalar_type(),
                               "torchvulkan [ERROR]: running statistics must be contiguous and of one dtype");
        TVK_CALL(tvk_batchnorm_forward_cl(to_tvk_dtype(st), y.data_ptr(), (float*)mean.data_ptr(), (float*)invstd.data_ptr(), input.data_ptr(),
                                          w.defined() ? w.data_ptr() : nullptr, b.defined() ? b.data_ptr() : nullptr,
                                          stats ? to_tvk_dtype(running_mean->scalar_type()) : TVK_F32, stats ? running_mean->data_ptr() : nullptr,
                                          stats ? running_var->data_ptr() : nullptr, rows, c, momentum, eps, ws.ptr, ws.bytes, scope.stream));
        return {y, mean, invstd};
    }
    at::Tensor x = contiguous_vulkan(input);
    const int64_t n = x.size(0), c = x.size(1), hw = (n * c) ? x.numel() / (n * c) : 0;
    const at::ScalarType st = input.scalar_type();
    at::Tensor w, b;
    if (weight.has_value() && weight->defined()) w = contiguous_vulkan(weight->to(st));
    if (bias.has_value() && bias->defined()) b = contiguous_vulkan(bias->to(st));
    at::Tensor y = empty_like_contig(x);
    at::Tensor mean = empty_vulkan({c}, at::kFloat, input.device()), invstd = empty_vulkan({c}, at::kFloat, input.device());
    if (x.numel()) {
        DeviceScope scope(input);
        uint64_t ws_bytes = 0;
        TVK_CALL(tvk_batchnorm_workspace_size(n, c, hw, &ws_bytes));
        Workspace ws(scope.device, ws_bytes);
        const bool stats = running_mean && running_mean->defined() && running_var && running_var->defined();
        if (stats) TORCH_CHECK(running_mean->is_contiguous() && running_var->is_contiguous() && running_mean->scalar_type() == running_var->scalar_type(),
                               "torchvulkan [ERROR]: running statistics must be contiguous and of one dtype");
        TVK_CALL(tvk_batchnorm_forward(to_tvk_dtype(st), y.data_ptr(), (float*)mean.data_ptr(), (float*)invstd.data_ptr(), x.data_ptr(),
                                       w.defined() ? w.data_ptr() : nullptr, b.defined() ? b.data_ptr() : nullptr,
                                       stats ? to_tvk_dtype(running_mean->scalar_type()) : TVK_F32, stats ? running_mean->data_ptr() : nullptr,
                                       stats ? running_var->data_ptr() : nullptr, n, c, hw, momentum, eps, ws.ptr, ws.bytes, scope.stream));
    }
    return {y, mean, invstd};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> native_batch_norm(const at::Tensor& input, const c10::optional<at::Tensor>& weight,
                                                                 const c10::optional<at::Tensor>& bias, const c10::optional<at::Tensor>& running_mean,
                                                                 const c10::optional<at::Tensor>& running_var, bool training, double momentum,
                                                                 double eps) {
    at::Tensor rm = running_mean.value_or(at::Tensor()), rv = running_var.value_or(at::Tensor());
    return batch_norm_train(input, weight, bias, &rm, &rv, training, momentum, eps);
}
std::tuple<at::Tensor, at::Tensor, at::Tensor> native_batch_norm_legit(const at::Tensor& input, const c10::optional<at::Tensor>& weight,
                                                                       const c10::optional<at::Tensor>& bias, at::Tensor& running_mean,
                                                                       at::Tensor& running_var, bool training, double momentum, double eps) {
    return batch_norm_train(input, weight, bias, &running_mean, &running_var, training, momentum, eps);
}
std::tuple<at::Tensor, at::Tensor, at::Tensor> native_batch_norm_legit_no_stats(const at::Tensor& input, const c10::optional<at::Tensor>& weight,
                                                                                const c10::optional<at::Tensor>& bias, bool training,
                                                                                double momentum, double eps) {
    return batch_norm_train(input, weight, bias, nullptr, nullptr, training, momentum, eps);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> native_batch_norm_backward(const at::Tensor& grad_out, const at::Tensor& input,
                                                                          const c10::optional<at::Tensor>& weight, const c10::optional<at::Tensor>& running_mean,
                                                                          const c10::optional<at::Tensor>& running_var, const c10::optional<at::Tensor>& save_mean,
                                                                          const c10::optional<at::Tensor>& save_invstd, bool train, double eps,
                                                                          std::array<bool, 3> output_mask) {
    require_float(input, "native_batch_norm_backward");
    if (!train) {
        // Evaluation mode (a frozen layer inside a model that is being trained): the statistics are constants, so
        // gx = g * w * invstd, gw = sum g * (x - mean) * invstd, gb = sum g, with invstd = rsqrt(running_var + eps).
        // A few elementwise and reduction launches on the device; not a hot path.
        TORCH_CHECK(running_mean.has_value() && running_mean->defined() && running_var.has_value() && running_var->defined(),
                    "torchvulkan [ERROR]: batch_norm backward in evaluation mode needs running_mean and running_var");
        const at::ScalarType st = input.scalar_type();
        std::vector<int64_t> bshape(input.dim(), 1), dims;
        bshape[1] = input.size(1);
        for (int64_t d = 0; d < input.dim(); ++d)
            if (d != 1) dims.push_back(d);
        at::Tensor invstd = at::rsqrt(running_var->to(at::kFloat) + eps), mean = running_mean->to(at::kFloat);
        at::Tensor g = grad_out.to(st);
        at::Tensor gx, gw, gb;
        if (output_mask[0]) {
            at::Tensor scale = (weight.has_value() && weight->defined()) ? weight->to(at::kFloat) * invstd : invstd;
            gx = g * scale.to(st).view(bshape);
        }
        if (output_mask[1]) gw = (g * ((input - mean.to(st).view(bshape)) * invstd.to(st).view(bshape))).sum(dims);
        if (output_mask[2]) gb = g.sum(dims);
        return {gx, gw, gb};
    }
    TORCH_CHECK(save_mean.has_value() && save_mean->defined() && save_invstd.has_value() && save_invstd->defined(),
                "torchvulkan [ERROR]: batch_norm backward needs the saved statistics");
    const at::ScalarType st = input.scalar_type();
    if (bn_channels_last(input) && input.numel()) {
        const int64_t c = input.size(1), rows = input.numel() / c;
        at::Tensor g = grad_out.to(st);
        if (!(g.strides() == input.strides() && (reinterpret_cast<uintptr_t>(g.data_ptr()) & 15) == 0)) g = g.contiguous(at::MemoryFormat::ChannelsLast);
        at::Tensor w;
        if (weight.has_value() && weight->defined()) w = contiguous_vulkan(weight->to(st));
        at::Tensor mean = contiguous_vulkan(save_mean->to(at::kFloat)), invstd = contiguous_vulkan(save_invstd->to(at::kFloat));
        at::Tensor gx, gw, gb;
        if (output_mask[0]) gx = at::empty_strided(input.sizes(), input.strides(), input.options());
        if (output_mask[1]) gw = empty_vulkan({c}, st, input.device());
        if (output_mask[2]) gb = empty_vulkan({c}, st, input.device());
        DeviceScope scope(input);
        uint64_t ws_bytes = 0;
        TVK_CALL(tvk_batchnorm_cl_workspace_size(rows, c, &ws_bytes));
        Workspace ws(scope.device, ws_bytes);
        TVK_CALL(tvk_batchnorm_backward_cl(to_tvk_dtype(st), gx.defined() ? gx.data_ptr() : nullptr, gw.defined() ? gw.data_ptr() : nullptr,
                                           gb.defined() ? gb.data_ptr() : nullptr, g.data_ptr(), input.data_ptr(), w.defined() ? w.data_ptr() : nullptr,
                                           (const float*)mean.data_ptr(), (const float*)invstd.data_ptr(), rows, c, ws.ptr, ws.bytes, scope.stream));
        return {gx, gw, gb};
    }
    at::Tensor x = contiguous_vulkan(input), g = contiguous_vulkan(grad_out.to(st));
    const int64_t n = x.size(0), c = x.size(1), hw = (n * c) ? x.numel() / (n * c) : 0;
    at::Tensor w;
    if (weight.has_value() && weight->defined()) w = contiguous_vulkan(weight->to(st));
    at::Tensor mean = contiguous_vulkan(save_mean->to(at::kFloat)), invstd = contiguous_vulkan(save_invstd->to(at::kFloat));
    at::Tensor gx, gw, gb;
    if (output_mask[0]) gx = empty_like_contig(x);
    if (output_mask[1]) gw = empty_vulkan({c}, st, input.device());
    if (output_mask[2]) gb = empty_vulkan({c}, st, input.device());
    if (x.numel()) {
        DeviceScope scope(input);
        uint64_t ws_bytes = 0;
        TVK_CALL(tvk_batchnorm_workspace_size(n, c, hw, &ws_bytes));
        Workspace ws(scope.device, ws_bytes);
        TVK_CALL(tvk_batchnorm_backward(to_tvk_dtype(st), gx.defined() ? gx.data_ptr() : nullptr, gw.defined() ? gw.data_ptr() : nullptr,
                                        gb.defined() ? gb.data_ptr() : nullptr, g.data_ptr(), x.data_ptr(), w.defined() ? w.data_ptr() : nullptr,
                                        (const float*)mean.data_ptr(), (const float*)invstd.data_ptr(), n, c, hw, ws.ptr, ws.bytes, scope.stream));
    }
    return {gx, gw, gb};
}

// ---- embedding --------------------------------------------------------------------------
at::Tensor embedding(const at::Tensor& weight, const at::Tensor& indices, c10::SymInt, bool, bool) {
    TORCH_CHECK(weight.dim() == 2, "'weight' must be 2-D");
    TORCH_CHECK(indices.scalar_type() == at::kLong || indices.scalar_type() == at::kInt, "Expected tensor for argument #1 'indices' to have one of the following scalar types: Long, Int");
    const int dt = to_tvk_dtype(weight.scalar_type());
    TORCH_CHECK(dt == TVK_F32 || dt == TVK_F16 || dt == TVK_BF16, "torchvulkan [NOT IMPLEMENTED]: embedding for dtype ", weight.scalar_type());
    at::Tensor table = contiguous_vulkan(weight), idx = contiguous_vulkan(indices.to(at::kLong));
    std::vector<int64_t> shape(idx.sizes().begin(), idx.sizes().end());
    shape.push_back(table.size(1));
    at::Tensor out = empty_vulkan(shape, weight.scalar_type(), weight.device());
    if (out.numel()) {
        DeviceScope scope(weight);
        TVK_CALL(tvk_embedding_forward(dt, out.data_ptr(), table.data_ptr(), (const int64_t*)idx.data_ptr(), idx.numel(), table.size(0), table.size(1),
                                       scope.stream));
    }
    return out;
}

at::Tensor embedding_dense_backward(const at::Tensor& grad_output, const at::Tensor& indices, c10::SymInt num_weights, c10::SymInt padding_idx,
                                    bool scale_grad_by_freq) {
    require_float(grad_output, "embedding_dense_backward");
    if (scale_grad_by_freq) TVK_NOT_IMPLEMENTED("embedding backward with scale_grad_by_freq");
    at::Tensor idx = contiguous_vulkan(indices.to(at::kLong));
    const int64_t dim = grad_output.size(-1);
    at::Tensor g = contiguous_vulkan(grad_output).reshape({-1, dim});
    const int64_t rows = num_weights.guard_int(__FILE__, __LINE__);
    at::Tensor out = empty_vulkan({rows, dim}, grad_output.scalar_type(), grad_output.device());
    if (out.numel()) {
        DeviceScope scope(grad_output);
        TVK_CALL(tvk_embedding_backward(to_tvk_dtype(grad_output.scalar_type()), out.data_ptr(), g.data_ptr(), (const int64_t*)idx.data_ptr(), idx.numel(),
                                        rows, dim, padding_idx.guard_int(__FILE__, __LINE__), scope.stream));
    }
    return out;
}

// ---- cat --------------------------------------------------------------------------------
at::Tensor cat(const at::ITensorListRef& tensors, int64_t dim) {
    std::vector<at::Tensor> ts;
    for (const at::Tensor& t : tensors)
        if (!(t.dim() == 1 && t.numel() == 0)) ts.push_back(t);   // legacy: empty 1-D tensors are skipped
    TORCH_CHECK(!ts.empty() || tensors.size() > 0, "torch.cat(): expected a non-empty list of Tensors");
    if (ts.empty()) return at::empty({0}, tensors.front().options());
    at::ScalarType st = ts[0].scalar_type();
    for (auto& t : ts) st = c10::promoteTypes(st, t.scalar_type());
    const int64_t nd = ts[0].dim();
    dim = at::maybe_wrap_dim(dim, nd);
    std::vector<int64_t> shape(ts[0].sizes().begin(), ts[0].sizes().end());
    int64_t total = 0;
    for (auto& t : ts) {
        TORCH_CHECK(t.dim() == nd, "Tensors must have same number of dimensions: got ", nd, " and ", t.dim());
        for (int64_t d = 0; d < nd; ++d)
            TORCH_CHECK(d == dim || t.size(d) == shape[d], "Sizes of tensors must match except in dimension ", dim, ". Expected size ", shape[d],
                        " but got size ", t.size(d), " for tensor in the list.");
        total += t.size(dim);
    }
    shape[dim] = total;
    at::Tensor out = empty_vulkan(shape, st, ts[0].device());
    int64_t off = 0;
    for (auto& t : ts) {
        if (t.size(dim) == 0) continue;
        out.narrow(dim, off, t.size(dim)).copy_(t);   // one strided-copy launch per input
        off += t.size(dim);
    }
    return out;
}
at::Tensor& cat_out(const at::ITensorListRef& tensors, int64_t dim, at::Tensor& out) { return copy_into(out, (cat)(tensors, dim)); }

// ---- optimizers -------------------------------------------------------------------------
// torch.amp.GradScaler hands fused optimizers its state instead of stepping around them: found_inf (skip the whole step when
// it is set) and, when unscale_() was not called first, grad_scale (the gradients are divided by it in place, as ATen's CUDA
// kernels do). The skip decision is read back - one synchronisation per step, where the unfused path has one as well.
// Returns false when the step is to be skipped.
bool apply_grad_scaler(at::TensorList grads, const c10::optional<at::Tensor>& grad_scale, const c10::optional<at::Tensor>& found_inf) {
    if (found_inf.has_value() && found_inf->defined() && found_inf->item<float>() != 0.f) return false;
    if (grad_scale.has_value() && grad_scale->defined()) {
        for (const at::Tensor& g : grads) {
            if (!g.defined() || g.numel() == 0) continue;
            at::Tensor gm = g;
            gm.div_(grad_scale->to(g.scalar_type()).reshape({}));
        }
    }
    return true;
}
double host_scalar(const at::Tensor& t) { return t.item<double>(); }  // CPU step counters cost nothing; device ones sync

void fused_adam_impl(at::TensorList params, at::TensorList grads, at::TensorList exp_avgs, at::TensorList exp_avg_sqs, at::TensorList max_exp_avg_sqs,
                     at::TensorList state_steps, double lr, double beta1, double beta2, double weight_decay, double eps, bool amsgrad, bool maximize,
                     const c10::optional<at::Tensor>& grad_scale, const c10::optional<at::Tensor>& found_inf, bool decoupled) {
    const size_t n = params.size();
    TORCH_CHECK(grads.size() == n && exp_avgs.size() == n && exp_avg_sqs.size() == n && state_steps.size() == n, "torchvulkan [ERROR]: fused adam: list sizes differ");
    if (amsgrad) TVK_NOT_IMPLEMENTED("fused Adam with amsgrad");
    (void)max_exp_avg_sqs;
    if (!apply_grad_scaler(grads, grad_scale, found_inf)) return;
    // One list launch per (device, dtype) run of the list. Step counters that live on the device (fp32 scalars, as
    // torch.optim creates them for fused optimizers) are read by the kernel; host counters are read here.
    std::vector<tvk_multi_item> items;
    size_t i = 0;
    while (i < n) {
        const at::Tensor& first = params[i];
        items.clear();
        int64_t host_step = 0;
        size_t j = i;
        for (; j < n; ++j) {
            const at::Tensor& p = params[j];
            if (p.scalar_type() != first.scalar_type() || p.device() != first.device()) break;
            if (p.numel() == 0) continue;
            require_float(p, "_fused_adam");
            TORCH_CHECK(p.is_non_overlapping_and_dense() && same_layout(grads[j], p) && same_layout(exp_avgs[j], p) && same_layout(exp_avg_sqs[j], p),
                        "torchvulkan [ERROR]: fused adam expects dense tensors with matching layouts");
            TORCH_CHECK(grads[j].scalar_type() == p.scalar_type() && exp_avgs[j].scalar_type() == p.scalar_type() && exp_avg_sqs[j].scalar_type() == p.scalar_type(),
                        "torchvulkan [ERROR]: fused adam expects one dtype per parameter group entry");
            const at::Tensor& st = state_steps[j];
            tvk_multi_item it = {{p.data_ptr(), grads[j].data_ptr(), exp_avgs[j].data_ptr(), exp_avg_sqs[j].data_ptr()}, p.numel(), nullptr};
            if (is_vulkan(st) && st.scalar_type() == at::kFloat && st.device() == p.device()) {
                it.step = (const float*)st.data_ptr();
            } else {
                const int64_t hs = (int64_t)host_scalar(st);
                if (host_step != 0 && hs != host_step) break;   // a different host step: next launch
                host_step = hs;
            }
            items.push_back(it);
        }
        if (!items.empty()) {
            DeviceScope scope(first);
            TVK_CALL(tvk_adam_step_multi(to_tvk_dtype(first.scalar_type()), items.data(), (int)items.size(), lr, beta1, beta2, eps, weight_decay, host_step,
                                         decoupled ? 1 : 0, maximize ? 1 : 0, scope.stream));
        }
        TORCH_CHECK(j > i, "torchvulkan [ERROR]: fused adam made no progress over the parameter list");
        i = j;
    }
}

// torch.optim advances the step tensors (_foreach_add_) before it calls the fused op, so the values
// read here are the 1-based step counts, as in the reference (optim.cpp:88-126).
void fused_adamw_(at::TensorList p, at::TensorList g, at::TensorList m, at::TensorList v, at::TensorList mx, at::TensorList steps, double lr,
                  double b1, double b2, double wd, double eps, bool amsgrad, bool maximize, const c10::optional<at::Tensor>& gs,
                  const c10::optional<at::Tensor>& fi) {
    fused_adam_impl(p, g, m, v, mx, steps, lr, b1, b2, wd, eps, amsgrad, maximize, gs, fi, true);
}
void fused_adamw_tensor_lr_(at::TensorList p, at::TensorList g, at::TensorList m, at::TensorList v, at::TensorList mx, at::TensorList steps,
                            const at::Tensor& lr, double b1, double b2, double wd, double eps, bool amsgrad, bool maximize,
                            const c10::optional<at::Tensor>& gs, const c10::optional<at::Tensor>& fi) {
    fused_adam_impl(p, g, m, v, mx, steps, host_scalar(lr), b1, b2, wd, eps, amsgrad, maximize, gs, fi, true);
}
void fused_adam_(at::TensorList p, at::TensorList g, at::TensorList m, at::TensorList v, at::TensorList mx, at::TensorList steps, double lr,
                 double b1, double b2, double wd, double eps, bool amsgrad, bool maximize, const c10::optional<at::Tensor>& gs,
                 const c10::optional<at::Tensor>& fi) {
    fused_adam_impl(p, g, m, v, mx, steps, lr, b1, b2, wd, eps, amsgrad, maximize, gs, fi, false);
}

void fused_sgd_(at::TensorList params, at::TensorList grads, at::TensorList bufs, double weight_decay, double momentum, double lr, double dampening,
                bool nesterov, bool maximize, bool is_first_step, const c10::optional<at::Tensor>& grad_scale, const c10::optional<at::Tensor>& found_inf) {
    const size_t n = params.size();
    TORCH_CHECK(grads.size() == n, "torchvulkan [ERROR]: fused sgd: list sizes differ");
    const bool has_momentum = momentum != 0.0;
    TORCH_CHECK(has_momentum ? bufs.size() == n : bufs.empty(), "torchvulkan [ERROR]: fused sgd: momentum buffer list size");
    if (!apply_grad_scaler(grads, grad_scale, found_inf)) return;
    std::vector<tvk_multi_item> items;
    size_t i = 0;
    while (i < n) {
        const at::Tensor& first = params[i];
        items.clear();
        size_t j = i;
        for (; j < n; ++j) {
            const at::Tensor& p = params[j];
            if (p.scalar_type() != first.scalar_type() || p.device() != first.device()) break;
            if (p.numel() == 0) continue;
            require_float(p, "_fused_sgd");
            TORCH_CHECK(p.is_non_overlapping_and_dense() && same_layout(grads[j], p) && grads[j].scalar_type() == p.scalar_type(),
                        "torchvulkan [ERROR]: fused sgd expects dense tensors with matching layouts and dtypes");
            if (has_momentum)
                TORCH_CHECK(same_layout(bufs[j], p) && bufs[j].scalar_type() == p.scalar_type(),
                            "torchvulkan [ERROR]: fused sgd expects momentum buffers laid out like their parameters");
            items.push_back({{p.data_ptr(), grads[j].data_ptr(), has_momentum ? bufs[j].data_ptr() : nullptr, nullptr}, p.numel(), nullptr});
        }
        if (!items.empty()) {
            DeviceScope scope(first);
            TVK_CALL(tvk_sgd_step_multi(to_tvk_dtype(first.scalar_type()), items.data(), (int)items.size(), lr, momentum, dampening, weight_decay,
                                        nesterov ? 1 : 0, maximize ? 1 : 0, is_first_step ? 1 : 0, scope.stream));
        }
        i = j > i ? j : i + 1;
    }
}

// ---- foreach list updates used by torch.optim's default (foreach) implementations --------------------
// a[i] = scale_a * a[i] + scale_b * b[i] + add for every tensor of the list; tensors the list kernel cannot take
// (another dtype, not dense, mismatched layouts) go through the single-tensor ops.
template <typename Fallback>
void foreach_axpby(at::TensorList as, const at::TensorList* bs, double scale_a, double scale_b, double add, Fallback&& single) {
    if (bs) TORCH_CHECK(bs->size() == as.size(), "torchvulkan [ERROR]: foreach: tensor lists must have the same length");
    std::vector<tvk_multi_item> items;
    size_t i = 0;
    while (i < as.size()) {
        const at::Tensor& first = as[i];
        items.clear();
        size_t j = i;
        for (; j < as.size(); ++j) {
            const at::Tensor& a = as[j];
            if (a.scalar_type() != first.scalar_type() || a.device() != first.device()) break;
            const bool ok = is_vulkan(a) && is_hot_float(a.scalar_type()) && a.is_non_overlapping_and_dense() &&
                            (!bs || (is_vulkan((*bs)[j]) && (*bs)[j].scalar_type() == a.scalar_type() && same_layout((*bs)[j], a)));
            if (!ok) { single(j); continue; }
            if (a.numel() == 0) continue;
            items.push_back({{a.data_ptr(), bs ? (*bs)[j].data_ptr() : nullptr, nullptr, nullptr}, a.numel(), nullptr});
        }
        if (!items.empty()) {
            DeviceScope scope(first);
            TVK_CALL(tvk_foreach_axpby(to_tvk_dtype(first.scalar_type()), items.data(), (int)items.size(), scale_a, scale_b, add, bs ? 1 : 0, scope.stream));
        }
        i = j > i ? j : i + 1;
    }
}
void foreach_add_scalar_(at::TensorList self, const at::Scalar& s) {
    foreach_axpby(self, nullptr, 1.0, 0.0, s.toDouble(), [&](size_t k) { const_cast<at::Tensor&>(self[k]).add_(s); });
}
void foreach_mul_scalar_(at::TensorList self, const at::Scalar& s) {
    foreach_axpby(self, nullptr, s.toDouble(), 0.0, 0.0, [&](size_t k) { const_cast<at::Tensor&>(self[k]).mul_(s); });
}
void foreach_add_list_(at::TensorList self, at::TensorList other, const at::Scalar& alpha) {
    foreach_axpby(self, &other, 1.0, alpha.toDouble(), 0.0, [&](size_t k) { const_cast<at::Tensor&>(self[k]).add_(other[k], alpha); });
}
void fused_sgd_tensor_lr_(at::TensorList p, at::TensorList g, at::TensorList b, double wd, double mom, const at::Tensor& lr, double damp, bool nesterov,
                          bool maximize, bool first, const c10::optional<at::Tensor>& gs, const c10::optional<at::Tensor>& fi) {
    fused_sgd_(p, g, b, wd, mom, host_scalar(lr), damp, nesterov, maximize, first, gs, fi);
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("_log_softmax", &log_softmax);
    m.impl("_log_softmax.out", &log_softmax_out);
    m.impl("_softmax", &softmax);
    m.impl("_softmax.out", &softmax_out);
    m.impl("_log_softmax_backward_data", &log_softmax_bwd);
    m.impl("_log_softmax_backward_data.out", &log_softmax_bwd_out);
    m.impl("_softmax_backward_data", &softmax_bwd);
    m.impl("_softmax_backward_data.out", &softmax_bwd_out);
    m.impl("nll_loss_forward", &nll_loss_forward);
    m.impl("nll_loss_backward", &nll_loss_backward);
    m.impl("_fused_rms_norm", &fused_rms_norm);
    m.impl("_fused_rms_norm_backward", &fused_rms_norm_backward);
    m.impl("native_batch_norm", &native_batch_norm);
    m.impl("_native_batch_norm_legit", &native_batch_norm_legit);
    m.impl("_native_batch_norm_legit.no_stats", &native_batch_norm_legit_no_stats);
    m.impl("native_batch_norm_backward", &native_batch_norm_backward);
    m.impl("embedding", &embedding);
    m.impl("embedding_dense_backward", &embedding_dense_backward);
    m.impl("cat", &cat);
    m.impl("cat.out", &cat_out);
    m.impl("_fused_adamw_", &fused_adamw_);
    m.impl("_fused_adamw_.tensor_lr", &fused_adamw_tensor_lr_);
    m.impl("_fused_adam_", &fused_adam_);
    m.impl("_fused_sgd_", &fused_sgd_);
    m.impl("_foreach_add_.Scalar", &foreach_add_scalar_);
    m.impl("_foreach_mul_.Scalar", &foreach_mul_scalar_);
    m.impl("_foreach_add_.List", &foreach_add_list_);
    m.impl("_fused_sgd_.tensor_lr", &fused_sgd_tensor_lr_);
}

}  // namespace tvk_aten
