// conv2d on the "vulkan" device: convolution_overrideable and convolution_backward_overrideable.
//
// Counterparts in the reference: convolution_vulkan / convolution_backward_vulkan
// (src/api/ops/conv.cpp:1088-1172, registered at conv.cpp:1303-1304). at::convolution routes every
// PrivateUse1 convolution to these two ops. As there, the bias is a broadcast add after the kernel and
// its gradient a sum over (n, h, w) (conv.cpp:1159-1170). 2-D, groups 1, dilation 1, stride 1 or 2,
// fp16 / bf16 are built; the rest raises "[NOT IMPLEMENTED]" (the hot path never falls back to the CPU).
#include "common.h"

namespace tvk_aten {
namespace {

tvk_conv2d_desc make_desc(const at::Tensor& input, const at::Tensor& weight, at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation,
                          bool transposed, int64_t groups) {
    TORCH_CHECK(input.dim() == 4 && weight.dim() == 4, "torchvulkan [NOT IMPLEMENTED]: convolution of ", input.dim() - 2,
                " spatial dimensions (2-D convolution is supported)");
    TORCH_CHECK(!transposed, "torchvulkan [NOT IMPLEMENTED]: transposed convolution");
    TORCH_CHECK(input.scalar_type() == weight.scalar_type(), "torchvulkan [ERROR]: convolution: input is ", input.scalar_type(), " but weight is ",
                weight.scalar_type());
    TORCH_CHECK(input.size(1) == weight.size(1) * groups, "torchvulkan [ERROR]: convolution: input has ", input.size(1), " channels, weight expects ",
                weight.size(1) * groups);
    auto at_or = [](at::IntArrayRef v, size_t i, int64_t dflt) { return v.empty() ? dflt : (v.size() == 1 ? v[0] : v[i]); };
    tvk_conv2d_desc d;
    d.dtype = to_tvk_dtype(input.scalar_type());
    d.n = input.size(0); d.cin = input.size(1); d.h = input.size(2); d.w = input.size(3);
    d.cout = weight.size(0); d.kh = weight.size(2); d.kw = weight.size(3);
    d.stride_h = at_or(stride, 0, 1); d.stride_w = at_or(stride, 1, 1);
    d.pad_h = at_or(padding, 0, 0); d.pad_w = at_or(padding, 1, 0);
    d.dilation_h = at_or(dilation, 0, 1); d.dilation_w = at_or(dilation, 1, 1);
    d.groups = groups;
    d.layout = 0;
    return d;
}

// Plain-contiguous or channels-last storage is passed to the kernels as it is; anything else is made contiguous first.
bool is_channels_last(const at::Tensor& t) { return t.dim() == 4 && !t.is_contiguous() && t.is_contiguous(at::MemoryFormat::ChannelsLast); }
at::Tensor dense4(const at::Tensor& t) { return is_channels_last(t) ? t : contiguous_vulkan(t); }
at::Tensor empty4(at::IntArrayRef sizes, const at::Tensor& like, bool channels_last) {
    if (!channels_last) return empty_vulkan(sizes, like.scalar_type(), like.device());
    return at::empty_strided(sizes, at::get_channels_last_strides_2d(sizes), like.options());
}

at::Tensor convolution(const at::Tensor& input, const at::Tensor& weight, const c10::optional<at::Tensor>& bias, at::IntArrayRef stride,
                       at::IntArrayRef padding, at::IntArrayRef dilation, bool transposed, at::IntArrayRef /*output_padding*/, int64_t groups) {
    tvk_conv2d_desc d = make_desc(input, weight, stride, padding, dilation, transposed, groups);
    at::Tensor x = dense4(input), w = dense4(weight);
    // the output follows the input's memory format (conv.cpp:1080-1086): channels-last in, channels-last out
    const bool cl = is_channels_last(x);
    d.layout = (cl ? (TVK_CONV_X_CHANNELS_LAST | TVK_CONV_Y_CHANNELS_LAST) : 0) | (is_channels_last(w) ? TVK_CONV_W_CHANNELS_LAST : 0);
    DeviceScope scope(x);
    uint64_t ws_bytes = 0;
    TVK_CALL(tvk_conv2d_workspace_size(&d, 0, &ws_bytes));
    const int64_t ho = (d.h + 2 * d.pad_h - d.kh) / d.stride_h + 1, wo = (d.w + 2 * d.pad_w - d.kw) / d.stride_w + 1;
    at::Tensor y = empty4({d.n, d.cout, ho, wo}, x, cl);
    if (y.numel()) {
        Workspace ws(scope.device, ws_bytes);
        TVK_CALL(tvk_conv2d_forward(&d, y.data_ptr(), x.data_ptr(), w.data_ptr(), ws.ptr, ws.bytes, scope.stream));
    }
    if (bias.has_value() && bias->defined()) y.add_(bias->view({1, -1, 1, 1}));
    return y;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> convolution_backward(const at::Tensor& grad_output, const at::Tensor& input, const at::Tensor& weight,
                                                                    at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation,
                                                                    bool transposed, at::IntArrayRef /*output_padding*/, int64_t groups,
                                                                    std::array<bool, 3> output_mask) {
    tvk_conv2d_desc d = make_desc(input, weight, stride, padding, dilation, transposed, groups);
    at::Tensor gy = dense4(grad_output);
    at::Tensor xin = dense4(input);
    const bool x_cl = is_channels_last(xin), y_cl = is_channels_last(gy), w_cl = is_channels_last(weight);
    TORCH_CHECK(gy.scalar_type() == input.scalar_type(), "torchvulkan [ERROR]: convolution backward: grad_output is ", gy.scalar_type(), " but input is ",
                input.scalar_type());
    DeviceScope scope(gy);
    at::Tensor gx, gw, gb;
    if (output_mask[0] || output_mask[1]) {
        at::Tensor w = dense4(weight);
        // dx follows x, dw follows w (whose layout the kernels read as it is)
        if (output_mask[0]) gx = empty4(input.sizes(), input, x_cl);
        if (output_mask[1]) gw = empty4(weight.sizes(), weight, w_cl);
        d.layout = (x_cl ? TVK_CONV_X_CHANNELS_LAST : 0) | (y_cl ? TVK_CONV_Y_CHANNELS_LAST : 0) | (is_channels_last(w) ? TVK_CONV_W_CHANNELS_LAST : 0);
        const bool want_gx = output_mask[0] && gx.numel() > 0;
        if (want_gx || output_mask[1]) {
            uint64_t ws_bytes = 0;
            TVK_CALL(tvk_conv2d_workspace_size(&d, 3, &ws_bytes));
            Workspace ws(scope.device, ws_bytes);
            TVK_CALL(tvk_conv2d_backward(&d, want_gx ? gx.data_ptr() : nullptr, output_mask[1] ? gw.data_ptr() : nullptr, gy.data_ptr(), xin.data_ptr(),
                                         w.data_ptr(), ws.ptr, ws.bytes, scope.stream));
        }
    }
    if (output_mask[2]) gb = gy.sum(at::IntArrayRef({0, 2, 3}));
    return std::make_tuple(gx, gw, gb);
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("convolution_overrideable", &convolution);
    m.impl("convolution_backward_overrideable", &convolution_backward);
}

}  // namespace tvk_aten
