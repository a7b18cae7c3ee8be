// conv2d on the "vulkan" device: convolution_overrideable and convolution_backward_overrideable.
//
// Counterparts in the reference: convolution_vulkan / convolution_backward_vulkan
// (src/api/ops/conv.cpp:1088-1172, registered at conv.cpp:1303-1304). at::convolution routes every
// PrivateUse1 convolution to these two ops. As there, the bias is a broadcast add after the kernel and
// its gradient a sum over (n, h, w) (conv.cpp:1159-1170). The implicit-GEMM kernels cover 2-D, groups 1, dilation 1,
// stride 1 or 2 in fp16 / bf16; fp32 and every other 2-D geometry go through unfold + GEMM inside the same C entry
// points. Around them, as in the reference's one entry for every flavour (conv.cpp:1088-1172, 1196-1294):
//   * 1-D convolutions run as 2-D ones of height 1;
//   * a transposed convolution is the input-gradient product of the forward one (its gradients are the forward
//     product and the weight-gradient product with the roles of input and output swapped);
//   * depthwise convolutions (one input channel per group) take the direct kernels of depthwise.cu;
//   * other grouped convolutions run group by group on channel slices.
//   * a 3-D convolution (transposed or not) is one 2-D convolution per depth tap over the batch n * depths, accumulated.
// What the kernels refuse raises "[NOT IMPLEMENTED]" (the hot path never falls back to the CPU).
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

at::Tensor conv2d_dense(const at::Tensor& input, const at::Tensor& weight, const c10::optional<at::Tensor>& bias, at::IntArrayRef stride,
                        at::IntArrayRef padding, at::IntArrayRef dilation, bool transposed, int64_t groups) {
    tvk_conv2d_desc d = make_desc(input, weight, stride, padding, dilation, transposed, groups);
    at::Tensor x = dense4(input), w = dense4(weight);
    // the output follows the input's memory format (conv.cpp:1080-1086): channels-last in, channels-last out
    const bool cl = is_channels_last(x);
    d.layout = (cl ? (TVK_CONV_X_CHANNELS_LAST | TVK_CONV_Y_CHANNELS_LAST) : 0) | (is_channels_last(w) ? TVK_CONV_W_CHANNELS_LAST : 0);
    DeviceScope scope(x);
    uint64_t ws_bytes = 0;
    TVK_CALL(tvk_conv2d_workspace_size(&d, 0, &ws_bytes));
    const int64_t ho = (d.h + 2 * d.pad_h - d.dilation_h * (d.kh - 1) - 1) / d.stride_h + 1, wo = (d.w + 2 * d.pad_w - d.dilation_w * (d.kw - 1) - 1) / d.stride_w + 1;
    TORCH_CHECK(ho > 0 && wo > 0, "torchvulkan [ERROR]: convolution: the filter does not fit the padded input");
    at::Tensor y = empty4({d.n, d.cout, ho, wo}, x, cl);
    if (y.numel()) {
        Workspace ws(scope.device, ws_bytes);
        TVK_CALL(tvk_conv2d_forward(&d, y.data_ptr(), x.data_ptr(), w.data_ptr(), ws.ptr, ws.bytes, scope.stream));
    }
    if (bias.has_value() && bias->defined()) y.add_(bias->view({1, -1, 1, 1}));
    return y;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> conv2d_dense_backward(const at::Tensor& grad_output, const at::Tensor& input, const at::Tensor& weight,
                                                                     at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation,
                                                                     bool transposed, int64_t groups, std::array<bool, 3> output_mask) {
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

using Vec2 = std::array<int64_t, 2>;
Vec2 pair_of(at::IntArrayRef v, int64_t dflt) {
    if (v.empty()) return {dflt, dflt};
    return v.size() == 1 ? Vec2{v[0], v[0]} : Vec2{v[0], v[1]};
}

// A convolution over an axis of extent 1 with a 1-tap filter and no padding does not depend on that axis' stride: ATen hands
// 1-D convolutions over as 2-D ones of height 1 with stride (1, s), and the tensor-core kernels want equal strides.
Vec2 effective_stride(const at::Tensor& input, const at::Tensor& weight, Vec2 st, Vec2 pd, Vec2 op) {
    if (input.size(2) == 1 && weight.size(2) == 1 && pd[0] == 0 && op[0] == 0) st[0] = st[1];
    else if (input.size(3) == 1 && weight.size(3) == 1 && pd[1] == 0 && op[1] == 0) st[1] = st[0];
    return st;
}

bool is_depthwise(const at::Tensor& input, const at::Tensor& weight, int64_t groups) {
    return groups > 1 && groups == input.size(1) && weight.size(1) == 1 && weight.size(0) % groups == 0;
}

tvk_conv2d_desc depthwise_desc(const at::Tensor& x, const at::Tensor& w, Vec2 st, Vec2 pd, Vec2 dl) {
    tvk_conv2d_desc d;
    d.dtype = to_tvk_dtype(x.scalar_type());
    d.n = x.size(0); d.cin = x.size(1); d.h = x.size(2); d.w = x.size(3);
    d.cout = w.size(0); d.kh = w.size(2); d.kw = w.size(3);
    d.stride_h = st[0]; d.stride_w = st[1]; d.pad_h = pd[0]; d.pad_w = pd[1]; d.dilation_h = dl[0]; d.dilation_w = dl[1];
    d.groups = x.size(1);
    d.layout = 0;
    return d;
}

// ---- 2-D convolution with groups (transposed == false) --------------------------------------------------------------
at::Tensor conv2d_any(const at::Tensor& input, const at::Tensor& weight, Vec2 st, Vec2 pd, Vec2 dl, int64_t groups) {
    TORCH_CHECK(groups >= 1 && input.size(1) % groups == 0 && weight.size(0) % groups == 0 && input.size(1) / groups == weight.size(1),
                "torchvulkan [ERROR]: convolution: input of ", input.size(1), " channels and weight ", weight.sizes(), " do not fit groups = ", groups);
    if (groups == 1) return conv2d_dense(input, weight, c10::nullopt, {st[0], st[1]}, {pd[0], pd[1]}, {dl[0], dl[1]}, false, 1);
    TORCH_CHECK(is_hot_float(input.scalar_type()) && input.scalar_type() == weight.scalar_type(), "torchvulkan [NOT IMPLEMENTED]: grouped convolution of ",
                input.scalar_type(), " with ", weight.scalar_type());
    if (is_depthwise(input, weight, groups)) {
        at::Tensor x = contiguous_vulkan(input), w = contiguous_vulkan(weight);
        tvk_conv2d_desc d = depthwise_desc(x, w, st, pd, dl);
        const int64_t ho = (d.h + 2 * d.pad_h - d.dilation_h * (d.kh - 1) - 1) / d.stride_h + 1, wo = (d.w + 2 * d.pad_w - d.dilation_w * (d.kw - 1) - 1) / d.stride_w + 1;
        TORCH_CHECK(ho > 0 && wo > 0, "torchvulkan [ERROR]: convolution: the filter does not fit the padded input");
        DeviceScope scope(x);
        at::Tensor y = empty_vulkan({d.n, d.cout, ho, wo}, x.scalar_type(), x.device());
        TVK_CALL(tvk_depthwise_conv2d_forward(&d, y.data_ptr(), x.data_ptr(), w.data_ptr(), scope.stream));
        return y;
    }
    // group by group on channel slices (each slice is made contiguous for the kernels)
    const int64_t cig = input.size(1) / groups, cog = weight.size(0) / groups;
    std::vector<at::Tensor> ys;
    ys.reserve(groups);
    for (int64_t g = 0; g < groups; ++g)
        ys.push_back(conv2d_dense(contiguous_vulkan(input.narrow(1, g * cig, cig)), weight.narrow(0, g * cog, cog), c10::nullopt, {st[0], st[1]}, {pd[0], pd[1]},
                                  {dl[0], dl[1]}, false, 1));
    return at::cat(ys, 1);
}

// gradients of conv2d_any; mask: {input, weight}
std::tuple<at::Tensor, at::Tensor> conv2d_any_backward(const at::Tensor& gy_in, const at::Tensor& input, const at::Tensor& weight, Vec2 st, Vec2 pd, Vec2 dl,
                                                        int64_t groups, bool need_gx, bool need_gw) {
    if (groups == 1) {
        auto r = conv2d_dense_backward(gy_in, input, weight, {st[0], st[1]}, {pd[0], pd[1]}, {dl[0], dl[1]}, false, 1, {need_gx, need_gw, false});
        return {std::get<0>(r), std::get<1>(r)};
    }
    at::Tensor gx, gw;
    if (is_depthwise(input, weight, groups)) {
        at::Tensor x = contiguous_vulkan(input), w = contiguous_vulkan(weight), gy = contiguous_vulkan(gy_in);
        tvk_conv2d_desc d = depthwise_desc(x, w, st, pd, dl);
        DeviceScope scope(x);
        if (need_gx) {
            gx = empty_vulkan(x.sizes(), x.scalar_type(), x.device());
            TVK_CALL(tvk_depthwise_conv2d_backward_input(&d, gx.data_ptr(), gy.data_ptr(), w.data_ptr(), scope.stream));
        }
        if (need_gw) {
            gw = empty_vulkan(w.sizes(), w.scalar_type(), w.device());
            TVK_CALL(tvk_depthwise_conv2d_backward_weight(&d, gw.data_ptr(), gy.data_ptr(), x.data_ptr(), scope.stream));
        }
        return {gx, gw};
    }
    const int64_t cig = input.size(1) / groups, cog = weight.size(0) / groups;
    std::vector<at::Tensor> gxs, gws;
    for (int64_t g = 0; g < groups; ++g) {
        auto r = conv2d_dense_backward(contiguous_vulkan(gy_in.narrow(1, g * cog, cog)), contiguous_vulkan(input.narrow(1, g * cig, cig)), weight.narrow(0, g * cog, cog),
                                       {st[0], st[1]}, {pd[0], pd[1]}, {dl[0], dl[1]}, false, 1, {need_gx, need_gw, false});
        if (need_gx) gxs.push_back(std::get<0>(r));
        if (need_gw) gws.push_back(std::get<1>(r));
    }
    if (need_gx) gx = at::cat(gxs, 1);
    if (need_gw) gw = at::cat(gws, 0);
    return {gx, gw};
}

// ---- transposed 2-D convolution: weight [cin, cout / groups, kh, kw] -------------------------------------------------
// y = conv_transpose(x, w) is the input gradient of the forward convolution z -> conv(z, w) taken at dy = x; so its own
// gradients are: grad_x = conv(grad_y, w), grad_w = weight gradient with (dy, x) = (x, grad_y).
Vec2 transposed_out(const at::Tensor& x, const at::Tensor& w, Vec2 st, Vec2 pd, Vec2 dl, Vec2 op) {
    return {(x.size(2) - 1) * st[0] - 2 * pd[0] + dl[0] * (w.size(2) - 1) + op[0] + 1, (x.size(3) - 1) * st[1] - 2 * pd[1] + dl[1] * (w.size(3) - 1) + op[1] + 1};
}

at::Tensor conv_transpose2d_any(const at::Tensor& input, const at::Tensor& weight, Vec2 st, Vec2 pd, Vec2 dl, Vec2 op, int64_t groups) {
    TORCH_CHECK(input.size(1) == weight.size(0), "torchvulkan [ERROR]: transposed convolution: input has ", input.size(1), " channels, weight expects ", weight.size(0));
    const Vec2 out = transposed_out(input, weight, st, pd, dl, op);
    TORCH_CHECK(out[0] > 0 && out[1] > 0, "torchvulkan [ERROR]: transposed convolution: empty output");
    // the forward convolution this one is the gradient of maps [n, cout, out] -> [n, cin, in]
    at::Tensor like = empty_vulkan({input.size(0), weight.size(1) * groups, out[0], out[1]}, input.scalar_type(), input.device());
    // (only the shape of `like` is used: the input-gradient product reads dy and w)
    return std::get<0>(conv2d_any_backward(input, like, weight, st, pd, dl, groups, true, false));
}

// ---- 3-D convolution: one 2-D convolution per depth tap -------------------------------------------------------------
// y[:, :, do] = sum over kd of conv2d(x[:, :, do * sd - pd + kd * dd], w[:, :, kd]). For one kd the valid output depths
// form a range and their input depths a strided slice, so each tap is ONE 2-D convolution over the batch n * depths
// (the tensor-core kernels see a large batch), accumulated into the output slice.
struct DepthTap {
    int64_t do0, count, d0;      // output depths do0 .. do0 + count, reading input depths d0 + i * sd
};
DepthTap depth_tap(int64_t D, int64_t Do, int64_t kd, int64_t sd, int64_t pd, int64_t dd) {
    // smallest / largest do with 0 <= do * sd - pd + kd * dd < D
    const int64_t off = kd * dd - pd;
    int64_t lo = off >= 0 ? 0 : (-off + sd - 1) / sd;
    int64_t hi = (D - 1 - off) >= 0 ? (D - 1 - off) / sd : -1;
    if (hi > Do - 1) hi = Do - 1;
    DepthTap t{lo, hi >= lo ? hi - lo + 1 : 0, lo * sd + off};
    return t;
}
// [n, c, depths, h, w] slice -> contiguous [n * depths, c, h, w]
at::Tensor fold_depth(const at::Tensor& t5) { return contiguous_vulkan(t5.permute({0, 2, 1, 3, 4})).view({t5.size(0) * t5.size(2), t5.size(1), t5.size(3), t5.size(4)}); }
at::Tensor unfold_depth(const at::Tensor& t4, int64_t n) { return t4.view({n, t4.size(0) / n, t4.size(1), t4.size(2), t4.size(3)}).permute({0, 2, 1, 3, 4}); }

struct Geo3 {
    std::array<int64_t, 3> st, pd, dl;
    int64_t Do;
};
Geo3 geo3(const at::Tensor& input, const at::Tensor& weight, at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation) {
    auto three = [](at::IntArrayRef v, int64_t dflt) {
        if (v.empty()) return std::array<int64_t, 3>{dflt, dflt, dflt};
        return v.size() == 1 ? std::array<int64_t, 3>{v[0], v[0], v[0]} : std::array<int64_t, 3>{v[0], v[1], v[2]};
    };
    Geo3 g{three(stride, 1), three(padding, 0), three(dilation, 1), 0};
    g.Do = (input.size(2) + 2 * g.pd[0] - g.dl[0] * (weight.size(2) - 1) - 1) / g.st[0] + 1;
    TORCH_CHECK(g.Do > 0, "torchvulkan [ERROR]: convolution: the filter does not fit the padded input");
    return g;
}

at::Tensor conv3d_by_taps(const at::Tensor& input, const at::Tensor& weight, at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation,
                          int64_t groups) {
    const Geo3 g = geo3(input, weight, stride, padding, dilation);
    const int64_t n = input.size(0);
    at::Tensor y;
    for (int64_t kd = 0; kd < weight.size(2); ++kd) {
        const DepthTap t = depth_tap(input.size(2), g.Do, kd, g.st[0], g.pd[0], g.dl[0]);
        if (t.count == 0) continue;
        at::Tensor x4 = fold_depth(input.slice(2, t.d0, t.d0 + (t.count - 1) * g.st[0] + 1, g.st[0]));
        at::Tensor y4 = conv2d_any(x4, contiguous_vulkan(weight.select(2, kd)), {g.st[1], g.st[2]}, {g.pd[1], g.pd[2]}, {g.dl[1], g.dl[2]}, groups);
        if (!y.defined()) y = at::zeros({n, weight.size(0), g.Do, y4.size(2), y4.size(3)}, input.options());
        y.slice(2, t.do0, t.do0 + t.count).add_(unfold_depth(y4, n));
    }
    TORCH_CHECK(y.defined(), "torchvulkan [ERROR]: convolution: no filter tap reaches the input");
    return y;
}

std::tuple<at::Tensor, at::Tensor> conv3d_by_taps_backward(const at::Tensor& gy, const at::Tensor& input, const at::Tensor& weight, at::IntArrayRef stride,
                                                            at::IntArrayRef padding, at::IntArrayRef dilation, int64_t groups, bool need_gx, bool need_gw) {
    const Geo3 g = geo3(input, weight, stride, padding, dilation);
    const int64_t n = input.size(0);
    at::Tensor gx, gw;
    if (need_gx) gx = at::zeros(input.sizes(), input.options());
    if (need_gw) gw = at::zeros(weight.sizes(), weight.options());
    for (int64_t kd = 0; kd < weight.size(2); ++kd) {
        const DepthTap t = depth_tap(input.size(2), g.Do, kd, g.st[0], g.pd[0], g.dl[0]);
        if (t.count == 0) continue;
        at::Tensor xs = input.slice(2, t.d0, t.d0 + (t.count - 1) * g.st[0] + 1, g.st[0]);
        at::Tensor x4 = fold_depth(xs), gy4 = fold_depth(gy.slice(2, t.do0, t.do0 + t.count));
        at::Tensor g4x, g4w;
        std::tie(g4x, g4w) = conv2d_any_backward(gy4, x4, contiguous_vulkan(weight.select(2, kd)), {g.st[1], g.st[2]}, {g.pd[1], g.pd[2]}, {g.dl[1], g.dl[2]}, groups,
                                                 need_gx, need_gw);
        if (need_gx) gx.slice(2, t.d0, t.d0 + (t.count - 1) * g.st[0] + 1, g.st[0]).add_(unfold_depth(g4x, n));
        if (need_gw) gw.select(2, kd).copy_(g4w);
    }
    return {gx, gw};
}

// Transposed 3-D convolution: the input gradient of the forward 3-D convolution that maps y's shape to x's shape. For one
// depth tap kd, input depth i of x adds conv_transpose2d(x[:, :, i], w[:, :, kd]) into output depth i * sd - pd + kd * dd:
// the same ranges as the forward convolution's taps with the roles of the two tensors exchanged, one transposed 2-D
// convolution over the batch n * depths per tap.
at::Tensor conv_transpose3d_by_taps(const at::Tensor& input, const at::Tensor& weight, at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation,
                                    at::IntArrayRef output_padding, int64_t groups) {
    auto three = [](at::IntArrayRef v, int64_t dflt) {
        if (v.empty()) return std::array<int64_t, 3>{dflt, dflt, dflt};
        return v.size() == 1 ? std::array<int64_t, 3>{v[0], v[0], v[0]} : std::array<int64_t, 3>{v[0], v[1], v[2]};
    };
    const auto st = three(stride, 1), pd = three(padding, 0), dl = three(dilation, 1), op = three(output_padding, 0);
    TORCH_CHECK(input.size(1) == weight.size(0), "torchvulkan [ERROR]: transposed convolution: input has ", input.size(1), " channels, weight expects ", weight.size(0));
    const int64_t n = input.size(0), D = input.size(2);
    const int64_t Dy = (D - 1) * st[0] - 2 * pd[0] + dl[0] * (weight.size(2) - 1) + op[0] + 1;
    TORCH_CHECK(Dy > 0, "torchvulkan [ERROR]: transposed convolution: empty output");
    at::Tensor y;
    for (int64_t kd = 0; kd < weight.size(2); ++kd) {
        // the forward convolution reads y's depths d0 + i * sd for x's depths do0 + i
        const DepthTap t = depth_tap(Dy, D, kd, st[0], pd[0], dl[0]);
        if (t.count == 0) continue;
        at::Tensor x4 = fold_depth(input.slice(2, t.do0, t.do0 + t.count));
        at::Tensor y4 = conv_transpose2d_any(x4, contiguous_vulkan(weight.select(2, kd)), {st[1], st[2]}, {pd[1], pd[2]}, {dl[1], dl[2]}, {op[1], op[2]}, groups);
        if (!y.defined()) y = at::zeros({n, weight.size(1) * groups, Dy, y4.size(2), y4.size(3)}, input.options());
        y.slice(2, t.d0, t.d0 + (t.count - 1) * st[0] + 1, st[0]).add_(unfold_depth(y4, n));
    }
    TORCH_CHECK(y.defined(), "torchvulkan [ERROR]: transposed convolution: no filter tap reaches the output");
    return y;
}

at::Tensor squeeze_h(const at::Tensor& t) { return t.defined() ? t.squeeze(2) : t; }

at::Tensor convolution_entry(const at::Tensor& input, const at::Tensor& weight, const c10::optional<at::Tensor>& bias, at::IntArrayRef stride,
                       at::IntArrayRef padding, at::IntArrayRef dilation, bool transposed, at::IntArrayRef output_padding, int64_t groups) {
    if (input.dim() == 3 && weight.dim() == 3) {
        // 1-D: a 2-D convolution of height 1 (the unit stride / zero padding along the added axis changes nothing)
        auto one = [](at::IntArrayRef v, int64_t dflt, int64_t h) { return std::vector<int64_t>{h, v.empty() ? dflt : v[0]}; };
        const int64_t s = stride.empty() ? 1 : stride[0];
        return convolution_entry(input.unsqueeze(2), weight.unsqueeze(2), bias, {s, s}, one(padding, 0, 0), one(dilation, 1, 1), transposed, one(output_padding, 0, 0), groups)
            .squeeze(2);
    }
    if (input.dim() == 5 && weight.dim() == 5) {
        at::Tensor y3 = transposed ? conv_transpose3d_by_taps(input, weight, stride, padding, dilation, output_padding, groups)
                                   : conv3d_by_taps(input, weight, stride, padding, dilation, groups);
        if (bias.has_value() && bias->defined()) y3.add_(bias->view({1, -1, 1, 1, 1}));
        return y3;
    }
    TORCH_CHECK(input.dim() == 4 && weight.dim() == 4, "torchvulkan [NOT IMPLEMENTED]: convolution of ", input.dim() - 2, " spatial dimensions");
    const Vec2 pd = pair_of(padding, 0), dl = pair_of(dilation, 1), op = pair_of(output_padding, 0);
    const Vec2 st = effective_stride(input, weight, pair_of(stride, 1), pd, op);
    at::Tensor y;
    if (!transposed && groups == 1) return conv2d_dense(input, weight, bias, {st[0], st[1]}, padding, dilation, false, 1);
    y = transposed ? conv_transpose2d_any(input, weight, st, pd, dl, op, groups) : conv2d_any(input, weight, st, pd, dl, groups);
    if (bias.has_value() && bias->defined()) y.add_(bias->view({1, -1, 1, 1}));
    return y;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> convolution_backward_entry(const at::Tensor& grad_output, const at::Tensor& input, const at::Tensor& weight,
                                                                    at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation,
                                                                    bool transposed, at::IntArrayRef output_padding, int64_t groups,
                                                                    std::array<bool, 3> output_mask) {
    if (input.dim() == 3 && weight.dim() == 3) {
        auto one = [](at::IntArrayRef v, int64_t dflt, int64_t h) { return std::vector<int64_t>{h, v.empty() ? dflt : v[0]}; };
        const int64_t s = stride.empty() ? 1 : stride[0];
        auto r = convolution_backward_entry(grad_output.unsqueeze(2), input.unsqueeze(2), weight.unsqueeze(2), {s, s}, one(padding, 0, 0), one(dilation, 1, 1), transposed,
                                      one(output_padding, 0, 0), groups, output_mask);
        return std::make_tuple(squeeze_h(std::get<0>(r)), squeeze_h(std::get<1>(r)), std::get<2>(r));
    }
    if (input.dim() == 5 && weight.dim() == 5) {
        at::Tensor gx3, gw3, gb3;
        if (!transposed) {
            std::tie(gx3, gw3) = conv3d_by_taps_backward(grad_output, input, weight, stride, padding, dilation, groups, output_mask[0], output_mask[1]);
        } else {
            // the forward 3-D convolution behind the transposed one maps grad_output's shape to input's shape
            if (output_mask[0]) gx3 = conv3d_by_taps(grad_output, weight, stride, padding, dilation, groups);
            if (output_mask[1]) gw3 = std::get<1>(conv3d_by_taps_backward(input, grad_output, weight, stride, padding, dilation, groups, false, true));
        }
        if (output_mask[2]) gb3 = grad_output.sum(at::IntArrayRef({0, 2, 3, 4}));
        return std::make_tuple(gx3, gw3, gb3);
    }
    TORCH_CHECK(input.dim() == 4 && weight.dim() == 4, "torchvulkan [NOT IMPLEMENTED]: convolution of ", input.dim() - 2, " spatial dimensions");
    const Vec2 pd = pair_of(padding, 0), dl = pair_of(dilation, 1);
    const Vec2 st = effective_stride(input, weight, pair_of(stride, 1), pd, pair_of(output_padding, 0));
    if (!transposed && groups == 1) return conv2d_dense_backward(grad_output, input, weight, {st[0], st[1]}, padding, dilation, false, 1, output_mask);
    at::Tensor gx, gw, gb;
    if (!transposed) {
        std::tie(gx, gw) = conv2d_any_backward(grad_output, input, weight, st, pd, dl, groups, output_mask[0], output_mask[1]);
    } else {
        // the forward convolution behind the transposed one maps grad_output's shape to input's shape
        if (output_mask[0]) gx = conv2d_any(grad_output, weight, st, pd, dl, groups);
        if (output_mask[1]) gw = std::get<1>(conv2d_any_backward(input, grad_output, weight, st, pd, dl, groups, false, true));
    }
    if (output_mask[2]) gb = grad_output.sum(at::IntArrayRef({0, 2, 3}));
    return std::make_tuple(gx, gw, gb);
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("convolution_overrideable", &convolution_entry);
    m.impl("convolution_backward_overrideable", &convolution_backward_entry);
}

}  // namespace tvk_aten
