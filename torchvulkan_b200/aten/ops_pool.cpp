// max_pool2d and avg_pool2d on the "vulkan" device, forward and backward, and the 3-D poolings composed from them.
//
// Counterparts in the reference: src/api/ops/pool.cpp (max_pool2d_with_indices, avg_pool2d and their backward entries).
// The kernels work on contiguous NCHW planes; a channels-last or strided input is made contiguous first and the outputs
// are NCHW. Output extents follow ATen's pooling_output_shape (floor or ceil mode, the last window must start inside the
// input or its left padding).
//
// A 3-D pooling window is a box, so it separates: pool height and width with depth riding as channels, then pool depth
// with (height x width) flattened into one axis. For the maximum the first stage's argmax is looked up at the depth the
// second stage picked, which gives ATen's flat index into (D, H, W) with its first-maximum rule; for the average the box
// count is the product of the per-axis counts in either padding-count mode, and a divisor override is applied once.
#include "common.h"

namespace tvk_aten {
namespace {

using Vec2 = std::array<int64_t, 2>;
Vec2 two(at::IntArrayRef v, const char* what, Vec2 dflt, bool allow_empty) {
    if (v.empty()) {
        TORCH_CHECK(allow_empty, "pool2d: ", what, " must either be a single int, or a tuple of two ints");
        return dflt;
    }
    TORCH_CHECK(v.size() == 1 || v.size() == 2, "pool2d: ", what, " must either be a single int, or a tuple of two ints");
    return v.size() == 1 ? Vec2{v[0], v[0]} : Vec2{v[0], v[1]};
}
int64_t out_extent(int64_t in, int64_t k, int64_t pad, int64_t stride, int64_t dil, bool ceil_mode) {
    const int64_t num = in + 2 * pad - dil * (k - 1) - 1 + (ceil_mode ? stride - 1 : 0);
    int64_t o = (num >= 0 ? num / stride : -((-num + stride - 1) / stride)) + 1;
    if (ceil_mode && (o - 1) * stride >= in + pad) --o;
    return o;
}
struct Pool {
    tvk_pool2d_desc d;
    std::vector<int64_t> out_shape;
};
Pool make_pool(const at::Tensor& x, at::IntArrayRef kernel, at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation, bool ceil_mode,
               const char* name) {
    TORCH_CHECK(x.dim() == 3 || x.dim() == 4, name, ": Expected 3D or 4D (batch mode) tensor, but got ", x.sizes());
    if (!is_hot_float(x.scalar_type())) TVK_NOT_IMPLEMENTED(name, " for dtype ", x.scalar_type(), " on the vulkan device");
    const Vec2 k = two(kernel, "kernel_size", {1, 1}, false), s = two(stride, "stride", k, true), p = two(padding, "padding", {0, 0}, true),
               dl = two(dilation, "dilation", {1, 1}, true);
    TORCH_CHECK(k[0] > 0 && k[1] > 0 && s[0] > 0 && s[1] > 0 && dl[0] > 0 && dl[1] > 0, name, ": kernel size, stride and dilation should be greater than zero");
    TORCH_CHECK(p[0] >= 0 && p[1] >= 0 && 2 * p[0] <= k[0] && 2 * p[1] <= k[1], name, ": pad should be at most half of effective kernel size, but got pad=", p[0],
                ", kernel_size=", k[0]);
    Pool r;
    const int64_t nd = x.dim(), H = x.size(nd - 2), W = x.size(nd - 1);
    const int64_t ho = out_extent(H, k[0], p[0], s[0], dl[0], ceil_mode), wo = out_extent(W, k[1], p[1], s[1], dl[1], ceil_mode);
    TORCH_CHECK(ho > 0 && wo > 0, name, ": Given input size ", x.sizes(), ", calculated output size is too small");
    r.d.dtype = to_tvk_dtype(x.scalar_type());
    r.d.planes = x.numel() / (H * W);
    r.d.h = H; r.d.w = W; r.d.ho = ho; r.d.wo = wo;
    r.d.kh = k[0]; r.d.kw = k[1]; r.d.stride_h = s[0]; r.d.stride_w = s[1]; r.d.pad_h = p[0]; r.d.pad_w = p[1]; r.d.dilation_h = dl[0]; r.d.dilation_w = dl[1];
    r.d.count_include_pad = 1;
    r.d.divisor_override = 0;
    r.out_shape.assign(x.sizes().begin(), x.sizes().end());
    r.out_shape[nd - 2] = ho;
    r.out_shape[nd - 1] = wo;
    return r;
}

std::tuple<at::Tensor, at::Tensor> max_pool2d_with_indices(const at::Tensor& self, at::IntArrayRef kernel, at::IntArrayRef stride, at::IntArrayRef padding,
                                                           at::IntArrayRef dilation, bool ceil_mode) {
    Pool p = make_pool(self, kernel, stride, padding, dilation, ceil_mode, "max_pool2d");
    at::Tensor x = contiguous_vulkan(self);
    at::Tensor y = empty_vulkan(p.out_shape, self.scalar_type(), self.device()), idx = empty_vulkan(p.out_shape, at::kLong, self.device());
    if (y.numel()) {
        DeviceScope scope(self);
        TVK_CALL(tvk_max_pool2d_forward(&p.d, y.data_ptr(), (int64_t*)idx.data_ptr(), x.data_ptr(), scope.stream));
    }
    return {y, idx};
}
at::Tensor max_pool2d_with_indices_backward(const at::Tensor& grad, const at::Tensor& self, at::IntArrayRef kernel, at::IntArrayRef stride, at::IntArrayRef padding,
                                            at::IntArrayRef dilation, bool ceil_mode, const at::Tensor& indices) {
    Pool p = make_pool(self, kernel, stride, padding, dilation, ceil_mode, "max_pool2d_backward");
    TORCH_CHECK(grad.sizes() == at::IntArrayRef(p.out_shape) && indices.sizes() == at::IntArrayRef(p.out_shape), "max_pool2d_backward: grad_output or indices do not fit the output shape");
    at::Tensor g = contiguous_vulkan(grad.to(self.scalar_type())), idx = contiguous_vulkan(indices);
    at::Tensor dx = empty_vulkan(self.sizes(), self.scalar_type(), self.device());
    if (dx.numel()) {
        DeviceScope scope(self);
        TVK_CALL(tvk_max_pool2d_backward(&p.d, dx.data_ptr(), g.data_ptr(), (const int64_t*)idx.data_ptr(), scope.stream));
    }
    return dx;
}

Pool make_avg(const at::Tensor& x, at::IntArrayRef kernel, at::IntArrayRef stride, at::IntArrayRef padding, bool ceil_mode, bool count_include_pad,
              c10::optional<int64_t> divisor_override, const char* name) {
    Pool p = make_pool(x, kernel, stride, padding, {1, 1}, ceil_mode, name);
    TORCH_CHECK(!divisor_override.has_value() || *divisor_override != 0, "divisor must be not zero");
    if (divisor_override.has_value() && *divisor_override < 0) TVK_NOT_IMPLEMENTED("avg_pool2d with a negative divisor_override");
    p.d.count_include_pad = count_include_pad ? 1 : 0;
    p.d.divisor_override = divisor_override.value_or(0);
    return p;
}
at::Tensor avg_pool2d(const at::Tensor& self, at::IntArrayRef kernel, at::IntArrayRef stride, at::IntArrayRef padding, bool ceil_mode, bool count_include_pad,
                      c10::optional<int64_t> divisor_override) {
    Pool p = make_avg(self, kernel, stride, padding, ceil_mode, count_include_pad, divisor_override, "avg_pool2d");
    at::Tensor x = contiguous_vulkan(self);
    at::Tensor y = empty_vulkan(p.out_shape, self.scalar_type(), self.device());
    if (y.numel()) {
        DeviceScope scope(self);
        TVK_CALL(tvk_avg_pool2d_forward(&p.d, y.data_ptr(), x.data_ptr(), scope.stream));
    }
    return y;
}
at::Tensor avg_pool2d_backward(const at::Tensor& grad, const at::Tensor& self, at::IntArrayRef kernel, at::IntArrayRef stride, at::IntArrayRef padding,
                               bool ceil_mode, bool count_include_pad, c10::optional<int64_t> divisor_override) {
    Pool p = make_avg(self, kernel, stride, padding, ceil_mode, count_include_pad, divisor_override, "avg_pool2d_backward");
    TORCH_CHECK(grad.sizes() == at::IntArrayRef(p.out_shape), "avg_pool2d_backward: grad_output does not fit the output shape");
    at::Tensor g = contiguous_vulkan(grad.to(self.scalar_type()));
    at::Tensor dx = empty_vulkan(self.sizes(), self.scalar_type(), self.device());
    if (dx.numel()) {
        DeviceScope scope(self);
        TVK_CALL(tvk_avg_pool2d_backward(&p.d, dx.data_ptr(), g.data_ptr(), scope.stream));
    }
    return dx;
}

using Vec3 = std::array<int64_t, 3>;
Vec3 three(at::IntArrayRef v, const char* what, Vec3 dflt, bool allow_empty) {
    if (v.empty()) {
        TORCH_CHECK(allow_empty, "pool3d: ", what, " must either be a single int, or a tuple of three ints");
        return dflt;
    }
    TORCH_CHECK(v.size() == 1 || v.size() == 3, "pool3d: ", what, " must either be a single int, or a tuple of three ints");
    return v.size() == 1 ? Vec3{v[0], v[0], v[0]} : Vec3{v[0], v[1], v[2]};
}
struct Volume {
    int64_t planes, D, H, W;
    std::vector<int64_t> lead;                          // the dimensions in front of (D, H, W)
    std::vector<int64_t> shape(int64_t d, int64_t h, int64_t w) const {
        std::vector<int64_t> s(lead);
        s.insert(s.end(), {d, h, w});
        return s;
    }
};
Volume volume_of(const at::Tensor& x, const char* name) {
    TORCH_CHECK(x.dim() == 4 || x.dim() == 5, name, ": Expected 4D or 5D (batch mode) tensor, but got ", x.sizes());
    const int64_t nd = x.dim();
    Volume v{1, x.size(nd - 3), x.size(nd - 2), x.size(nd - 1), {}};
    for (int64_t d = 0; d < nd - 3; ++d) { v.lead.push_back(x.size(d)); v.planes *= x.size(d); }
    return v;
}

std::tuple<at::Tensor, at::Tensor> max_pool3d_with_indices(const at::Tensor& self, at::IntArrayRef kernel, at::IntArrayRef stride, at::IntArrayRef padding,
                                                           at::IntArrayRef dilation, bool ceil_mode) {
    const Vec3 k = three(kernel, "kernel_size", {1, 1, 1}, false), s = three(stride, "stride", k, true), p = three(padding, "padding", {0, 0, 0}, true),
               dl = three(dilation, "dilation", {1, 1, 1}, true);
    const Volume v = volume_of(self, "max_pool3d");
    at::Tensor x = contiguous_vulkan(self).reshape({v.planes, v.D, v.H, v.W});
    auto [v1, i1] = at::max_pool2d_with_indices(x, {k[1], k[2]}, {s[1], s[2]}, {p[1], p[2]}, {dl[1], dl[2]}, ceil_mode);
    const int64_t Ho = v1.size(2), Wo = v1.size(3), area = Ho * Wo;
    auto [v2, i2] = at::max_pool2d_with_indices(v1.reshape({v.planes, 1, v.D, area}), {k[0], 1}, {s[0], 1}, {p[0], 0}, {dl[0], 1}, ceil_mode);
    const int64_t Do = v2.size(2);
    at::Tensor picked = i2.reshape({v.planes, Do * area});                                       // depth * area + position
    at::Tensor in_plane = at::gather(i1.reshape({v.planes, v.D * area}), 1, picked);            // h * W + w at that depth
    // depth * H * W for every (depth, position) the second stage can pick, built on the host
    at::Tensor plane_base = at::arange(v.D, at::TensorOptions().dtype(at::kLong).device(at::kCPU)).mul_(v.H * v.W).repeat_interleave(area).to(self.device());
    at::Tensor index = at::index_select(plane_base, 0, picked.reshape({-1})).reshape({v.planes, Do * area}) + in_plane;
    return {v2.reshape(v.shape(Do, Ho, Wo)), index.reshape(v.shape(Do, Ho, Wo))};
}
at::Tensor max_pool3d_with_indices_backward(const at::Tensor& grad, const at::Tensor& self, at::IntArrayRef, at::IntArrayRef, at::IntArrayRef, at::IntArrayRef,
                                            bool, const at::Tensor& indices) {
    const Volume v = volume_of(self, "max_pool3d_backward");
    TORCH_CHECK(grad.sizes() == indices.sizes(), "max_pool3d_backward: grad_output and indices differ in shape");
    if (self.numel() == 0) return at::zeros_like(self);
    at::Tensor zero = at::zeros({v.planes, v.D * v.H * v.W}, self.options());
    at::Tensor g = contiguous_vulkan(grad.to(self.scalar_type())).reshape({v.planes, -1});
    return at::scatter_add(zero, 1, contiguous_vulkan(indices).reshape({v.planes, -1}), g).reshape(self.sizes());
}

at::Tensor avg_pool3d(const at::Tensor& self, at::IntArrayRef kernel, at::IntArrayRef stride, at::IntArrayRef padding, bool ceil_mode, bool count_include_pad,
                      c10::optional<int64_t> divisor_override) {
    const Vec3 k = three(kernel, "kernel_size", {1, 1, 1}, false), s = three(stride, "stride", k, true), p = three(padding, "padding", {0, 0, 0}, true);
    const Volume v = volume_of(self, "avg_pool3d");
    const c10::optional<int64_t> first = divisor_override.has_value() ? c10::optional<int64_t>(1) : c10::nullopt;     // sum now, divide once
    at::Tensor a = at::avg_pool2d(contiguous_vulkan(self).reshape({v.planes, v.D, v.H, v.W}), {k[1], k[2]}, {s[1], s[2]}, {p[1], p[2]}, ceil_mode, count_include_pad, first);
    const int64_t Ho = a.size(2), Wo = a.size(3);
    at::Tensor b = at::avg_pool2d(a.reshape({v.planes, 1, v.D, Ho * Wo}), {k[0], 1}, {s[0], 1}, {p[0], 0}, ceil_mode, count_include_pad, divisor_override);
    return b.reshape(v.shape(b.size(2), Ho, Wo));
}
at::Tensor avg_pool3d_backward(const at::Tensor& grad, const at::Tensor& self, at::IntArrayRef kernel, at::IntArrayRef stride, at::IntArrayRef padding,
                               bool ceil_mode, bool count_include_pad, c10::optional<int64_t> divisor_override) {
    const Vec3 k = three(kernel, "kernel_size", {1, 1, 1}, false), s = three(stride, "stride", k, true), p = three(padding, "padding", {0, 0, 0}, true);
    const Volume v = volume_of(self, "avg_pool3d_backward");
    const c10::optional<int64_t> first = divisor_override.has_value() ? c10::optional<int64_t>(1) : c10::nullopt;
    const int64_t nd = grad.dim(), Do = grad.size(nd - 3), Ho = grad.size(nd - 2), Wo = grad.size(nd - 1);
    at::Tensor middle = empty_vulkan({v.planes, 1, v.D, Ho * Wo}, self.scalar_type(), self.device());            // only its shape is read
    at::Tensor g = contiguous_vulkan(grad.to(self.scalar_type())).reshape({v.planes, 1, Do, Ho * Wo});
    at::Tensor ga = at::avg_pool2d_backward(g, middle, {k[0], 1}, {s[0], 1}, {p[0], 0}, ceil_mode, count_include_pad, divisor_override);
    at::Tensor x = contiguous_vulkan(self).reshape({v.planes, v.D, v.H, v.W});
    return at::avg_pool2d_backward(ga.reshape({v.planes, v.D, Ho, Wo}), x, {k[1], k[2]}, {s[1], s[2]}, {p[1], p[2]}, ceil_mode, count_include_pad, first).reshape(self.sizes());
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("max_pool2d_with_indices", &max_pool2d_with_indices);
    m.impl("max_pool2d_with_indices_backward", &max_pool2d_with_indices_backward);
    m.impl("avg_pool2d", &avg_pool2d);
    m.impl("avg_pool2d_backward", &avg_pool2d_backward);
    m.impl("max_pool3d_with_indices", &max_pool3d_with_indices);
    m.impl("max_pool3d_with_indices_backward", &max_pool3d_with_indices_backward);
    m.impl("avg_pool3d", &avg_pool3d);
    m.impl("avg_pool3d_backward", &avg_pool3d_backward);
}

}  // namespace tvk_aten
