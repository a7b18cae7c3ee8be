// Operators behind common torch.nn modules that are a handful of this backend's launches each: the fused LSTM / GRU cells
// (nn.LSTM, nn.GRU route every non-CPU device to them), the 4-D cross-entropy of segmentation heads, reflection and
// replication padding, weight normalisation.
//
// Counterparts in the reference: src/api/decompositions.cpp (the RNN cells, weight norm and the loss reshapes are written
// there over the backend's own elementwise operators as well), src/api/ops/shape.cpp (padding). The cell "workspace" tensors
// are private to the forward / backward pair of this backend.
#include "common.h"

#include <cmath>
#include <limits>

namespace tvk_aten {
namespace {

at::Tensor opt(const c10::optional<at::Tensor>& t) { return (t.has_value() && t->defined()) ? *t : at::Tensor(); }

// ---- LSTM cell: gates (i, f, g, o) = input_gates + hidden_gates (+ biases); cy = f cx + i g; hy = o tanh(cy) -------------
std::tuple<at::Tensor, at::Tensor, at::Tensor> lstm_cell(const at::Tensor& input_gates, const at::Tensor& hidden_gates, const at::Tensor& cx,
                                                          const c10::optional<at::Tensor>& input_bias, const c10::optional<at::Tensor>& hidden_bias) {
    at::Tensor gates = input_gates + hidden_gates;
    if (opt(input_bias).defined()) gates = gates + opt(input_bias);
    if (opt(hidden_bias).defined()) gates = gates + opt(hidden_bias);
    auto c = gates.chunk(4, 1);
    at::Tensor i = at::sigmoid(c[0]), f = at::sigmoid(c[1]), g = at::tanh(c[2]), o = at::sigmoid(c[3]);
    at::Tensor cy = f * cx + i * g;
    at::Tensor hy = o * at::tanh(cy);
    return {hy, cy, at::cat({i, f, g, o}, 1)};                  // workspace: the activated gates
}
std::tuple<at::Tensor, at::Tensor, at::Tensor> lstm_cell_backward(const c10::optional<at::Tensor>& grad_hy_o, const c10::optional<at::Tensor>& grad_cy_o,
                                                                   const at::Tensor& cx, const at::Tensor& cy, const at::Tensor& workspace, bool has_bias) {
    auto c = workspace.chunk(4, 1);
    const at::Tensor &i = c[0], &f = c[1], &g = c[2], &o = c[3];
    at::Tensor grad_hy = opt(grad_hy_o).defined() ? opt(grad_hy_o) : at::zeros_like(cy);
    at::Tensor tcy = at::tanh(cy);
    at::Tensor gcy = grad_hy * o * (1.0 - tcy * tcy);
    if (opt(grad_cy_o).defined()) gcy = gcy + opt(grad_cy_o);
    at::Tensor di = gcy * g * i * (1.0 - i), df = gcy * cx * f * (1.0 - f), dg = gcy * i * (1.0 - g * g), dout = grad_hy * tcy * o * (1.0 - o);
    at::Tensor grad_gates = at::cat({di, df, dg, dout}, 1);
    at::Tensor grad_bias = has_bias ? grad_gates.sum(at::IntArrayRef({0})) : at::Tensor();
    return {grad_gates, gcy * f, grad_bias};
}

// ---- GRU cell: r = s(ir + hr), z = s(iz + hz), n = tanh(in + r hn), hy = (1 - z) n + z hx ------------------------------------
std::tuple<at::Tensor, at::Tensor> gru_cell(const at::Tensor& input_gates, const at::Tensor& hidden_gates, const at::Tensor& hx,
                                             const c10::optional<at::Tensor>& input_bias, const c10::optional<at::Tensor>& hidden_bias) {
    at::Tensor ig = opt(input_bias).defined() ? input_gates + opt(input_bias) : input_gates;
    at::Tensor hg = opt(hidden_bias).defined() ? hidden_gates + opt(hidden_bias) : hidden_gates;
    auto ic = ig.chunk(3, 1), hc = hg.chunk(3, 1);
    at::Tensor r = at::sigmoid(ic[0] + hc[0]), z = at::sigmoid(ic[1] + hc[1]);
    at::Tensor n = at::tanh(ic[2] + r * hc[2]);
    at::Tensor hy = n + z * (hx - n);
    return {hy, at::cat({r, z, n, hx, hc[2]}, 1)};               // workspace: r, z, n, hx, the hidden side of n
}
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> gru_cell_backward(const at::Tensor& grad_hy, const at::Tensor& workspace, bool has_bias) {
    auto c = workspace.chunk(5, 1);
    const at::Tensor &r = c[0], &z = c[1], &n = c[2], &hx = c[3], &hn = c[4];
    at::Tensor dn = grad_hy * (1.0 - z) * (1.0 - n * n);
    at::Tensor dz = grad_hy * (hx - n) * z * (1.0 - z);
    at::Tensor dr = dn * hn * r * (1.0 - r);
    at::Tensor gi = at::cat({dr, dz, dn}, 1), gh = at::cat({dr, dz, dn * r}, 1);
    at::Tensor gib, ghb;
    if (has_bias) { gib = gi.sum(at::IntArrayRef({0})); ghb = gh.sum(at::IntArrayRef({0})); }
    return {gi, gh, grad_hy * z, gib, ghb};
}

// ---- cross-entropy over [N, C, H, W] logits (segmentation): the 2-D loss on the pixels as rows ------------------------------
std::tuple<at::Tensor, at::Tensor> nll_loss2d_forward(const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight, int64_t reduction,
                                                       c10::SymInt ignore_index) {
    TORCH_CHECK(self.dim() == 4 && target.dim() == 3, "nll_loss2d: expected [N, C, H, W] input and [N, H, W] target");
    const int64_t C = self.size(1);
    at::Tensor rows = contiguous_vulkan(self.permute({0, 2, 3, 1})).reshape({-1, C});
    at::Tensor out, total;
    std::tie(out, total) = at::nll_loss_forward_symint(rows, target.reshape({-1}), weight, reduction, ignore_index);
    if (reduction == at::Reduction::None) out = out.reshape(target.sizes());
    return {out, total};
}
at::Tensor nll_loss2d_backward(const at::Tensor& grad_output, const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight, int64_t reduction,
                               c10::SymInt ignore_index, const at::Tensor& total_weight) {
    const int64_t N = self.size(0), C = self.size(1), H = self.size(2), W = self.size(3);
    at::Tensor rows = contiguous_vulkan(self.permute({0, 2, 3, 1})).reshape({-1, C});
    at::Tensor g = reduction == at::Reduction::None ? grad_output.reshape({-1}) : grad_output;
    at::Tensor grad_rows = at::nll_loss_backward_symint(g, rows, target.reshape({-1}), weight, reduction, ignore_index, total_weight);
    return contiguous_vulkan(grad_rows.reshape({N, H, W, C}).permute({0, 3, 1, 2}));
}

// ---- reflection / replication padding: a gather per padded axis with host-computed source indices; the gradient adds back --
at::Tensor pad_indices(int64_t n, int64_t before, int64_t after, bool reflect, const at::Device& dev) {
    std::vector<int64_t> idx(n + before + after);
    for (int64_t o = 0; o < (int64_t)idx.size(); ++o) {
        int64_t s = o - before;
        if (reflect) { if (s < 0) s = -s; if (s >= n) s = 2 * (n - 1) - s; }
        else s = std::min<int64_t>(std::max<int64_t>(s, 0), n - 1);
        idx[o] = s;
    }
    return at::tensor(idx, at::TensorOptions().dtype(at::kLong)).to(dev);
}
at::Tensor pad_gather(const at::Tensor& self, at::IntArrayRef padding, bool reflect, const char* name) {
    const int64_t axes = (int64_t)padding.size() / 2;
    TORCH_CHECK(padding.size() % 2 == 0 && axes >= 1 && axes <= self.dim(), name, ": padding does not fit the input");
    at::Tensor r = self;
    for (int64_t a = 0; a < axes; ++a) {
        const int64_t dim = self.dim() - 1 - a, n = self.size(dim), before = padding[2 * a], after = padding[2 * a + 1];
        TORCH_CHECK(before >= 0 && after >= 0, "torchvulkan [NOT IMPLEMENTED]: ", name, " with negative padding");
        TORCH_CHECK(!reflect || (before < n && after < n), name, ": Padding size should be less than the corresponding input dimension");
        if (before == 0 && after == 0) continue;
        r = at::index_select(r, dim, pad_indices(n, before, after, reflect, self.device()));
    }
    return r.is_same(self) ? self.clone() : r;
}
at::Tensor pad_gather_backward(const at::Tensor& grad, const at::Tensor& self, at::IntArrayRef padding, bool reflect) {
    const int64_t axes = (int64_t)padding.size() / 2;
    at::Tensor g = grad;
    for (int64_t a = 0; a < axes; ++a) {
        const int64_t dim = self.dim() - 1 - a, n = self.size(dim), before = padding[2 * a], after = padding[2 * a + 1];
        if (before == 0 && after == 0) continue;
        std::vector<int64_t> shape(g.sizes().begin(), g.sizes().end());
        shape[dim] = n;
        g = at::zeros(shape, g.options()).index_add(dim, pad_indices(n, before, after, reflect, self.device()), g);
    }
    return g;
}
at::Tensor reflection_pad(const at::Tensor& self, at::IntArrayRef padding) { return pad_gather(self, padding, true, "reflection_pad"); }
at::Tensor replication_pad(const at::Tensor& self, at::IntArrayRef padding) { return pad_gather(self, padding, false, "replication_pad"); }
at::Tensor reflection_pad_backward(const at::Tensor& grad, const at::Tensor& self, at::IntArrayRef padding) { return pad_gather_backward(grad, self, padding, true); }
at::Tensor replication_pad_backward(const at::Tensor& grad, const at::Tensor& self, at::IntArrayRef padding) { return pad_gather_backward(grad, self, padding, false); }

// ---- weight normalisation: w = v * g / ||v|| with the norm over every dimension but `dim` ------------------------------------
std::vector<int64_t> other_dims(const at::Tensor& v, int64_t dim) {
    std::vector<int64_t> d;
    for (int64_t i = 0; i < v.dim(); ++i)
        if (i != dim) d.push_back(i);
    return d;
}
std::tuple<at::Tensor, at::Tensor> weight_norm_interface(const at::Tensor& v, const at::Tensor& g, int64_t dim) {
    dim = at::maybe_wrap_dim(dim, v.dim());
    at::Tensor norms = at::linalg_vector_norm(v, 2, other_dims(v, dim), true);
    return {v * (g / norms), norms};
}
std::tuple<at::Tensor, at::Tensor> weight_norm_interface_backward(const at::Tensor& grad_w, const at::Tensor& v, const at::Tensor& g, const at::Tensor& norms, int64_t dim) {
    dim = at::maybe_wrap_dim(dim, v.dim());
    at::Tensor dot = (grad_w * v).sum(other_dims(v, dim), true);
    at::Tensor grad_g = dot / norms;
    at::Tensor grad_v = (g / norms) * (grad_w - v * (dot / (norms * norms)));
    return {grad_v, grad_g};
}

// ---- F.unfold / F.fold: patches as columns. Each spatial axis is a gather with the index vector (tap, output position) ->
// padded input position; the adjoint adds the columns back. [N, C, H, W] <-> [N, C * kh * kw, Ho * Wo] ------------------
struct PatchAxis {
    int64_t out, padded;
    at::Tensor index;           // [k * out] positions in the padded axis
};
PatchAxis patch_axis(int64_t in, int64_t k, int64_t dil, int64_t pad, int64_t stride, const at::Device& dev) {
    PatchAxis a;
    a.padded = in + 2 * pad;
    a.out = (a.padded - dil * (k - 1) - 1) / stride + 1;
    TORCH_CHECK(a.out > 0, "im2col / col2im: the sliding blocks do not fit the padded input");
    std::vector<int64_t> idx((size_t)(k * a.out));
    for (int64_t t = 0; t < k; ++t)
        for (int64_t o = 0; o < a.out; ++o) idx[(size_t)(t * a.out + o)] = o * stride + t * dil;
    a.index = at::tensor(idx, at::TensorOptions().dtype(at::kLong)).to(dev);
    return a;
}
std::array<int64_t, 2> pair2(at::IntArrayRef v, const char* what) {
    TORCH_CHECK(v.size() == 1 || v.size() == 2, "im2col / col2im: ", what, " must have one or two values");
    return {v[0], v.size() == 1 ? v[0] : v[1]};
}
at::Tensor im2col(const at::Tensor& self, at::IntArrayRef kernel, at::IntArrayRef dilation, at::IntArrayRef padding, at::IntArrayRef stride) {
    TORCH_CHECK(self.dim() == 3 || self.dim() == 4, "im2col: expected a 3-D or 4-D input");
    at::Tensor x = self.dim() == 3 ? self.unsqueeze(0) : self;
    const auto k = pair2(kernel, "kernel_size"), d = pair2(dilation, "dilation"), p = pair2(padding, "padding"), st = pair2(stride, "stride");
    const int64_t N = x.size(0), C = x.size(1);
    const PatchAxis h = patch_axis(x.size(2), k[0], d[0], p[0], st[0], x.device()), w = patch_axis(x.size(3), k[1], d[1], p[1], st[1], x.device());
    at::Tensor xp = (p[0] || p[1]) ? at::constant_pad_nd(x, {p[1], p[1], p[0], p[0]}, 0) : x;
    at::Tensor g = at::index_select(at::index_select(xp, 2, h.index), 3, w.index);              // [N, C, kh*Ho, kw*Wo]
    g = g.reshape({N, C, k[0], h.out, k[1], w.out}).permute({0, 1, 2, 4, 3, 5});                // [N, C, kh, kw, Ho, Wo]
    at::Tensor cols = contiguous_vulkan(g).reshape({N, C * k[0] * k[1], h.out * w.out});
    return self.dim() == 3 ? cols.squeeze(0) : cols;
}
at::Tensor col2im(const at::Tensor& self, c10::SymIntArrayRef output_size, at::IntArrayRef kernel, at::IntArrayRef dilation, at::IntArrayRef padding,
                  at::IntArrayRef stride) {
    TORCH_CHECK((self.dim() == 2 || self.dim() == 3) && output_size.size() == 2, "col2im: expected a 2-D or 3-D input and two output sizes");
    at::Tensor cols = self.dim() == 2 ? self.unsqueeze(0) : self;
    const auto k = pair2(kernel, "kernel_size"), d = pair2(dilation, "dilation"), p = pair2(padding, "padding"), st = pair2(stride, "stride");
    const int64_t H = output_size[0].guard_int(__FILE__, __LINE__), W = output_size[1].guard_int(__FILE__, __LINE__);
    const int64_t N = cols.size(0), C = cols.size(1) / (k[0] * k[1]);
    const PatchAxis h = patch_axis(H, k[0], d[0], p[0], st[0], cols.device()), w = patch_axis(W, k[1], d[1], p[1], st[1], cols.device());
    TORCH_CHECK(cols.size(1) == C * k[0] * k[1] && cols.size(2) == h.out * w.out, "col2im: the input does not fit output_size and the sliding blocks");
    at::Tensor g = contiguous_vulkan(cols.reshape({N, C, k[0], k[1], h.out, w.out}).permute({0, 1, 2, 4, 3, 5})).reshape({N, C, k[0] * h.out, k[1] * w.out});
    at::Tensor gw = at::zeros({N, C, k[0] * h.out, w.padded}, cols.options()).index_add(3, w.index, g);
    at::Tensor gh = at::zeros({N, C, h.padded, w.padded}, cols.options()).index_add(2, h.index, gw);
    at::Tensor out = contiguous_vulkan(gh.narrow(2, p[0], H).narrow(3, p[1], W));
    return self.dim() == 2 ? out.squeeze(0) : out;
}

// embedding rows named by `indices` whose p-norm exceeds max_norm are scaled down to it (nn.Embedding(max_norm=...))
at::Tensor& embedding_renorm_(at::Tensor& self, const at::Tensor& indices, double max_norm, double norm_type) {
    TORCH_CHECK(self.dim() == 2, "embedding_renorm_: the weight must be 2-D");
    if (indices.numel() == 0) return self;
    at::Tensor hits = at::zeros({self.size(0)}, self.options().dtype(at::kFloat)).index_add(0, indices.reshape({-1}), at::ones({indices.numel()}, self.options().dtype(at::kFloat)));
    at::Tensor norms = at::linalg_vector_norm(self, norm_type, at::IntArrayRef({1}), false, at::kFloat);
    at::Tensor over = at::logical_and(at::gt(hits, 0), at::gt(norms, max_norm));
    at::Tensor scale = at::where(over, max_norm / (norms + 1e-7), at::ones({}, norms.options()));
    self.mul_(scale.to(self.scalar_type()).unsqueeze(1));
    return self;
}
at::Tensor trace(const at::Tensor& self) {
    TORCH_CHECK(self.dim() == 2, "trace: expected a matrix");
    return self.diagonal().sum();
}
at::Tensor tri_indices(int64_t row, int64_t col, int64_t offset, bool lower, c10::optional<at::ScalarType> dtype, const c10::optional<at::Device>& device) {
    at::TensorOptions host = at::TensorOptions().dtype(dtype.value_or(at::kLong)).device(at::kCPU);
    at::Tensor t = lower ? at::tril_indices(row, col, offset, host) : at::triu_indices(row, col, offset, host);
    return device.has_value() ? t.to(*device) : t;
}
at::Tensor tril_indices(int64_t row, int64_t col, int64_t offset, c10::optional<at::ScalarType> dtype, c10::optional<at::Layout>, c10::optional<at::Device> device,
                        c10::optional<bool>) {
    return tri_indices(row, col, offset, true, dtype, device);
}
at::Tensor triu_indices(int64_t row, int64_t col, int64_t offset, c10::optional<at::ScalarType> dtype, c10::optional<at::Layout>, c10::optional<at::Device> device,
                        c10::optional<bool>) {
    return tri_indices(row, col, offset, false, dtype, device);
}

// ---- F.grid_sample, 2-D, bilinear or nearest, zeros or border padding ------------------------------------------------------
// Sampling positions are turned into flat pixel offsets and corner weights with elementwise launches; the corner values are
// gathered from input viewed as [N, C, H*W] and the gradient with respect to the input is the scatter-add of the same
// corners. Coordinates follow ATen's grid sampler: x in [-1, 1] maps to pixel centres (align_corners) or pixel edges.
struct GridAxis {
    at::Tensor pos;        // unnormalised (and, for border padding, clamped) coordinate, fp32 [N, P]
    at::Tensor inside;     // border padding: 1 where the coordinate was not clamped (its derivative), else undefined
    double scale;          // d pos / d grid
};
GridAxis grid_axis(const at::Tensor& g, int64_t size, bool align_corners, int64_t padding_mode) {
    GridAxis a;
    if (align_corners) { a.scale = 0.5 * (double)(size - 1); a.pos = (g + 1.0) * a.scale; }
    else { a.scale = 0.5 * (double)size; a.pos = (g + 1.0) * a.scale - 0.5; }
    if (padding_mode == 1) {
        a.inside = at::logical_and(at::ge(a.pos, 0.0), at::le(a.pos, (double)(size - 1))).to(at::kFloat);
        a.pos = at::clamp(a.pos, 0.0, (double)(size - 1));
    }
    return a;
}
struct Corner {
    at::Tensor index, weight;      // [N, 1, P] Long flat offsets (clamped into the image) and fp32 weights (0 outside the image)
};
Corner make_corner(const at::Tensor& xi, const at::Tensor& yi, const at::Tensor& w, int64_t H, int64_t W) {
    at::Tensor valid = at::logical_and(at::logical_and(at::ge(xi, 0.0), at::le(xi, (double)(W - 1))), at::logical_and(at::ge(yi, 0.0), at::le(yi, (double)(H - 1)))).to(at::kFloat);
    at::Tensor xc = at::clamp(xi, 0.0, (double)(W - 1)), yc = at::clamp(yi, 0.0, (double)(H - 1));
    Corner c;
    c.index = (yc * (double)W + xc).to(at::kLong).unsqueeze(1);
    c.weight = (w * valid).unsqueeze(1);
    return c;
}
void check_grid_sampler(const at::Tensor& input, const at::Tensor& grid, int64_t interpolation_mode, int64_t padding_mode) {
    TORCH_CHECK(input.dim() == 4 && grid.dim() == 4 && grid.size(3) == 2 && grid.size(0) == input.size(0), "grid_sampler_2d: expected input [N, C, H, W] and grid [N, Ho, Wo, 2]");
    if (interpolation_mode > 1) TVK_NOT_IMPLEMENTED("grid_sample with bicubic interpolation");
    if (padding_mode > 1) TVK_NOT_IMPLEMENTED("grid_sample with reflection padding");
    if (!is_hot_float(input.scalar_type())) TVK_NOT_IMPLEMENTED("grid_sample for dtype ", input.scalar_type());
}
std::vector<Corner> grid_corners(const GridAxis& gx, const GridAxis& gy, int64_t H, int64_t W, bool nearest) {
    if (nearest) {
        at::Tensor one = at::ones({}, gx.pos.options());
        return {make_corner(at::round(gx.pos), at::round(gy.pos), one.expand_as(gx.pos), H, W)};
    }
    at::Tensor x0 = at::floor(gx.pos), y0 = at::floor(gy.pos);
    at::Tensor wx1 = gx.pos - x0, wy1 = gy.pos - y0, wx0 = 1.0 - wx1, wy0 = 1.0 - wy1;
    return {make_corner(x0, y0, wx0 * wy0, H, W), make_corner(x0 + 1.0, y0, wx1 * wy0, H, W), make_corner(x0, y0 + 1.0, wx0 * wy1, H, W),
            make_corner(x0 + 1.0, y0 + 1.0, wx1 * wy1, H, W)};
}
at::Tensor grid_sampler_2d(const at::Tensor& input, const at::Tensor& grid, int64_t interpolation_mode, int64_t padding_mode, bool align_corners) {
    check_grid_sampler(input, grid, interpolation_mode, padding_mode);
    const int64_t N = input.size(0), C = input.size(1), H = input.size(2), W = input.size(3), Ho = grid.size(1), Wo = grid.size(2), P = Ho * Wo;
    at::Tensor g = grid.to(at::kFloat).reshape({N, P, 2});
    const GridAxis gx = grid_axis(g.select(2, 0), W, align_corners, padding_mode), gy = grid_axis(g.select(2, 1), H, align_corners, padding_mode);
    at::Tensor flat = contiguous_vulkan(input).reshape({N, C, H * W}).to(at::kFloat);
    at::Tensor out;
    for (const Corner& c : grid_corners(gx, gy, H, W, interpolation_mode == 1)) {
        at::Tensor v = at::gather(flat, 2, c.index.expand({N, C, P})) * c.weight;
        out = out.defined() ? out + v : v;
    }
    return out.reshape({N, C, Ho, Wo}).to(input.scalar_type());
}
std::tuple<at::Tensor, at::Tensor> grid_sampler_2d_backward(const at::Tensor& grad_output, const at::Tensor& input, const at::Tensor& grid, int64_t interpolation_mode,
                                                             int64_t padding_mode, bool align_corners, std::array<bool, 2> output_mask) {
    check_grid_sampler(input, grid, interpolation_mode, padding_mode);
    const int64_t N = input.size(0), C = input.size(1), H = input.size(2), W = input.size(3), Ho = grid.size(1), Wo = grid.size(2), P = Ho * Wo;
    at::Tensor g = grid.to(at::kFloat).reshape({N, P, 2});
    const GridAxis gx = grid_axis(g.select(2, 0), W, align_corners, padding_mode), gy = grid_axis(g.select(2, 1), H, align_corners, padding_mode);
    const bool nearest = interpolation_mode == 1;
    const std::vector<Corner> corners = grid_corners(gx, gy, H, W, nearest);
    at::Tensor go = grad_output.to(at::kFloat).reshape({N, C, P});
    at::Tensor grad_input, grad_grid;
    if (output_mask[0]) {
        at::Tensor acc = at::zeros({N, C, H * W}, go.options());
        for (const Corner& c : corners) acc = acc.scatter_add(2, c.index.expand({N, C, P}), go * c.weight);
        grad_input = acc.reshape({N, C, H, W}).to(input.scalar_type());
    }
    if (output_mask[1]) {
        if (nearest) {
            grad_grid = at::zeros(grid.sizes(), grid.options());
        } else {
            // values of the four corners (0 outside the image), then d out / d x = sum_c go * ((v10 - v00) wy0 + (v11 - v01) wy1), likewise y
            at::Tensor flat = contiguous_vulkan(input).reshape({N, C, H * W}).to(at::kFloat);
            at::Tensor x0 = at::floor(gx.pos), y0 = at::floor(gy.pos);
            at::Tensor wx1 = (gx.pos - x0).unsqueeze(1), wy1 = (gy.pos - y0).unsqueeze(1), wx0 = 1.0 - wx1, wy0 = 1.0 - wy1;
            std::vector<at::Tensor> v;
            for (const Corner& c : corners) {
                // the corner's validity is its weight being a product of the fractional weights: recover the 0 / 1 mask from index clamping instead
                v.push_back(at::gather(flat, 2, c.index.expand({N, C, P})));
            }
            // re-mask the values with each corner's validity (weight / unmasked weight is not safe at zero weights)
            at::Tensor one = at::ones({}, gx.pos.options());
            const at::Tensor xs[4] = {x0, x0 + 1.0, x0, x0 + 1.0}, ys[4] = {y0, y0, y0 + 1.0, y0 + 1.0};
            for (int i = 0; i < 4; ++i) v[i] = v[i] * make_corner(xs[i], ys[i], one.expand_as(gx.pos), H, W).weight;
            at::Tensor dx = (go * ((v[1] - v[0]) * wy0 + (v[3] - v[2]) * wy1)).sum(at::IntArrayRef({1})) * gx.scale;      // [N, P]
            at::Tensor dy = (go * ((v[2] - v[0]) * wx0 + (v[3] - v[1]) * wx1)).sum(at::IntArrayRef({1})) * gy.scale;
            if (padding_mode == 1) { dx = dx * gx.inside; dy = dy * gy.inside; }
            grad_grid = at::stack({dx, dy}, 2).reshape(grid.sizes()).to(grid.scalar_type());
        }
    }
    return {grad_input, grad_grid};
}

// ---- pairwise distances (torch.cdist, the nearest-codebook search of vector quantisers) ------------------------------------------
// p = 2 through the matmul expansion |a|^2 + |b|^2 - 2 a.b (the large term is one tensor-core product); other p by broadcasting.
at::Tensor cdist_forward(const at::Tensor& x1, const at::Tensor& x2, double p, c10::optional<int64_t>) {
    TORCH_CHECK(x1.dim() >= 2 && x2.dim() >= 2 && x1.size(-1) == x2.size(-1), "cdist: expected two batches of row vectors of the same length");
    if (p == 2.0) {
        at::Tensor a2 = (x1 * x1).sum(at::IntArrayRef({-1}), true), b2 = (x2 * x2).sum(at::IntArrayRef({-1}), false).unsqueeze(-2);
        return at::sqrt(at::clamp_min(a2 + b2 - at::matmul(x1, x2.transpose(-1, -2)) * 2.0, 0.0));
    }
    at::Tensor diff = at::abs(x1.unsqueeze(-2) - x2.unsqueeze(-3));
    if (p == 1.0) return diff.sum(at::IntArrayRef({-1}));
    if (std::isinf(p)) return at::amax(diff, {-1}, false);
    if (p == 0.0) return at::ne(diff, 0).to(x1.scalar_type()).sum(at::IntArrayRef({-1}));
    return at::pow(at::pow(diff, p).sum(at::IntArrayRef({-1})), 1.0 / p);
}
at::Tensor cdist_backward(const at::Tensor& grad, const at::Tensor& x1, const at::Tensor& x2, double p, const at::Tensor& cdist) {
    if (p != 2.0) TVK_NOT_IMPLEMENTED("the gradient of cdist for p other than 2");
    // d/dx1_i = sum_j grad_ij (x1_i - x2_j) / d_ij (0 where the distance is 0): x1 * rowsum(G) - G @ x2 with G = grad / d
    at::Tensor G = at::where(at::gt(cdist, 0), grad / cdist, at::zeros({}, grad.options()));
    return x1 * G.sum(at::IntArrayRef({-1}), true) - at::matmul(G, x2);
}

// bucketize / searchsorted: the insertion position is the number of boundaries below (right: not above) the value - a broadcast
// comparison and an exact integer count. For boundary vectors of a few thousand entries.
at::Tensor count_below(const at::Tensor& seq, const at::Tensor& values, bool right, bool out_int32) {
    at::Tensor b = seq.unsqueeze(-2), v = values.unsqueeze(-1);
    at::Tensor pos = (right ? at::le(b, v) : at::lt(b, v)).sum(at::IntArrayRef({-1}));
    return out_int32 ? pos.to(at::kInt) : pos;
}
at::Tensor bucketize(const at::Tensor& self, const at::Tensor& boundaries, bool out_int32, bool right) {
    TORCH_CHECK(boundaries.dim() == 1, "boundaries tensor must be 1 dimension, but got dim(", boundaries.dim(), ")");
    return count_below(boundaries, self, right, out_int32);
}
at::Tensor searchsorted(const at::Tensor& sorted_sequence, const at::Tensor& self, bool out_int32, bool right, c10::optional<c10::string_view> side,
                        const c10::optional<at::Tensor>& sorter) {
    if (sorter.has_value() && sorter->defined()) TVK_NOT_IMPLEMENTED("searchsorted with a sorter");
    const bool r = right || (side.has_value() && *side == "right");
    TORCH_CHECK(sorted_sequence.dim() == 1 || sorted_sequence.dim() == self.dim(), "searchsorted: the sorted sequence must be 1-D or have the dimensions of the values");
    return count_below(sorted_sequence, self, r, out_int32);
}

at::Tensor vdot(const at::Tensor& a, const at::Tensor& b) { return at::dot(a, b); }                 // real tensors: no conjugate
at::Tensor& where_self_out(const at::Tensor& cond, const at::Tensor& a, const at::Tensor& b, at::Tensor& out) {
    at::Tensor r = at::where(cond, a, b);
    if (out.sizes() != r.sizes()) out.resize_(r.sizes());
    out.copy_(r);
    return out;
}

// ---- nn.EmbeddingBag (sum and mean) ----------------------------------------------------------------------------------------
// Bags are runs of `indices` starting at `offsets`. The bag of every position is the number of later bag starts at or before
// it (a searchsorted over the starts); the output is an index_add of the gathered rows into their bags, the weight gradient
// an index_add of the bags' gradients into the rows. Entries equal to padding_idx weigh nothing and are not counted in a
// mean. Positions ride in fp32, which bounds the number of indices.
struct Bags {
    at::Tensor indices, bag, scale;            // Long [n], Long [n], and the per-entry factor (undefined = all ones)
    int64_t count;
};
Bags bags_of(const at::Tensor& indices_in, const at::Tensor& offsets_in, bool include_last_offset, const c10::optional<at::Tensor>& per_sample_weights,
             int64_t padding_idx, at::ScalarType dtype) {
    TORCH_CHECK(indices_in.dim() == 1 && offsets_in.dim() == 1, "embedding_bag: indices and offsets must be 1-D here (a 2-D input is flattened by the caller)");
    Bags b;
    b.indices = indices_in.scalar_type() == at::kLong ? indices_in : indices_in.to(at::kLong);
    const int64_t n = b.indices.numel();
    TORCH_CHECK(n < (int64_t{1} << 24), "torchvulkan [NOT IMPLEMENTED]: embedding_bag over 2^24 indices or more");
    b.count = offsets_in.numel() - (include_last_offset ? 1 : 0);
    TORCH_CHECK(b.count >= 0, "embedding_bag: include_last_offset needs at least one offset");
    const at::TensorOptions long_opts = b.indices.options();
    if (b.count <= 1 || n == 0) {
        b.bag = at::zeros({n}, long_opts);
    } else {
        at::Tensor later_starts = offsets_in.narrow(0, 1, b.count - 1).to(at::kFloat).contiguous();
        at::Tensor positions = at::arange(n, at::TensorOptions().dtype(at::kFloat).device(at::kCPU)).to(b.indices.device());
        b.bag = at::searchsorted(later_starts, positions, false, true);
    }
    if (padding_idx >= 0) b.scale = at::ne(b.indices, padding_idx).to(dtype);
    if (per_sample_weights.has_value() && per_sample_weights->defined()) {
        TORCH_CHECK(per_sample_weights->dim() == 1 && per_sample_weights->numel() == n, "embedding_bag: per_sample_weights must have one entry per index");
        b.scale = b.scale.defined() ? b.scale * per_sample_weights->to(dtype) : per_sample_weights->to(dtype);
    }
    return b;
}
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> embedding_bag(const at::Tensor& weight, const at::Tensor& indices, const at::Tensor& offsets, bool,
                                                                         int64_t mode, bool sparse, const c10::optional<at::Tensor>& per_sample_weights,
                                                                         bool include_last_offset, int64_t padding_idx) {
    if (mode != 0 && mode != 1) TVK_NOT_IMPLEMENTED("embedding_bag in max mode");
    if (sparse) TVK_NOT_IMPLEMENTED("embedding_bag with sparse gradients");
    TORCH_CHECK(weight.dim() == 2, "embedding_bag: weight must be 2-D");
    const at::ScalarType st = weight.scalar_type();
    Bags b = bags_of(indices, offsets, include_last_offset, per_sample_weights, padding_idx, st);
    const int64_t n = b.indices.numel(), D = weight.size(1);
    at::Tensor out = at::zeros({b.count, D}, weight.options()), sizes = at::zeros({b.count}, weight.options().dtype(at::kFloat));
    if (n > 0 && b.count > 0) {
        at::Tensor rows = at::index_select(weight, 0, b.indices);
        if (b.scale.defined()) rows = rows * b.scale.unsqueeze(1);
        out = out.index_add(0, b.bag, rows);
        at::Tensor counted = padding_idx >= 0 ? at::ne(b.indices, padding_idx).to(at::kFloat) : at::ones({n}, sizes.options());
        sizes = sizes.index_add(0, b.bag, counted);
        if (mode == 1) out = out / at::clamp_min(sizes, 1.0).to(st).unsqueeze(1);
    }
    return {out, b.bag, sizes.to(at::kLong), at::empty({0}, b.indices.options())};
}
at::Tensor embedding_bag_backward(const at::Tensor& grad, const at::Tensor& indices, const at::Tensor& offsets, const at::Tensor& offset2bag,
                                  const at::Tensor& bag_size, const at::Tensor&, c10::SymInt num_weights, bool scale_grad_by_freq, int64_t mode, bool sparse,
                                  const c10::optional<at::Tensor>& per_sample_weights, int64_t padding_idx) {
    if (mode != 0 && mode != 1) TVK_NOT_IMPLEMENTED("embedding_bag backward in max mode");
    if (sparse || scale_grad_by_freq) TVK_NOT_IMPLEMENTED("embedding_bag backward with sparse gradients or scale_grad_by_freq");
    const at::ScalarType st = grad.scalar_type();
    Bags b = bags_of(indices, offsets, offsets.numel() > grad.size(0), per_sample_weights, padding_idx, st);
    at::Tensor table = at::zeros({num_weights.guard_int(__FILE__, __LINE__), grad.size(1)}, grad.options());
    if (b.indices.numel() == 0 || grad.size(0) == 0) return table;
    const at::Tensor& bag = offset2bag.numel() == b.indices.numel() ? offset2bag : b.bag;
    at::Tensor g = at::index_select(grad, 0, bag);
    if (mode == 1) g = g / at::index_select(at::clamp_min(bag_size.to(at::kFloat), 1.0).to(st), 0, bag).unsqueeze(1);
    if (b.scale.defined()) g = g * b.scale.unsqueeze(1);
    return table.index_add(0, b.indices, g);
}
at::Tensor embedding_bag_per_sample_weights_backward(const at::Tensor& grad, const at::Tensor& weight, const at::Tensor& indices, const at::Tensor& offsets,
                                                     const at::Tensor& offset2bag, int64_t mode, int64_t padding_idx) {
    TORCH_CHECK(mode == 0, "embedding_bag_backward: per_sample_weights only supported for mode='sum'");
    Bags b = bags_of(indices, offsets, offsets.numel() > grad.size(0), c10::nullopt, padding_idx, grad.scalar_type());
    if (b.indices.numel() == 0) return at::zeros({0}, grad.options());
    const at::Tensor& bag = offset2bag.numel() == b.indices.numel() ? offset2bag : b.bag;
    at::Tensor dots = at::sum(at::index_select(grad, 0, bag) * at::index_select(weight, 0, b.indices), {1});
    return b.scale.defined() ? dots * b.scale : dots;
}

// ---- inference fast paths of nn.MultiheadAttention and nn.TransformerEncoderLayer ------------------------------------------
// In eval mode without gradients those modules call one operator for the whole block on every device type they list, this
// one included. A mask marks what is EXCLUDED (nonzero / True / -inf), shaped by mask_type: 0 = [T, T] over (query, key),
// 1 = [B, T] key padding, 2 = [B, H, T, T]. A row with every key excluded comes out NaN, as ATen's own kernels leave it.
at::Tensor excluded_positions(const c10::optional<at::Tensor>& mask, c10::optional<int64_t> mask_type, int64_t B, int64_t T) {
    at::Tensor m = opt(mask);
    if (!m.defined()) return m;
    TORCH_CHECK(mask_type.has_value(), "a mask needs its mask_type");
    if (m.scalar_type() != at::kBool) m = m.to(at::kBool);
    switch (*mask_type) {
        case 0: TORCH_CHECK(m.dim() == 2 && m.size(0) == T && m.size(1) == T, "mask_type 0 expects a [T, T] mask"); return m.view({1, 1, T, T});
        case 1: TORCH_CHECK(m.dim() == 2 && m.size(0) == B && m.size(1) == T, "mask_type 1 expects a [B, T] mask"); return m.view({B, 1, 1, T});
        case 2: TORCH_CHECK(m.dim() == 4 && m.size(0) == B && m.size(2) == T && m.size(3) == T, "mask_type 2 expects a [B, H, T, T] mask"); return m;
        default: TORCH_CHECK(false, "unknown mask_type ", *mask_type);
    }
}
std::tuple<at::Tensor, at::Tensor> native_multi_head_attention(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value, int64_t embed_dim,
                                                               int64_t num_head, const at::Tensor& qkv_weight, const at::Tensor& qkv_bias,
                                                               const at::Tensor& proj_weight, const at::Tensor& proj_bias, const c10::optional<at::Tensor>& mask,
                                                               bool need_weights, bool average_attn_weights, c10::optional<int64_t> mask_type) {
    TORCH_CHECK(!query.is_nested() && !key.is_nested() && !value.is_nested(), "torchvulkan [NOT IMPLEMENTED]: multi-head attention on nested tensors");
    TORCH_CHECK(query.dim() == 3 && query.size(2) == embed_dim, "expected a [batch, sequence, ", embed_dim, "] query, got ", query.sizes());
    TORCH_CHECK(query.is_same(key) && key.is_same(value), "torchvulkan [NOT IMPLEMENTED]: the fused multi-head attention block is self-attention only");
    TORCH_CHECK(num_head > 0 && embed_dim % num_head == 0, "embed_dim ", embed_dim, " is not divisible by num_head ", num_head);
    TORCH_CHECK(qkv_weight.dim() == 2 && qkv_weight.size(0) == 3 * embed_dim && qkv_weight.size(1) == embed_dim, "expected a [3 * embed_dim, embed_dim] qkv_weight");
    const int64_t B = query.size(0), T = query.size(1), D = embed_dim, H = num_head, dh = D / H;
    auto parts = at::linear(query, qkv_weight, qkv_bias).chunk(3, -1);
    auto heads = [&](const at::Tensor& t) { return t.reshape({B, T, H, dh}).transpose(1, 2); };           // [B, H, T, dh]
    at::Tensor q = heads(parts[0]), k = heads(parts[1]), v = heads(parts[2]);
    at::Tensor excluded = excluded_positions(mask, mask_type, B, T);
    at::Tensor mixed, weights;
    if (!need_weights && !excluded.defined()) {
        mixed = at::scaled_dot_product_attention(q, k, v);
    } else {
        at::Tensor scores = at::matmul(q * (1.0 / std::sqrt(static_cast<double>(dh))), k.transpose(-1, -2));
        if (excluded.defined()) scores = scores.masked_fill(excluded, -std::numeric_limits<double>::infinity());
        at::Tensor w = at::softmax(scores, -1);
        mixed = at::matmul(w, v);
        if (need_weights) weights = average_attn_weights ? at::mean(w, {1}) : w;
    }
    at::Tensor out = at::linear(mixed.transpose(1, 2).reshape({B, T, D}), proj_weight, proj_bias);
    return {out, weights};
}
at::Tensor transformer_encoder_layer_fwd(const at::Tensor& src, int64_t embed_dim, int64_t num_heads, const at::Tensor& qkv_weight, const at::Tensor& qkv_bias,
                                         const at::Tensor& proj_weight, const at::Tensor& proj_bias, bool use_gelu, bool norm_first, double eps,
                                         const at::Tensor& norm_weight_1, const at::Tensor& norm_bias_1, const at::Tensor& norm_weight_2,
                                         const at::Tensor& norm_bias_2, const at::Tensor& ffn_weight_1, const at::Tensor& ffn_bias_1,
                                         const at::Tensor& ffn_weight_2, const at::Tensor& ffn_bias_2, const c10::optional<at::Tensor>& mask,
                                         c10::optional<int64_t> mask_type) {
    TORCH_CHECK(!src.is_nested(), "torchvulkan [NOT IMPLEMENTED]: the transformer encoder layer on nested tensors");
    at::Tensor x = norm_first ? at::layer_norm(src, {embed_dim}, norm_weight_1, norm_bias_1, eps) : src;
    x = std::get<0>(native_multi_head_attention(x, x, x, embed_dim, num_heads, qkv_weight, qkv_bias, proj_weight, proj_bias, mask, false, true, mask_type));
    x = x + src;
    if (!norm_first) x = at::layer_norm(x, {embed_dim}, norm_weight_1, norm_bias_1, eps);
    at::Tensor residual = x;
    if (norm_first) x = at::layer_norm(x, {embed_dim}, norm_weight_2, norm_bias_2, eps);
    x = at::linear(x, ffn_weight_1, ffn_bias_1);
    x = at::linear(use_gelu ? at::gelu(x) : at::relu(x), ffn_weight_2, ffn_bias_2);
    x = x + residual;
    if (!norm_first) x = at::layer_norm(x, {embed_dim}, norm_weight_2, norm_bias_2, eps);
    return x;
}
// nn.TransformerEncoder asks this before packing a padded batch into a nested tensor. There are no nested tensors on this
// device, so the answer is always "not left aligned": the batch stays padded and the layers receive the padding mask.
bool nested_tensor_from_mask_left_aligned(const at::Tensor&, const at::Tensor&) { return false; }

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("_embedding_bag", &embedding_bag);
    m.impl("_embedding_bag_forward_only", &embedding_bag);
    m.impl("_embedding_bag_backward", &embedding_bag_backward);
    m.impl("_embedding_bag_per_sample_weights_backward", &embedding_bag_per_sample_weights_backward);
    m.impl("_native_multi_head_attention", &native_multi_head_attention);
    m.impl("_transformer_encoder_layer_fwd", &transformer_encoder_layer_fwd);
    m.impl("_nested_tensor_from_mask_left_aligned", &nested_tensor_from_mask_left_aligned);
    m.impl("_thnn_fused_lstm_cell", &lstm_cell);
    m.impl("_thnn_fused_lstm_cell_backward_impl", &lstm_cell_backward);
    m.impl("_thnn_fused_gru_cell", &gru_cell);
    m.impl("_thnn_fused_gru_cell_backward", &gru_cell_backward);
    m.impl("nll_loss2d_forward", &nll_loss2d_forward);
    m.impl("nll_loss2d_backward", &nll_loss2d_backward);
    m.impl("reflection_pad1d", &reflection_pad);
    m.impl("reflection_pad2d", &reflection_pad);
    m.impl("reflection_pad1d_backward", &reflection_pad_backward);
    m.impl("reflection_pad2d_backward", &reflection_pad_backward);
    m.impl("reflection_pad3d", &reflection_pad);
    m.impl("reflection_pad3d_backward", &reflection_pad_backward);
    m.impl("replication_pad3d", &replication_pad);
    m.impl("replication_pad3d_backward", &replication_pad_backward);
    m.impl("replication_pad1d", &replication_pad);
    m.impl("replication_pad2d", &replication_pad);
    m.impl("replication_pad1d_backward", &replication_pad_backward);
    m.impl("replication_pad2d_backward", &replication_pad_backward);
    m.impl("_weight_norm_interface", &weight_norm_interface);
    m.impl("_weight_norm_interface_backward", &weight_norm_interface_backward);
    m.impl("grid_sampler_2d", &grid_sampler_2d);
    m.impl("grid_sampler_2d_backward", &grid_sampler_2d_backward);
    m.impl("_cdist_forward", &cdist_forward);
    m.impl("_cdist_backward", &cdist_backward);
    m.impl("bucketize.Tensor", &bucketize);
    m.impl("searchsorted.Tensor", &searchsorted);
    m.impl("im2col", &im2col);
    m.impl("col2im", &col2im);
    m.impl("embedding_renorm_", &embedding_renorm_);
    m.impl("trace", &trace);
    m.impl("tril_indices", &tril_indices);
    m.impl("triu_indices", &triu_indices);
    m.impl("vdot", &vdot);
    m.impl("where.self_out", &where_self_out);
}

}  // namespace tvk_aten
