// Operators behind common torch.nn modules that are a handful of this backend's launches each: the fused LSTM / GRU cells
// (nn.LSTM, nn.GRU route every non-CPU device to them), the 4-D cross-entropy of segmentation heads, reflection and
// replication padding, weight normalisation.
//
// Counterparts in the reference: src/api/decompositions.cpp (the RNN cells, weight norm and the loss reshapes are written
// there over the backend's own elementwise operators as well), src/api/ops/shape.cpp (padding). The cell "workspace" tensors
// are private to the forward / backward pair of this backend.
#include "common.h"

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

at::Tensor vdot(const at::Tensor& a, const at::Tensor& b) { return at::dot(a, b); }                 // real tensors: no conjugate
at::Tensor& where_self_out(const at::Tensor& cond, const at::Tensor& a, const at::Tensor& b, at::Tensor& out) {
    at::Tensor r = at::where(cond, a, b);
    if (out.sizes() != r.sizes()) out.resize_(r.sizes());
    out.copy_(r);
    return out;
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
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
    m.impl("replication_pad1d", &replication_pad);
    m.impl("replication_pad2d", &replication_pad);
    m.impl("replication_pad1d_backward", &replication_pad_backward);
    m.impl("replication_pad2d_backward", &replication_pad_backward);
    m.impl("_weight_norm_interface", &weight_norm_interface);
    m.impl("_weight_norm_interface_backward", &weight_norm_interface_backward);
    m.impl("vdot", &vdot);
    m.impl("where.self_out", &where_self_out);
}

}  // namespace tvk_aten
