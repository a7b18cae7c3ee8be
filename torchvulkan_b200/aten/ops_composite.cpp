// Operators that are a few launches of this backend's own kernels: full and per-dimension max / min, all / any, variance
// and standard deviation, vector norms, masked_fill, tril / triu, the factory ranges, mse_loss.
//
// Counterparts in the reference: src/api/ops/reduce.cpp (max, min, all, any, prod ... registered at reduce.cpp:740-800),
// src/api/ops/indexing.cpp:423 (max.dim_max), src/api/ops/shape.cpp:269 (tril.out), src/api/ops/binary.cpp (masked ops).
// None of these is a hot path of the five benchmark configurations; they are here so that a training script's bookkeeping
// (gradient clipping, metrics, masks, position ids) runs on the device without a host round trip. Each is written over
// ATen calls that dispatch to the kernels of ops_eltwise.cpp / ops_reduce.cpp; reductions of 16-bit tensors accumulate in
// fp32 inside those kernels.
#include "common.h"

#include <algorithm>
#include <cmath>
#include <limits>

namespace tvk_aten {
namespace {

std::vector<int64_t> all_dims(const at::Tensor& t) {
    std::vector<int64_t> d(t.dim());
    for (int64_t i = 0; i < t.dim(); ++i) d[i] = i;
    return d;
}
std::vector<int64_t> dims_or_all(const at::Tensor& t, at::OptionalIntArrayRef dim) {
    if (!dim.has_value() || dim->empty()) return all_dims(t);
    return std::vector<int64_t>(dim->begin(), dim->end());
}
at::Tensor& into(at::Tensor& out, const at::Tensor& value) {
    if (out.sizes() != value.sizes()) out.resize_(value.sizes());
    out.copy_(value);
    return out;
}

// ---- max / min ----------------------------------------------------------------------------
at::Tensor max_all(const at::Tensor& self) {
    TORCH_CHECK(self.numel() > 0, "max(): Expected reduction dim to be specified for input.numel() == 0. Specify the reduction dim with the 'dim' argument.");
    return self.dim() == 0 ? self.clone() : at::amax(self, all_dims(self), false);
}
at::Tensor min_all(const at::Tensor& self) {
    TORCH_CHECK(self.numel() > 0, "min(): Expected reduction dim to be specified for input.numel() == 0. Specify the reduction dim with the 'dim' argument.");
    return self.dim() == 0 ? self.clone() : at::amin(self, all_dims(self), false);
}
at::Tensor& max_unary_out(const at::Tensor& self, at::Tensor& out) { return into(out, max_all(self)); }
at::Tensor& min_unary_out(const at::Tensor& self, at::Tensor& out) { return into(out, min_all(self)); }
// values by amax / amin, indices by argmax / argmin (the first extremum, NaN first: the rule of arg_reduce.slang:49-65)
std::tuple<at::Tensor, at::Tensor> max_dim(const at::Tensor& self, int64_t dim, bool keepdim) {
    return {at::amax(self, {dim}, keepdim), at::argmax(self, dim, keepdim)};
}
std::tuple<at::Tensor, at::Tensor> min_dim(const at::Tensor& self, int64_t dim, bool keepdim) {
    return {at::amin(self, {dim}, keepdim), at::argmin(self, dim, keepdim)};
}
std::tuple<at::Tensor&, at::Tensor&> max_dim_out(const at::Tensor& self, int64_t dim, bool keepdim, at::Tensor& values, at::Tensor& indices) {
    into(values, at::amax(self, {dim}, keepdim));
    into(indices, at::argmax(self, dim, keepdim));
    return {values, indices};
}
std::tuple<at::Tensor&, at::Tensor&> min_dim_out(const at::Tensor& self, int64_t dim, bool keepdim, at::Tensor& values, at::Tensor& indices) {
    into(values, at::amin(self, {dim}, keepdim));
    into(indices, at::argmin(self, dim, keepdim));
    return {values, indices};
}

// ---- all / any ----------------------------------------------------------------------------
// the truth values as 0 / 1 floats, reduced by amin (all) or amax (any)
at::Tensor truth01(const at::Tensor& self) { return (self.scalar_type() == at::kBool ? self : at::ne(self, 0)).to(at::kFloat); }
at::Tensor all_any(const at::Tensor& self, std::vector<int64_t> dims, bool keepdim, bool is_all) {
    if (self.numel() == 0 || self.dim() == 0) {
        // the empty conjunction is true, the empty disjunction false; a 0-dim tensor is its own truth value
        if (self.dim() == 0 && self.numel()) return at::ne(self, 0);
        std::vector<int64_t> shape;
        for (int64_t i = 0; i < self.dim(); ++i) {
            const bool reduced = std::find_if(dims.begin(), dims.end(), [&](int64_t d) { return (d < 0 ? d + self.dim() : d) == i; }) != dims.end();
            if (!reduced) shape.push_back(self.size(i));
            else if (keepdim) shape.push_back(1);
        }
        at::Tensor r = at::empty(shape, self.options().dtype(at::kBool));
        r.fill_(is_all);
        return r;
    }
    at::Tensor f = truth01(self);
    return at::gt(is_all ? at::amin(f, dims, keepdim) : at::amax(f, dims, keepdim), 0.5);
}
at::Tensor all_full(const at::Tensor& self) { return all_any(self, all_dims(self), false, true); }
at::Tensor any_full(const at::Tensor& self) { return all_any(self, all_dims(self), false, false); }
at::Tensor all_dim(const at::Tensor& self, int64_t dim, bool keepdim) { return all_any(self, {dim}, keepdim, true); }
at::Tensor any_dim(const at::Tensor& self, int64_t dim, bool keepdim) { return all_any(self, {dim}, keepdim, false); }
at::Tensor all_dims_fn(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim) { return all_any(self, dims_or_all(self, dim), keepdim, true); }
at::Tensor any_dims_fn(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim) { return all_any(self, dims_or_all(self, dim), keepdim, false); }
at::Tensor& all_all_out(const at::Tensor& self, at::Tensor& out) { return into(out, all_full(self)); }
at::Tensor& any_all_out(const at::Tensor& self, at::Tensor& out) { return into(out, any_full(self)); }
at::Tensor& all_out(const at::Tensor& self, int64_t dim, bool keepdim, at::Tensor& out) { return into(out, all_dim(self, dim, keepdim)); }
at::Tensor& any_out(const at::Tensor& self, int64_t dim, bool keepdim, at::Tensor& out) { return into(out, any_dim(self, dim, keepdim)); }
at::Tensor& all_dims_out(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, at::Tensor& out) { return into(out, all_dims_fn(self, dim, keepdim)); }
at::Tensor& any_dims_out(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, at::Tensor& out) { return into(out, any_dims_fn(self, dim, keepdim)); }

// ---- variance, standard deviation, vector norm --------------------------------------------------
// two passes in fp32: the mean, then the sum of squared deviations divided by n - correction
std::tuple<at::Tensor, at::Tensor> var_mean_impl(const at::Tensor& self, at::OptionalIntArrayRef dim, const c10::optional<at::Scalar>& correction, bool keepdim) {
    TORCH_CHECK(is_hot_float(self.scalar_type()), "torchvulkan [NOT IMPLEMENTED]: var / std of ", self.scalar_type());
    const std::vector<int64_t> dims = dims_or_all(self, dim);
    at::Tensor x = self.to(at::kFloat);
    int64_t n = 1;
    for (int64_t d : dims) n *= self.size(d < 0 ? d + self.dim() : d);
    at::Tensor mean = self.dim() == 0 ? x : at::mean(x, dims, true);
    at::Tensor dev = x - mean;
    at::Tensor ss = self.dim() == 0 ? dev * dev : at::sum(dev * dev, dims, true);
    const double denom = (double)n - (correction.has_value() ? correction->toDouble() : 1.0);
    at::Tensor var = ss * (denom > 0.0 ? 1.0 / denom : std::numeric_limits<double>::quiet_NaN());
    if (!keepdim && self.dim() > 0) {
        std::vector<int64_t> sorted(dims);
        for (auto& d : sorted) d = d < 0 ? d + self.dim() : d;
        std::sort(sorted.rbegin(), sorted.rend());
        for (int64_t d : sorted) { var = var.squeeze(d); mean = mean.squeeze(d); }
    }
    return {var.to(self.scalar_type()), mean.to(self.scalar_type())};
}
at::Tensor var_correction(const at::Tensor& self, at::OptionalIntArrayRef dim, const c10::optional<at::Scalar>& correction, bool keepdim) {
    return std::get<0>(var_mean_impl(self, dim, correction, keepdim));
}
at::Tensor std_correction(const at::Tensor& self, at::OptionalIntArrayRef dim, const c10::optional<at::Scalar>& correction, bool keepdim) {
    return at::sqrt(std::get<0>(var_mean_impl(self, dim, correction, keepdim)));
}
std::tuple<at::Tensor, at::Tensor> var_mean_correction(const at::Tensor& self, at::OptionalIntArrayRef dim, const c10::optional<at::Scalar>& correction, bool keepdim) {
    return var_mean_impl(self, dim, correction, keepdim);
}
std::tuple<at::Tensor, at::Tensor> std_mean_correction(const at::Tensor& self, at::OptionalIntArrayRef dim, const c10::optional<at::Scalar>& correction, bool keepdim) {
    auto vm = var_mean_impl(self, dim, correction, keepdim);
    return {at::sqrt(std::get<0>(vm)), std::get<1>(vm)};
}

at::Tensor vector_norm(const at::Tensor& self, const at::Scalar& ord_s, at::OptionalIntArrayRef dim, bool keepdim, c10::optional<at::ScalarType> dtype) {
    const at::ScalarType out_st = dtype.value_or(self.scalar_type());
    TORCH_CHECK(is_hot_float(self.scalar_type()) && is_hot_float(out_st), "torchvulkan [NOT IMPLEMENTED]: vector norm of ", self.scalar_type());
    const double ord = ord_s.toDouble();
    at::Tensor x = self.to(at::kFloat);
    if (self.dim() == 0) x = x.reshape({1});
    const std::vector<int64_t> dims = self.dim() == 0 ? std::vector<int64_t>{0} : dims_or_all(self, dim);
    const bool keep = keepdim && self.dim() > 0;
    at::Tensor r;
    if (ord == 2.0) r = at::sqrt(at::sum(x * x, dims, keep));
    else if (ord == 1.0) r = at::sum(at::abs(x), dims, keep);
    else if (std::isinf(ord)) r = ord > 0 ? at::amax(at::abs(x), dims, keep) : at::amin(at::abs(x), dims, keep);
    else if (ord == 0.0) r = at::sum(at::ne(x, 0).to(at::kFloat), dims, keep);
    else r = at::pow(at::sum(at::pow(at::abs(x), ord), dims, keep), 1.0 / ord);
    if (self.dim() == 0) r = r.reshape({});
    return r.to(out_st);
}
at::Tensor& vector_norm_out(const at::Tensor& self, const at::Scalar& ord, at::OptionalIntArrayRef dim, bool keepdim, c10::optional<at::ScalarType> dtype, at::Tensor& out) {
    return into(out, vector_norm(self, ord, dim, keepdim, dtype));
}

// ---- masks ---------------------------------------------------------------------------------
at::Tensor& masked_fill_scalar_(at::Tensor& self, const at::Tensor& mask, const at::Scalar& value) {
    TORCH_CHECK(mask.scalar_type() == at::kBool, "masked_fill_ only supports boolean masks, but got mask with dtype ", mask.scalar_type());
    at::Tensor v = at::empty({}, self.options());
    v.fill_(value);
    self.copy_(at::where(mask, v, self));
    return self;
}
at::Tensor& masked_fill_tensor_(at::Tensor& self, const at::Tensor& mask, const at::Tensor& value) {
    TORCH_CHECK(mask.scalar_type() == at::kBool, "masked_fill_ only supports boolean masks, but got mask with dtype ", mask.scalar_type());
    TORCH_CHECK(value.dim() == 0, "masked_fill_ only supports a 0-dimensional value tensor, but got tensor with ", value.dim(), " dimension(s).");
    self.copy_(at::where(mask, value.to(self.options()), self));
    return self;
}

// lower / upper triangle of the last two dimensions: the band mask is built on the host (rows x cols booleans) and applied
// with one where launch
at::Tensor tri_impl(const at::Tensor& self, int64_t diagonal, bool lower) {
    TORCH_CHECK(self.dim() >= 2, lower ? "tril" : "triu", ": input tensor must have at least 2 dimensions");
    const int64_t rows = self.size(-2), cols = self.size(-1);
    at::Tensor band = at::ones({rows, cols}, at::TensorOptions().dtype(at::kBool).device(at::kCPU));
    band = lower ? band.tril(diagonal) : band.triu(diagonal);
    at::Tensor zero = at::empty({}, self.options());
    zero.fill_(0);
    return at::where(band.to(self.device()), self, zero);
}
at::Tensor tril(const at::Tensor& self, int64_t diagonal) { return tri_impl(self, diagonal, true); }
at::Tensor triu(const at::Tensor& self, int64_t diagonal) { return tri_impl(self, diagonal, false); }
at::Tensor& tril_(at::Tensor& self, int64_t diagonal) { self.copy_(tri_impl(self, diagonal, true)); return self; }
at::Tensor& triu_(at::Tensor& self, int64_t diagonal) { self.copy_(tri_impl(self, diagonal, false)); return self; }
at::Tensor& tril_out(const at::Tensor& self, int64_t diagonal, at::Tensor& out) { return into(out, tri_impl(self, diagonal, true)); }
at::Tensor& triu_out(const at::Tensor& self, int64_t diagonal, at::Tensor& out) { return into(out, tri_impl(self, diagonal, false)); }

// ---- ranges: computed on the host (they are index vectors, a few KB) and copied to the device ---------------------
at::Tensor& arange_out(const at::Scalar& start, const at::Scalar& end, const at::Scalar& step, at::Tensor& out) {
    at::Tensor host = at::arange(start, end, step, out.options().device(at::kCPU));
    return into(out, host);
}
at::Tensor& linspace_out(const at::Scalar& start, const at::Scalar& end, int64_t steps, at::Tensor& out) {
    at::Tensor host = at::linspace(start, end, steps, out.options().device(at::kCPU));
    return into(out, host);
}
at::Tensor& eye_m_out(int64_t n, int64_t m, at::Tensor& out) {
    at::Tensor host = at::eye(n, m, out.options().device(at::kCPU));
    return into(out, host);
}
at::Tensor& eye_out(int64_t n, at::Tensor& out) { return eye_m_out(n, n, out); }

// ---- mse_loss ------------------------------------------------------------------------------
at::Tensor mse_loss(const at::Tensor& self, const at::Tensor& target, int64_t reduction) {
    at::Tensor d = self - target;
    at::Tensor sq = d * d;
    if (reduction == at::Reduction::Mean) return sq.numel() ? at::mean(sq, all_dims(sq), false) : sq.sum() / 0.0;
    if (reduction == at::Reduction::Sum) return at::sum(sq, all_dims(sq), false);
    return sq;
}
at::Tensor mse_loss_backward(const at::Tensor& grad, const at::Tensor& self, const at::Tensor& target, int64_t reduction) {
    const double norm = reduction == at::Reduction::Mean ? 2.0 / (double)std::max<int64_t>(self.numel(), 1) : 2.0;
    return (self - target) * grad * norm;
}

// ---- smooth-L1 / Huber losses, xlogy (kl_div, binary_cross_entropy) ---------------------------------
at::Tensor reduce_loss(const at::Tensor& v, int64_t reduction) {
    if (reduction == at::Reduction::Mean) return v.numel() ? at::mean(v, all_dims(v), false) : v.sum() / 0.0;
    if (reduction == at::Reduction::Sum) return at::sum(v, all_dims(v), false);
    return v;
}
double loss_norm(const at::Tensor& self, int64_t reduction) { return reduction == at::Reduction::Mean ? 1.0 / (double)std::max<int64_t>(self.numel(), 1) : 1.0; }
// |d| < beta ? 0.5 d^2 / beta : |d| - 0.5 beta   (beta == 0: the L1 loss)
at::Tensor smooth_l1_loss(const at::Tensor& self, const at::Tensor& target, int64_t reduction, double beta) {
    TORCH_CHECK(beta >= 0, "smooth_l1_loss does not support negative values for beta.");
    at::Tensor d = at::abs(self - target);
    if (beta == 0) return reduce_loss(d, reduction);
    return reduce_loss(at::where(at::lt(d, beta), d * d * (0.5 / beta), d - 0.5 * beta), reduction);
}
at::Tensor smooth_l1_loss_backward(const at::Tensor& grad, const at::Tensor& self, const at::Tensor& target, int64_t reduction, double beta) {
    at::Tensor d = self - target;
    at::Tensor slope = beta == 0 ? at::sign(d) : at::clamp(d * (1.0 / beta), -1.0, 1.0);
    return slope * grad * loss_norm(self, reduction);
}
// |d| <= delta ? 0.5 d^2 : delta (|d| - 0.5 delta)
at::Tensor huber_loss(const at::Tensor& self, const at::Tensor& target, int64_t reduction, double delta) {
    TORCH_CHECK(delta > 0, "huber_loss does not support non-positive values for delta.");
    at::Tensor d = at::abs(self - target);
    return reduce_loss(at::where(at::le(d, delta), d * d * 0.5, (d - 0.5 * delta) * delta), reduction);
}
at::Tensor huber_loss_backward(const at::Tensor& grad, const at::Tensor& self, const at::Tensor& target, int64_t reduction, double delta) {
    return at::clamp(self - target, -delta, delta) * grad * loss_norm(self, reduction);
}
// x * log(y), 0 where x == 0 (whatever y), NaN where y is NaN
at::Tensor vk_xlogy(const at::Tensor& x, const at::Tensor& y) {
    at::Tensor zero = at::zeros({}, y.options());
    at::Tensor r = at::where(at::eq(x, 0), zero, x * at::log(y));
    return at::where(at::isnan(y), y, r);
}
at::Tensor& xlogy_out(const at::Tensor& x, const at::Tensor& y, at::Tensor& out) { return into(out, vk_xlogy(x, y)); }

// binary_cross_entropy on probabilities: -(t log x + (1 - t) log(1 - x)), each logarithm clamped at -100 as ATen does
at::Tensor bce(const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight, int64_t reduction) {
    at::Tensor lx = at::clamp_min(at::log(self), -100.0), l1x = at::clamp_min(at::log1p(at::neg(self)), -100.0);
    at::Tensor v = at::neg(target * lx + (1.0 - target) * l1x);
    if (weight.has_value() && weight->defined()) v = v * *weight;
    return reduce_loss(v, reduction);
}
at::Tensor bce_backward(const at::Tensor& grad, const at::Tensor& self, const at::Tensor& target, const c10::optional<at::Tensor>& weight, int64_t reduction) {
    // d/dx = (x - t) / max(x (1 - x), eps)
    at::Tensor g = (self - target) / at::clamp_min(self * (1.0 - self), 1e-12) * grad * loss_norm(self, reduction);
    if (weight.has_value() && weight->defined()) g = g * *weight;
    return g;
}

// adaptive pooling to an output that divides the input evenly is ordinary pooling with kernel = stride = in / out
std::array<int64_t, 2> even_windows(const at::Tensor& self, at::IntArrayRef output_size, const char* name) {
    TORCH_CHECK(output_size.size() == 2 && (self.dim() == 3 || self.dim() == 4), name, ": expected a 3-D or 4-D input and two output sizes");
    const int64_t H = self.size(-2), W = self.size(-1);
    if (output_size[0] <= 0 || output_size[1] <= 0 || H % output_size[0] != 0 || W % output_size[1] != 0)
        TVK_NOT_IMPLEMENTED(name, " to an output size that does not divide the input (", H, " x ", W, " -> ", output_size[0], " x ", output_size[1], ")");
    return {H / output_size[0], W / output_size[1]};
}
bool divides_evenly(const at::Tensor& self, at::IntArrayRef output_size) {
    return output_size.size() == 2 && output_size[0] > 0 && output_size[1] > 0 && self.size(-2) % output_size[0] == 0 && self.size(-1) % output_size[1] == 0;
}
// [out, in] matrix whose row o averages inputs floor(o in / out) .. ceil((o + 1) in / out) - 1: the adaptive pooling window
at::Tensor adaptive_avg_matrix(int64_t in, int64_t out, const at::Tensor& like) {
    std::vector<float> a(static_cast<size_t>(out * in), 0.f);
    for (int64_t o = 0; o < out; ++o) {
        const int64_t s = (o * in) / out, e = ((o + 1) * in + out - 1) / out;
        for (int64_t i = s; i < e; ++i) a[static_cast<size_t>(o * in + i)] = 1.f / static_cast<float>(e - s);
    }
    return at::tensor(a, at::TensorOptions().dtype(at::kFloat)).view({out, in}).to(like.device()).to(like.scalar_type());
}
// uneven windows: the pooling is separable, one averaging matrix per axis, so it is two matrix products
at::Tensor adaptive_avg_by_matrices(const at::Tensor& x, int64_t H, int64_t W, int64_t Ho, int64_t Wo, bool transpose) {
    at::Tensor ah = adaptive_avg_matrix(H, Ho, x), aw = adaptive_avg_matrix(W, Wo, x);
    at::Tensor x3 = x.contiguous().reshape({-1, x.size(-2), x.size(-1)});
    at::Tensor y = transpose ? at::matmul(at::matmul(ah.t().contiguous(), x3), aw) : at::matmul(at::matmul(ah, x3), aw.t().contiguous());
    std::vector<int64_t> shape(x.sizes().begin(), x.sizes().end());
    shape[shape.size() - 2] = y.size(-2);
    shape[shape.size() - 1] = y.size(-1);
    return y.reshape(shape);
}
at::Tensor adaptive_avg_pool2d(const at::Tensor& self, at::IntArrayRef output_size) {
    if (divides_evenly(self, output_size)) {
        const auto k = even_windows(self, output_size, "adaptive_avg_pool2d");
        return at::avg_pool2d(self, {k[0], k[1]}, {k[0], k[1]});
    }
    TORCH_CHECK(output_size.size() == 2 && (self.dim() == 3 || self.dim() == 4) && output_size[0] > 0 && output_size[1] > 0,
                "adaptive_avg_pool2d: expected a 3-D or 4-D input and two positive output sizes");
    return adaptive_avg_by_matrices(self, self.size(-2), self.size(-1), output_size[0], output_size[1], false);
}
at::Tensor adaptive_avg_pool2d_backward(const at::Tensor& grad, const at::Tensor& self) {
    if (divides_evenly(self, {grad.size(-2), grad.size(-1)})) {
        const auto k = even_windows(self, {grad.size(-2), grad.size(-1)}, "adaptive_avg_pool2d_backward");
        return at::avg_pool2d_backward(grad, self, {k[0], k[1]}, {k[0], k[1]}, {0, 0}, false, true, c10::nullopt);
    }
    return adaptive_avg_by_matrices(grad, self.size(-2), self.size(-1), grad.size(-2), grad.size(-1), true);
}
// Uneven windows: a host-built table [Ho * Wo, L] of the flat input positions of every window, in row-major window order and
// padded by repeating the window's last row / column (a repeat cannot win the first-maximum rule), turns the pooling into one
// gather and one maximum along the last axis.
at::Tensor adaptive_window_table(int64_t H, int64_t W, int64_t Ho, int64_t Wo, const at::Device& dev) {
    auto start = [](int64_t o, int64_t in, int64_t out) { return (o * in) / out; };
    auto stop = [](int64_t o, int64_t in, int64_t out) { return ((o + 1) * in + out - 1) / out; };
    int64_t Lh = 1, Lw = 1;
    for (int64_t o = 0; o < Ho; ++o) Lh = std::max(Lh, stop(o, H, Ho) - start(o, H, Ho));
    for (int64_t o = 0; o < Wo; ++o) Lw = std::max(Lw, stop(o, W, Wo) - start(o, W, Wo));
    std::vector<int64_t> t;
    t.reserve(static_cast<size_t>(Ho * Wo * Lh * Lw));
    for (int64_t oh = 0; oh < Ho; ++oh)
        for (int64_t ow = 0; ow < Wo; ++ow)
            for (int64_t a = 0; a < Lh; ++a) {
                const int64_t h = std::min(start(oh, H, Ho) + a, stop(oh, H, Ho) - 1);
                for (int64_t b = 0; b < Lw; ++b) t.push_back(h * W + std::min(start(ow, W, Wo) + b, stop(ow, W, Wo) - 1));
            }
    return at::tensor(t, at::TensorOptions().dtype(at::kLong)).view({Ho * Wo, Lh * Lw}).to(dev);
}
std::tuple<at::Tensor, at::Tensor> adaptive_max_pool2d(const at::Tensor& self, at::IntArrayRef output_size) {
    if (divides_evenly(self, output_size)) {
        const auto k = even_windows(self, output_size, "adaptive_max_pool2d");
        return at::max_pool2d_with_indices(self, {k[0], k[1]}, {k[0], k[1]});
    }
    TORCH_CHECK(output_size.size() == 2 && (self.dim() == 3 || self.dim() == 4) && output_size[0] > 0 && output_size[1] > 0,
                "adaptive_max_pool2d: expected a 3-D or 4-D input and two positive output sizes");
    const int64_t H = self.size(-2), W = self.size(-1), Ho = output_size[0], Wo = output_size[1];
    at::Tensor table = adaptive_window_table(H, W, Ho, Wo, self.device());
    at::Tensor flat = self.contiguous().reshape({-1, H * W});
    const int64_t B = flat.size(0);
    at::Tensor windows = at::index_select(flat, 1, table.reshape({-1})).reshape({B, Ho * Wo, table.size(1)});
    auto [values, arg] = at::max(windows, -1, false);
    at::Tensor index = at::gather(table.unsqueeze(0).expand({B, Ho * Wo, table.size(1)}).contiguous(), 2, arg.unsqueeze(-1)).squeeze(-1);
    std::vector<int64_t> shape(self.sizes().begin(), self.sizes().end());
    shape[shape.size() - 2] = Ho;
    shape[shape.size() - 1] = Wo;
    return {values.reshape(shape), index.reshape(shape)};
}
at::Tensor adaptive_max_pool2d_backward(const at::Tensor& grad, const at::Tensor& self, const at::Tensor& indices) {
    if (divides_evenly(self, {grad.size(-2), grad.size(-1)})) {
        const auto k = even_windows(self, {grad.size(-2), grad.size(-1)}, "adaptive_max_pool2d_backward");
        return at::max_pool2d_with_indices_backward(grad, self, {k[0], k[1]}, {k[0], k[1]}, {0, 0}, {1, 1}, false, indices);
    }
    const int64_t HW = self.size(-2) * self.size(-1), B = HW == 0 ? 0 : self.numel() / HW;
    at::Tensor zero = at::zeros({B, HW}, grad.options());
    return at::scatter_add(zero, 1, indices.contiguous().reshape({B, -1}), grad.contiguous().reshape({B, -1})).reshape(self.sizes());
}

// Running maximum / minimum with the position it came from, as a log-step scan along the last axis: at step s every
// element is compared with the running result s places to its left. A strictly better left value wins, so ties keep the
// later position, and a NaN on the left wins over any number; both are ATen's rules.
void cum_extreme(const at::Tensor& self, at::Tensor& values, at::Tensor& indices, int64_t dim, bool is_max, const char* name) {
    const at::ScalarType st = self.scalar_type();
    const bool floating = is_hot_float(st);
    if (!(floating || st == at::kLong || st == at::kInt)) TVK_NOT_IMPLEMENTED(name, " for dtype ", st);
    if (self.numel() == 0) return;
    if (self.dim() == 0) { values.copy_(self); indices.zero_(); return; }
    dim = at::maybe_wrap_dim(dim, self.dim());
    const int64_t n = self.size(dim);
    at::Tensor moved = self.movedim(dim, -1).contiguous();
    const auto moved_shape = moved.sizes().vec();
    at::Tensor v = moved.reshape({-1, n});
    at::Tensor idx = at::arange(n, at::TensorOptions().dtype(at::kLong).device(at::kCPU)).to(self.device()).expand({v.size(0), n}).contiguous();
    at::Scalar worst;
    if (floating) worst = is_max ? -std::numeric_limits<double>::infinity() : std::numeric_limits<double>::infinity();
    else if (st == at::kLong) worst = is_max ? std::numeric_limits<int64_t>::min() : std::numeric_limits<int64_t>::max() - 1023;   // the fill goes through a double: 2^63 - 1024 is the largest value that survives
    else worst = static_cast<int64_t>(is_max ? std::numeric_limits<int32_t>::min() : std::numeric_limits<int32_t>::max());
    for (int64_t s = 1; s < n; s *= 2) {
        at::Tensor lv = at::full_like(v, worst), li = at::zeros_like(idx);
        lv.narrow(1, s, n - s).copy_(v.narrow(1, 0, n - s));
        li.narrow(1, s, n - s).copy_(idx.narrow(1, 0, n - s));
        at::Tensor take = is_max ? at::gt(lv, v) : at::lt(lv, v);
        if (floating) take = at::logical_or(take, at::logical_and(at::isnan(lv), at::logical_not(at::isnan(v))));
        v = at::where(take, lv, v);
        idx = at::where(take, li, idx);
    }
    values.copy_(v.reshape(moved_shape).movedim(-1, dim));
    indices.copy_(idx.reshape(moved_shape).movedim(-1, dim));
}
void cummax_helper(const at::Tensor& self, at::Tensor& values, at::Tensor& indices, int64_t dim) { cum_extreme(self, values, indices, dim, true, "cummax"); }
void cummin_helper(const at::Tensor& self, at::Tensor& values, at::Tensor& indices, int64_t dim) { cum_extreme(self, values, indices, dim, false, "cummin"); }

// torch.unique without a dimension: sort, mark the first element of every run, compact. The inverse is the run number
// scattered back through the sort permutation; a count is the distance between consecutive run starts. Integers are sorted
// as fp32, so they must be below 2^24 in magnitude, and run numbers are carried in fp32, which bounds the element count.
std::tuple<at::Tensor, at::Tensor, at::Tensor> unique2(const at::Tensor& self, bool, bool return_inverse, bool return_counts) {
    const at::ScalarType st = self.scalar_type();
    const bool floating = is_hot_float(st);
    if (!(floating || st == at::kLong || st == at::kInt)) TVK_NOT_IMPLEMENTED("unique for dtype ", st);
    const at::TensorOptions long_opts = self.options().dtype(at::kLong);
    const int64_t n = self.numel();
    if (n == 0) return {at::empty({0}, self.options()), at::empty(return_inverse ? self.sizes() : at::IntArrayRef{0}, long_opts), at::empty({0}, long_opts)};
    TORCH_CHECK(n <= (int64_t{1} << 24), "torchvulkan [NOT IMPLEMENTED]: unique of more than 2^24 elements");
    at::Tensor flat = self.contiguous().reshape({-1});
    at::Tensor work = floating ? flat : flat.to(at::kFloat);
    if (!floating && at::amax(at::abs(work), {0}).item<float>() >= 16777216.f) TVK_NOT_IMPLEMENTED("unique of integers of magnitude 2^24 or more");
    auto [vals, perm] = at::sort(work, 0, false);
    at::Tensor first = at::ones({n}, self.options().dtype(at::kBool));
    if (n > 1) first.narrow(0, 1, n - 1).copy_(at::ne(vals.narrow(0, 1, n - 1), vals.narrow(0, 0, n - 1)));
    at::Tensor uniq = at::masked_select(vals, first).to(st);
    at::Tensor inverse = at::empty({0}, long_opts), counts = at::empty({0}, long_opts);
    if (return_inverse) {
        at::Tensor run = at::cumsum(first.to(at::kFloat), 0) - 1.0;
        inverse = at::scatter_add(at::zeros({n}, run.options()), 0, perm, run).to(at::kLong).reshape(self.sizes());
    }
    if (return_counts) {
        at::Tensor pos = at::nonzero(first).reshape({-1});
        const int64_t u = pos.numel();
        at::Tensor next = at::full({u}, n, long_opts);
        if (u > 1) next.narrow(0, 0, u - 1).copy_(pos.narrow(0, 1, u - 1));
        counts = next - pos;
    }
    return {uniq, inverse, counts};
}
// bincount: ones (or the weights) added at their bin; the largest value sizes the result, which costs one read-back
at::Tensor bincount(const at::Tensor& self, const c10::optional<at::Tensor>& weights, int64_t minlength) {
    TORCH_CHECK(self.dim() == 1 && (self.scalar_type() == at::kLong || self.scalar_type() == at::kInt), "bincount only supports 1-d non-negative integral inputs.");
    TORCH_CHECK(minlength >= 0, "minlength should be >= 0");
    const bool weighted = weights.has_value() && weights->defined();
    const at::TensorOptions long_opts = self.options().dtype(at::kLong);
    if (self.numel() == 0) return at::zeros({minlength}, weighted ? weights->options() : long_opts);
    TORCH_CHECK(self.numel() <= (int64_t{1} << 24), "torchvulkan [NOT IMPLEMENTED]: bincount of more than 2^24 elements");
    at::Tensor as_float = self.to(at::kFloat);
    const float lo = at::amin(as_float, {0}).item<float>(), hi = at::amax(as_float, {0}).item<float>();
    TORCH_CHECK(lo >= 0.f, "bincount only supports 1-d non-negative integral inputs.");
    if (hi >= 16777216.f) TVK_NOT_IMPLEMENTED("bincount of values of 2^24 or more");
    const int64_t bins = std::max<int64_t>(static_cast<int64_t>(hi) + 1, minlength);
    at::Tensor index = self.scalar_type() == at::kLong ? self : self.to(at::kLong);
    if (weighted) {
        TORCH_CHECK(weights->dim() == 1 && weights->size(0) == self.size(0), "weights should be 1-d and have the same length as input");
        if (!is_hot_float(weights->scalar_type())) TVK_NOT_IMPLEMENTED("bincount with weights of dtype ", weights->scalar_type());
        return at::scatter_add(at::zeros({bins}, weights->options()), 0, index, *weights);
    }
    return at::scatter_add(at::zeros({bins}, as_float.options()), 0, index, at::ones_like(as_float)).to(at::kLong);
}

// cross product along a dimension of length 3: c_i = a_{i+1} b_{i+2} - a_{i+2} b_{i+1}, the shifted operands being rolls
at::Tensor vk_linalg_cross(const at::Tensor& self, const at::Tensor& other, int64_t dim) {
    auto both = at::broadcast_tensors({self, other});
    dim = at::maybe_wrap_dim(dim, both[0].dim());
    TORCH_CHECK(both[0].size(dim) == 3, "linalg.cross: inputs dimension ", dim, " must have length 3. Got ", self.size(dim), " and ", other.size(dim));
    at::Tensor a = both[0].contiguous(), b = both[1].contiguous();
    return at::roll(a, {-1}, {dim}) * at::roll(b, {-2}, {dim}) - at::roll(a, {-2}, {dim}) * at::roll(b, {-1}, {dim});
}
at::Tensor& vk_linalg_cross_out(const at::Tensor& self, const at::Tensor& other, int64_t dim, at::Tensor& out) { return into(out, vk_linalg_cross(self, other, dim)); }

// adaptive average pooling of a volume: one averaging matrix per axis, depth first and then the two plane axes
at::Tensor adaptive_avg_volume(const at::Tensor& x, at::IntArrayRef in, at::IntArrayRef out, bool transpose) {
    TORCH_CHECK(x.dim() == 4 || x.dim() == 5, "adaptive_avg_pool3d: expected a 4-D or 5-D input, got ", x.sizes());
    auto mat = [&](int i) {
        at::Tensor a = adaptive_avg_matrix(in[i], out[i], x);
        return transpose ? a.t().contiguous() : a;                        // forward [out, in]; backward [in, out]
    };
    const int64_t d0 = x.size(-3), h0 = x.size(-2), w0 = x.size(-1);
    const int64_t d1 = transpose ? in[0] : out[0], h1 = transpose ? in[1] : out[1], w1 = transpose ? in[2] : out[2];
    at::Tensor v = x.contiguous().reshape({-1, d0, h0 * w0});
    const int64_t P = v.size(0);
    v = at::matmul(mat(0), v).reshape({P * d1, h0, w0});
    v = at::matmul(at::matmul(mat(1), v), mat(2).t().contiguous());
    std::vector<int64_t> shape(x.sizes().begin(), x.sizes().end() - 3);
    shape.insert(shape.end(), {d1, h1, w1});
    return v.reshape(shape);
}
at::Tensor adaptive_avg_pool3d(const at::Tensor& self, at::IntArrayRef output_size) {
    TORCH_CHECK(output_size.size() == 3 && output_size[0] > 0 && output_size[1] > 0 && output_size[2] > 0, "adaptive_avg_pool3d: output_size must be three positive sizes");
    return adaptive_avg_volume(self, {self.size(-3), self.size(-2), self.size(-1)}, output_size, false);
}
at::Tensor adaptive_avg_pool3d_backward(const at::Tensor& grad, const at::Tensor& self) {
    return adaptive_avg_volume(grad, {self.size(-3), self.size(-2), self.size(-1)}, {grad.size(-3), grad.size(-2), grad.size(-1)}, true);
}

// a scalar base raised to a tensor of exponents
at::Tensor pow_scalar(const at::Scalar& base, const at::Tensor& exponent) {
    if (!is_hot_float(exponent.scalar_type())) TVK_NOT_IMPLEMENTED("pow(scalar, tensor) for exponent dtype ", exponent.scalar_type());
    return at::pow(at::full_like(exponent, base), exponent);
}
// torch.normal with tensor parameters: standard normal draws, scaled and shifted
at::Tensor normal_draw(at::IntArrayRef shape, const at::Tensor& like, c10::optional<at::Generator> gen) {
    if (!is_hot_float(like.scalar_type())) TVK_NOT_IMPLEMENTED("normal for dtype ", like.scalar_type());
    return at::empty(shape, like.options()).normal_(0.0, 1.0, gen);
}
at::Tensor normal_tensor_float(const at::Tensor& mean, double std, c10::optional<at::Generator> gen) {
    TORCH_CHECK(std >= 0.0, "normal expects std >= 0.0, but found std ", std);
    return normal_draw(mean.sizes(), mean, gen) * std + mean;
}
at::Tensor normal_float_tensor(double mean, const at::Tensor& std, c10::optional<at::Generator> gen) { return normal_draw(std.sizes(), std, gen) * std + mean; }
at::Tensor normal_tensor_tensor(const at::Tensor& mean, const at::Tensor& std, c10::optional<at::Generator> gen) {
    return normal_draw(at::infer_size(mean.sizes(), std.sizes()), mean, gen) * std + mean;
}

// membership test by comparing every element with every candidate (candidates are expected to be few)
at::Tensor isin_tensors(const at::Tensor& elements, const at::Tensor& test_elements, bool, bool invert) {
    TORCH_CHECK(elements.numel() * std::max<int64_t>(test_elements.numel(), 1) <= (int64_t{1} << 30), "torchvulkan [NOT IMPLEMENTED]: isin over more than 2^30 comparisons");
    at::Tensor tests = is_vulkan(test_elements) ? test_elements : test_elements.to(elements.device());
    at::Tensor elems = is_vulkan(elements) ? elements : elements.to(tests.device());
    at::Tensor found = tests.numel() == 0 ? at::zeros(elems.sizes(), elems.options().dtype(at::kBool))
                                          : at::any(at::eq(elems.contiguous().unsqueeze(-1), tests.contiguous().reshape({-1})), -1, false);
    return invert ? at::logical_not(found) : found;
}
at::Tensor isin_tensor_scalar(const at::Tensor& elements, const at::Scalar& test, bool, bool invert) { return invert ? at::ne(elements, test) : at::eq(elements, test); }
at::Tensor isin_scalar_tensor(const at::Scalar& element, const at::Tensor& tests, bool assume_unique, bool invert) {
    return isin_tensors(at::full({}, element, tests.options()), tests, assume_unique, invert);
}

at::Tensor nansum(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, c10::optional<at::ScalarType> dtype) {
    return at::sum(at::where(at::isnan(self), at::zeros({}, self.options()), self), dim, keepdim, dtype);
}
// logit(x) = log(x / (1 - x)), x clamped to [eps, 1 - eps] when eps is given
at::Tensor logit(const at::Tensor& self, c10::optional<double> eps) {
    at::Tensor x = eps.has_value() ? at::clamp(self, *eps, 1.0 - *eps) : self;
    return at::log(x / (1.0 - x));
}
at::Tensor logit_backward(const at::Tensor& grad, const at::Tensor& self, c10::optional<double> eps) {
    const double lo = eps.value_or(0.0), hi = 1.0 - lo;
    at::Tensor outside = at::logical_or(at::lt(self, lo), at::gt(self, hi));
    at::Tensor fill = at::full({}, eps.has_value() ? 0.0 : std::numeric_limits<double>::quiet_NaN(), grad.options());
    return at::where(outside, fill, grad / (self * (1.0 - self)));
}
std::tuple<at::Tensor, at::Tensor> aminmax(const at::Tensor& self, c10::optional<int64_t> dim, bool keepdim) {
    if (dim.has_value()) return {at::amin(self, {*dim}, keepdim), at::amax(self, {*dim}, keepdim)};
    TORCH_CHECK(self.numel() > 0, "aminmax(): cannot compute aminmax over an empty dimension as the operation has no identity.");
    at::Tensor flat = self.reshape({-1});
    at::Tensor lo = at::amin(flat, {0}, false), hi = at::amax(flat, {0}, false);
    if (!keepdim) return {lo, hi};
    std::vector<int64_t> ones(self.dim(), 1);
    return {lo.reshape(ones), hi.reshape(ones)};
}
// channel i of group j moves to position i * groups + j
at::Tensor channel_shuffle(const at::Tensor& self, c10::SymInt groups_sym) {
    const int64_t groups = groups_sym.guard_int(__FILE__, __LINE__);
    TORCH_CHECK(self.dim() > 2, "channel_shuffle expects input with > 2 dims, but got input with sizes ", self.sizes());
    const int64_t c = self.size(1);
    TORCH_CHECK(groups > 0 && c % groups == 0, "Number of groups to divide channels in must be positive and divide the number of channels; got ", groups, " for ", c, " channels");
    if (self.numel() == 0) return self.clone();
    return self.contiguous().reshape({self.size(0), groups, c / groups, -1}).transpose(1, 2).contiguous().reshape(self.sizes());
}
// repeat_interleave of a vector of counts: output position p belongs to the first entry whose running total exceeds p
at::Tensor repeat_interleave_counts(const at::Tensor& repeats, c10::optional<c10::SymInt> output_size) {
    TORCH_CHECK(repeats.dim() == 1 && (repeats.scalar_type() == at::kLong || repeats.scalar_type() == at::kInt), "repeat_interleave only accept 1D vector of int or long as repeat");
    if (repeats.numel() == 0) return at::empty({0}, repeats.options().dtype(at::kLong));
    TORCH_CHECK(repeats.numel() <= (int64_t{1} << 24), "torchvulkan [NOT IMPLEMENTED]: repeat_interleave of more than 2^24 counts");
    at::Tensor totals = at::cumsum(repeats.to(at::kFloat), 0);
    const int64_t n = output_size.has_value() ? output_size->guard_int(__FILE__, __LINE__) : static_cast<int64_t>(totals.narrow(0, repeats.numel() - 1, 1).item<float>());
    TORCH_CHECK(n < (int64_t{1} << 24), "torchvulkan [NOT IMPLEMENTED]: repeat_interleave to 2^24 elements or more");
    at::Tensor positions = at::arange(n, at::TensorOptions().dtype(at::kFloat).device(at::kCPU)).to(repeats.device());
    return at::searchsorted(totals, positions, false, true);
}
// max_unpool2d: every pooled value goes back to the flat position its index names, zeros elsewhere
at::Tensor max_unpool2d(const at::Tensor& self, const at::Tensor& indices, at::IntArrayRef output_size) {
    TORCH_CHECK(output_size.size() == 2, "There should be exactly two elements (height, width) in output_size");
    TORCH_CHECK((self.dim() == 3 || self.dim() == 4) && self.sizes() == indices.sizes(), "max_unpool2d: expected a 3-D or 4-D input and indices of its shape");
    TORCH_CHECK(indices.scalar_type() == at::kLong, "elements in indices should be type int64");
    const int64_t planes = self.numel() ? self.numel() / (self.size(-2) * self.size(-1)) : 0;
    std::vector<int64_t> shape(self.sizes().begin(), self.sizes().end() - 2);
    shape.insert(shape.end(), {output_size[0], output_size[1]});
    if (planes == 0) return at::zeros(shape, self.options());
    at::Tensor zero = at::zeros({planes, output_size[0] * output_size[1]}, self.options());
    return at::scatter_add(zero, 1, indices.contiguous().reshape({planes, -1}), self.contiguous().reshape({planes, -1})).reshape(shape);
}

// prelu with its weight already broadcast to the input (ATen reshapes it before calling the kernel)
at::Tensor prelu_kernel(const at::Tensor& self, const at::Tensor& weight) { return at::where(at::gt(self, 0), self, weight * self); }
std::tuple<at::Tensor, at::Tensor> prelu_kernel_backward(const at::Tensor& grad, const at::Tensor& self, const at::Tensor& weight) {
    at::Tensor pos = at::gt(self, 0), zero = at::zeros({}, grad.options());
    return {at::where(pos, grad, weight * grad), at::where(pos, zero, self * grad)};
}
// glu(x) = a * sigmoid(b) over the two halves of dim
at::Tensor glu(const at::Tensor& self, int64_t dim) {
    dim = at::maybe_wrap_dim(dim, self.dim());
    TORCH_CHECK(self.size(dim) % 2 == 0, "Halving dimension must be even, but dimension ", dim, " is size ", self.size(dim));
    const int64_t h = self.size(dim) / 2;
    return self.narrow(dim, 0, h) * at::sigmoid(self.narrow(dim, h, h));
}
at::Tensor glu_backward(const at::Tensor& grad, const at::Tensor& self, int64_t dim) {
    dim = at::maybe_wrap_dim(dim, self.dim());
    const int64_t h = self.size(dim) / 2;
    at::Tensor a = self.narrow(dim, 0, h), sg = at::sigmoid(self.narrow(dim, h, h));
    return at::cat({grad * sg, grad * a * sg * (1.0 - sg)}, dim);
}

// the norm family of torch.norm / F.pairwise_distance: the vector norm over the given dimensions
at::Tensor norm_dim(const at::Tensor& self, const c10::optional<at::Scalar>& p, at::IntArrayRef dim, bool keepdim) {
    return vector_norm(self, p.value_or(2.0), dim, keepdim, c10::nullopt);
}
at::Tensor norm_dim_dtype(const at::Tensor& self, const c10::optional<at::Scalar>& p, at::IntArrayRef dim, bool keepdim, at::ScalarType dtype) {
    return vector_norm(self, p.value_or(2.0), dim, keepdim, dtype);
}
at::Tensor norm_scalar(const at::Tensor& self, const at::Scalar& p) { return vector_norm(self, p, c10::nullopt, false, c10::nullopt); }
at::Tensor norm_dtype(const at::Tensor& self, const c10::optional<at::Scalar>& p, at::ScalarType dtype) { return vector_norm(self, p.value_or(2.0), c10::nullopt, false, dtype); }
at::Tensor& norm_out(const at::Tensor& self, const c10::optional<at::Scalar>& p, at::IntArrayRef dim, bool keepdim, at::Tensor& out) {
    return into(out, norm_dim(self, p, dim, keepdim));
}
at::Tensor& norm_dtype_out(const at::Tensor& self, const c10::optional<at::Scalar>& p, at::IntArrayRef dim, bool keepdim, at::ScalarType dtype, at::Tensor& out) {
    return into(out, norm_dim_dtype(self, p, dim, keepdim, dtype));
}

// ---- nearest and bilinear 2-D upsampling ---------------------------------------------------------------------------
// Both are separable: rows of the output are rows of the input picked (nearest) or blended (bilinear) by per-axis index
// and weight vectors, which are computed on the host (a few hundred numbers) exactly as ATen computes them, and applied
// with index_select and lerp on the device; the gradients are the adjoints (index_add) of the same selections.
struct AxisMap {
    at::Tensor i0, i1, w1;      // source indices and the weight of i1 (bilinear); nearest uses i0 only
};
double area_scale(int64_t in, int64_t out, bool align_corners, const c10::optional<double>& scale) {
    if (align_corners) return out > 1 ? (double)(in - 1) / (double)(out - 1) : 0.0;
    return (scale.has_value() && *scale > 0) ? 1.0 / *scale : (double)in / (double)out;
}
AxisMap nearest_axis(int64_t in, int64_t out, const c10::optional<double>& scale, const at::Device& dev) {
    const float s = (float)((scale.has_value() && *scale > 0) ? 1.0 / *scale : (double)in / (double)out);
    std::vector<int64_t> idx(out);
    for (int64_t o = 0; o < out; ++o) idx[o] = std::min<int64_t>((int64_t)std::floor((float)o * s), in - 1);
    AxisMap m;
    m.i0 = at::tensor(idx, at::TensorOptions().dtype(at::kLong)).to(dev);
    return m;
}
AxisMap bilinear_axis(int64_t in, int64_t out, bool align_corners, const c10::optional<double>& scale, const at::Device& dev) {
    const float s = (float)area_scale(in, out, align_corners, scale);
    std::vector<int64_t> i0(out), i1(out);
    std::vector<float> w(out);
    for (int64_t o = 0; o < out; ++o) {
        float src = align_corners ? s * (float)o : std::max(s * ((float)o + 0.5f) - 0.5f, 0.0f);
        int64_t lo = std::min<int64_t>((int64_t)src, in - 1);
        i0[o] = lo;
        i1[o] = std::min<int64_t>(lo + 1, in - 1);
        w[o] = std::min(std::max(src - (float)lo, 0.0f), 1.0f);
    }
    AxisMap m;
    m.i0 = at::tensor(i0, at::TensorOptions().dtype(at::kLong)).to(dev);
    m.i1 = at::tensor(i1, at::TensorOptions().dtype(at::kLong)).to(dev);
    m.w1 = at::tensor(w, at::TensorOptions().dtype(at::kFloat)).to(dev);
    return m;
}
at::Tensor upsample_nearest2d(const at::Tensor& self, at::IntArrayRef size, c10::optional<double> sh, c10::optional<double> sw) {
    TORCH_CHECK(self.dim() == 4 && size.size() == 2, "upsample_nearest2d: expected a 4-D input and two output sizes");
    const AxisMap h = nearest_axis(self.size(2), size[0], sh, self.device()), w = nearest_axis(self.size(3), size[1], sw, self.device());
    return at::index_select(at::index_select(self, 2, h.i0), 3, w.i0);
}
at::Tensor upsample_nearest2d_backward(const at::Tensor& grad, at::IntArrayRef size, at::IntArrayRef input_size, c10::optional<double> sh, c10::optional<double> sw) {
    const AxisMap h = nearest_axis(input_size[2], size[0], sh, grad.device()), w = nearest_axis(input_size[3], size[1], sw, grad.device());
    at::Tensor gw = at::zeros({grad.size(0), grad.size(1), grad.size(2), input_size[3]}, grad.options()).index_add(3, w.i0, grad);
    return at::zeros({grad.size(0), grad.size(1), input_size[2], input_size[3]}, grad.options()).index_add(2, h.i0, gw);
}
at::Tensor blend_axis(const at::Tensor& x, int64_t dim, const AxisMap& m) {
    std::vector<int64_t> view(x.dim(), 1);
    view[dim] = m.w1.numel();
    at::Tensor w = m.w1.to(x.scalar_type()).view(view);
    at::Tensor a = at::index_select(x, dim, m.i0), b = at::index_select(x, dim, m.i1);
    return a + (b - a) * w;
}
at::Tensor blend_axis_backward(const at::Tensor& g, int64_t dim, const AxisMap& m, int64_t in) {
    std::vector<int64_t> view(g.dim(), 1), shape(g.sizes().begin(), g.sizes().end());
    view[dim] = m.w1.numel();
    shape[dim] = in;
    at::Tensor w = m.w1.to(g.scalar_type()).view(view);
    return at::zeros(shape, g.options()).index_add(dim, m.i0, g * (1.0 - w)).index_add(dim, m.i1, g * w);
}
at::Tensor upsample_bilinear2d(const at::Tensor& self, at::IntArrayRef size, bool align_corners, c10::optional<double> sh, c10::optional<double> sw) {
    TORCH_CHECK(self.dim() == 4 && size.size() == 2, "upsample_bilinear2d: expected a 4-D input and two output sizes");
    const AxisMap h = bilinear_axis(self.size(2), size[0], align_corners, sh, self.device()), w = bilinear_axis(self.size(3), size[1], align_corners, sw, self.device());
    return blend_axis(blend_axis(self, 2, h), 3, w);
}
at::Tensor upsample_bilinear2d_backward(const at::Tensor& grad, at::IntArrayRef size, at::IntArrayRef input_size, bool align_corners, c10::optional<double> sh,
                                        c10::optional<double> sw) {
    const AxisMap h = bilinear_axis(input_size[2], size[0], align_corners, sh, grad.device()), w = bilinear_axis(input_size[3], size[1], align_corners, sw, grad.device());
    return blend_axis_backward(blend_axis_backward(grad, 3, w, input_size[3]), 2, h, input_size[2]);
}

// Bicubic upsampling is separable as well: four taps per axis around floor(source position), indices clamped to the
// edge, weights from the cubic convolution kernel with A = -0.75 evaluated in fp32 on the host as ATen evaluates them.
struct CubicAxis {
    at::Tensor index[4], weight[4];
};
CubicAxis cubic_axis(int64_t in, int64_t out, bool align_corners, const c10::optional<double>& scale, const at::Device& dev) {
    const float s = (float)area_scale(in, out, align_corners, scale), A = -0.75f;
    auto near = [A](float x) { return ((A + 2.f) * x - (A + 3.f)) * x * x + 1.f; };                 // |x| <= 1
    auto far = [A](float x) { return ((A * x - 5.f * A) * x + 8.f * A) * x - 4.f * A; };            // 1 < |x| < 2
    std::vector<int64_t> idx[4];
    std::vector<float> w[4];
    for (int64_t o = 0; o < out; ++o) {
        const float real = align_corners ? s * (float)o : s * ((float)o + 0.5f) - 0.5f;
        const float fl = std::floor(real), t = real - fl;
        const int64_t base = (int64_t)fl;
        const float ws[4] = {far(t + 1.f), near(t), near(1.f - t), far(2.f - t)};
        for (int k = 0; k < 4; ++k) {
            idx[k].push_back(std::min<int64_t>(std::max<int64_t>(base - 1 + k, 0), in - 1));
            w[k].push_back(ws[k]);
        }
    }
    CubicAxis m;
    for (int k = 0; k < 4; ++k) {
        m.index[k] = at::tensor(idx[k], at::TensorOptions().dtype(at::kLong)).to(dev);
        m.weight[k] = at::tensor(w[k], at::TensorOptions().dtype(at::kFloat)).to(dev);
    }
    return m;
}
at::Tensor cubic_blend(const at::Tensor& x, int64_t dim, const CubicAxis& m) {
    std::vector<int64_t> view(x.dim(), 1);
    view[dim] = m.weight[0].numel();
    at::Tensor r;
    for (int k = 0; k < 4; ++k) {
        at::Tensor term = at::index_select(x, dim, m.index[k]) * m.weight[k].to(x.scalar_type()).view(view);
        r = r.defined() ? r + term : term;
    }
    return r;
}
at::Tensor cubic_blend_backward(const at::Tensor& g, int64_t dim, const CubicAxis& m, int64_t in) {
    std::vector<int64_t> view(g.dim(), 1), shape(g.sizes().begin(), g.sizes().end());
    view[dim] = m.weight[0].numel();
    shape[dim] = in;
    at::Tensor r = at::zeros(shape, g.options());
    for (int k = 0; k < 4; ++k) r = r.index_add(dim, m.index[k], g * m.weight[k].to(g.scalar_type()).view(view));
    return r;
}
at::Tensor upsample_bicubic2d(const at::Tensor& self, at::IntArrayRef size, bool align_corners, c10::optional<double> sh, c10::optional<double> sw) {
    TORCH_CHECK(self.dim() == 4 && size.size() == 2, "upsample_bicubic2d: expected a 4-D input and two output sizes");
    TORCH_CHECK(self.size(2) > 0 && self.size(3) > 0 && size[0] > 0 && size[1] > 0, "upsample_bicubic2d: input and output sizes should be greater than 0");
    return cubic_blend(cubic_blend(self, 2, cubic_axis(self.size(2), size[0], align_corners, sh, self.device())), 3,
                       cubic_axis(self.size(3), size[1], align_corners, sw, self.device()));
}
at::Tensor upsample_bicubic2d_backward(const at::Tensor& grad, at::IntArrayRef size, at::IntArrayRef input_size, bool align_corners, c10::optional<double> sh,
                                       c10::optional<double> sw) {
    at::Tensor gw = cubic_blend_backward(grad, 3, cubic_axis(input_size[3], size[1], align_corners, sw, grad.device()), input_size[3]);
    return cubic_blend_backward(gw, 2, cubic_axis(input_size[2], size[0], align_corners, sh, grad.device()), input_size[2]);
}

// nan_to_num: NaN -> nan (0), +inf -> posinf (the dtype's largest value), -inf -> neginf (its lowest)
at::Tensor vk_nan_to_num(const at::Tensor& self, c10::optional<double> nan, c10::optional<double> posinf, c10::optional<double> neginf) {
    TORCH_CHECK(is_hot_float(self.scalar_type()), "torchvulkan [NOT IMPLEMENTED]: nan_to_num for ", self.scalar_type());
    const double top = self.scalar_type() == at::kHalf ? 65504.0 : (self.scalar_type() == at::kBFloat16 ? 3.3895313892515355e38 : 3.4028234663852886e38);
    auto constant = [&](double v) { at::Tensor t = at::empty({}, self.options()); t.fill_(v); return t; };
    at::Tensor r = at::where(at::isnan(self), constant(nan.value_or(0.0)), self);
    r = at::where(at::eq(self, std::numeric_limits<double>::infinity()), constant(posinf.value_or(top)), r);
    return at::where(at::eq(self, -std::numeric_limits<double>::infinity()), constant(neginf.value_or(-top)), r);
}
at::Tensor& nan_to_num_out(const at::Tensor& self, c10::optional<double> nan, c10::optional<double> posinf, c10::optional<double> neginf, at::Tensor& out) {
    return into(out, vk_nan_to_num(self, nan, posinf, neginf));
}
at::Tensor& nan_to_num_(at::Tensor& self, c10::optional<double> nan, c10::optional<double> posinf, c10::optional<double> neginf) {
    self.copy_(vk_nan_to_num(self, nan, posinf, neginf));
    return self;
}
at::Tensor count_nonzero(const at::Tensor& self, at::IntArrayRef dims) {
    at::Tensor nz = self.scalar_type() == at::kBool ? self : at::ne(self, 0);
    return dims.empty() ? nz.sum() : nz.sum(dims);
}
// softshrink(x) = x > l ? x - l : x < -l ? x + l : 0
at::Tensor softshrink(const at::Tensor& self, const at::Scalar& lambd) {
    at::Tensor zero = at::zeros({}, self.options());
    return at::where(at::gt(self, lambd), self - lambd, at::where(at::lt(self, -lambd.toDouble()), self + lambd, zero));
}
at::Tensor softshrink_backward(const at::Tensor& grad, const at::Tensor& self, const at::Scalar& lambd) {
    return at::where(at::gt(at::abs(self), lambd), grad, at::zeros({}, grad.options()));
}
// index_fill: the slices named by index along dim take one value
at::Tensor& index_fill_scalar_(at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Scalar& value) {
    dim = at::maybe_wrap_dim(dim, std::max<int64_t>(self.dim(), 1));
    TORCH_CHECK(self.dim() > 0 && index.dim() <= 1, "index_fill_(): expected a tensor with dimensions and a vector of indices");
    if (index.numel() == 0) return self;
    at::Tensor hits = at::zeros({self.size(dim)}, self.options().dtype(at::kFloat)).index_add(0, index.reshape({-1}), at::ones({index.numel()}, self.options().dtype(at::kFloat)));
    std::vector<int64_t> view(self.dim(), 1);
    view[dim] = self.size(dim);
    self.masked_fill_(at::gt(hits, 0).view(view), value);
    return self;
}

// ---- the 1-D and 3-D forms, and "nearest-exact": the same per-axis selections over one or three spatial axes ------------------------
// exact: ATen's nearest-exact rounds at pixel centres, floor((o + 0.5) * scale)
AxisMap nearest_axis_any(int64_t in, int64_t out, const c10::optional<double>& scale, bool exact, const at::Device& dev) {
    if (!exact) return nearest_axis(in, out, scale, dev);
    const float s = (float)((scale.has_value() && *scale > 0) ? 1.0 / *scale : (double)in / (double)out);
    std::vector<int64_t> idx(out);
    for (int64_t o = 0; o < out; ++o) idx[o] = std::min<int64_t>((int64_t)std::floor(((float)o + 0.5f) * s), in - 1);
    AxisMap m;
    m.i0 = at::tensor(idx, at::TensorOptions().dtype(at::kLong)).to(dev);
    return m;
}
at::Tensor nearest_nd(const at::Tensor& self, at::IntArrayRef size, std::initializer_list<c10::optional<double>> scales, bool exact) {
    const int64_t nsp = (int64_t)size.size();
    TORCH_CHECK(self.dim() == nsp + 2, "upsample_nearest: expected a ", nsp + 2, "-D input");
    at::Tensor r = self;
    int64_t a = 0;
    for (const auto& sc : scales) { r = at::index_select(r, 2 + a, nearest_axis_any(self.size(2 + a), size[a], sc, exact, self.device()).i0); ++a; }
    return r;
}
at::Tensor nearest_nd_backward(const at::Tensor& grad, at::IntArrayRef size, at::IntArrayRef input_size, std::initializer_list<c10::optional<double>> scales, bool exact) {
    at::Tensor g = grad;
    int64_t a = 0;
    for (const auto& sc : scales) {
        std::vector<int64_t> shape(g.sizes().begin(), g.sizes().end());
        shape[2 + a] = input_size[2 + a];
        g = at::zeros(shape, g.options()).index_add(2 + a, nearest_axis_any(input_size[2 + a], size[a], sc, exact, grad.device()).i0, g);
        ++a;
    }
    return g;
}
at::Tensor linear_nd(const at::Tensor& self, at::IntArrayRef size, bool align_corners, std::initializer_list<c10::optional<double>> scales) {
    const int64_t nsp = (int64_t)size.size();
    TORCH_CHECK(self.dim() == nsp + 2, "upsample_linear: expected a ", nsp + 2, "-D input");
    at::Tensor r = self;
    int64_t a = 0;
    for (const auto& sc : scales) { r = blend_axis(r, 2 + a, bilinear_axis(self.size(2 + a), size[a], align_corners, sc, self.device())); ++a; }
    return r;
}
at::Tensor linear_nd_backward(const at::Tensor& grad, at::IntArrayRef size, at::IntArrayRef input_size, bool align_corners, std::initializer_list<c10::optional<double>> scales) {
    at::Tensor g = grad;
    int64_t a = 0;
    for (const auto& sc : scales) { g = blend_axis_backward(g, 2 + a, bilinear_axis(input_size[2 + a], size[a], align_corners, sc, grad.device()), input_size[2 + a]); ++a; }
    return g;
}
using OptD = c10::optional<double>;
at::Tensor up_nearest1d(const at::Tensor& x, at::IntArrayRef size, OptD s) { return nearest_nd(x, size, {s}, false); }
at::Tensor up_nearest1d_bw(const at::Tensor& g, at::IntArrayRef size, at::IntArrayRef in, OptD s) { return nearest_nd_backward(g, size, in, {s}, false); }
at::Tensor up_nearest3d(const at::Tensor& x, at::IntArrayRef size, OptD sd, OptD sh, OptD sw) { return nearest_nd(x, size, {sd, sh, sw}, false); }
at::Tensor up_nearest3d_bw(const at::Tensor& g, at::IntArrayRef size, at::IntArrayRef in, OptD sd, OptD sh, OptD sw) { return nearest_nd_backward(g, size, in, {sd, sh, sw}, false); }
at::Tensor up_exact1d(const at::Tensor& x, at::IntArrayRef size, OptD s) { return nearest_nd(x, size, {s}, true); }
at::Tensor up_exact1d_bw(const at::Tensor& g, at::IntArrayRef size, at::IntArrayRef in, OptD s) { return nearest_nd_backward(g, size, in, {s}, true); }
at::Tensor up_exact2d(const at::Tensor& x, at::IntArrayRef size, OptD sh, OptD sw) { return nearest_nd(x, size, {sh, sw}, true); }
at::Tensor up_exact2d_bw(const at::Tensor& g, at::IntArrayRef size, at::IntArrayRef in, OptD sh, OptD sw) { return nearest_nd_backward(g, size, in, {sh, sw}, true); }
at::Tensor up_exact3d(const at::Tensor& x, at::IntArrayRef size, OptD sd, OptD sh, OptD sw) { return nearest_nd(x, size, {sd, sh, sw}, true); }
at::Tensor up_exact3d_bw(const at::Tensor& g, at::IntArrayRef size, at::IntArrayRef in, OptD sd, OptD sh, OptD sw) { return nearest_nd_backward(g, size, in, {sd, sh, sw}, true); }
at::Tensor up_linear1d(const at::Tensor& x, at::IntArrayRef size, bool ac, OptD s) { return linear_nd(x, size, ac, {s}); }
at::Tensor up_linear1d_bw(const at::Tensor& g, at::IntArrayRef size, at::IntArrayRef in, bool ac, OptD s) { return linear_nd_backward(g, size, in, ac, {s}); }
at::Tensor up_trilinear3d(const at::Tensor& x, at::IntArrayRef size, bool ac, OptD sd, OptD sh, OptD sw) { return linear_nd(x, size, ac, {sd, sh, sw}); }
at::Tensor up_trilinear3d_bw(const at::Tensor& g, at::IntArrayRef size, at::IntArrayRef in, bool ac, OptD sd, OptD sh, OptD sw) {
    return linear_nd_backward(g, size, in, ac, {sd, sh, sw});
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("upsample_nearest1d", &up_nearest1d);
    m.impl("upsample_nearest1d_backward", &up_nearest1d_bw);
    m.impl("upsample_nearest3d", &up_nearest3d);
    m.impl("upsample_nearest3d_backward", &up_nearest3d_bw);
    m.impl("_upsample_nearest_exact1d", &up_exact1d);
    m.impl("_upsample_nearest_exact1d_backward", &up_exact1d_bw);
    m.impl("_upsample_nearest_exact2d", &up_exact2d);
    m.impl("_upsample_nearest_exact2d_backward", &up_exact2d_bw);
    m.impl("_upsample_nearest_exact3d", &up_exact3d);
    m.impl("_upsample_nearest_exact3d_backward", &up_exact3d_bw);
    m.impl("upsample_linear1d", &up_linear1d);
    m.impl("upsample_linear1d_backward", &up_linear1d_bw);
    m.impl("upsample_trilinear3d", &up_trilinear3d);
    m.impl("upsample_trilinear3d_backward", &up_trilinear3d_bw);
    m.impl("nan_to_num", &vk_nan_to_num);
    m.impl("nan_to_num.out", &nan_to_num_out);
    m.impl("nan_to_num_", &nan_to_num_);
    m.impl("count_nonzero.dim_IntList", &count_nonzero);
    m.impl("softshrink", &softshrink);
    m.impl("softshrink_backward", &softshrink_backward);
    m.impl("index_fill_.int_Scalar", &index_fill_scalar_);
    m.impl("binary_cross_entropy", &bce);
    m.impl("binary_cross_entropy_backward", &bce_backward);
    m.impl("upsample_bicubic2d", &upsample_bicubic2d);
    m.impl("upsample_bicubic2d_backward", &upsample_bicubic2d_backward);
    m.impl("_adaptive_avg_pool3d", &adaptive_avg_pool3d);
    m.impl("_adaptive_avg_pool3d_backward", &adaptive_avg_pool3d_backward);
    m.impl("pow.Scalar", &pow_scalar);
    m.impl("normal.Tensor_float", &normal_tensor_float);
    m.impl("normal.float_Tensor", &normal_float_tensor);
    m.impl("normal.Tensor_Tensor", &normal_tensor_tensor);
    m.impl("isin.Tensor_Tensor", &isin_tensors);
    m.impl("isin.Tensor_Scalar", &isin_tensor_scalar);
    m.impl("isin.Scalar_Tensor", &isin_scalar_tensor);
    m.impl("nansum", &nansum);
    m.impl("logit", &logit);
    m.impl("logit_backward", &logit_backward);
    m.impl("aminmax", &aminmax);
    m.impl("channel_shuffle", &channel_shuffle);
    m.impl("repeat_interleave.Tensor", &repeat_interleave_counts);
    m.impl("max_unpool2d", &max_unpool2d);
    m.impl("linalg_cross", &vk_linalg_cross);
    m.impl("linalg_cross.out", &vk_linalg_cross_out);
    m.impl("_unique2", &unique2);
    m.impl("bincount", &bincount);
    m.impl("_cummax_helper", &cummax_helper);
    m.impl("_cummin_helper", &cummin_helper);
    m.impl("_adaptive_avg_pool2d", &adaptive_avg_pool2d);
    m.impl("_adaptive_avg_pool2d_backward", &adaptive_avg_pool2d_backward);
    m.impl("adaptive_max_pool2d", &adaptive_max_pool2d);
    m.impl("adaptive_max_pool2d_backward", &adaptive_max_pool2d_backward);
    m.impl("_prelu_kernel", &prelu_kernel);
    m.impl("_prelu_kernel_backward", &prelu_kernel_backward);
    m.impl("glu", &glu);
    m.impl("glu_backward", &glu_backward);
    m.impl("norm.ScalarOpt_dim", &norm_dim);
    m.impl("norm.ScalarOpt_dim_dtype", &norm_dim_dtype);
    m.impl("norm.Scalar", &norm_scalar);
    m.impl("norm.ScalarOpt_dtype", &norm_dtype);
    m.impl("norm.out", &norm_out);
    m.impl("norm.dtype_out", &norm_dtype_out);
    m.impl("upsample_nearest2d", &upsample_nearest2d);
    m.impl("upsample_nearest2d_backward", &upsample_nearest2d_backward);
    m.impl("upsample_bilinear2d", &upsample_bilinear2d);
    m.impl("upsample_bilinear2d_backward", &upsample_bilinear2d_backward);
    m.impl("smooth_l1_loss", &smooth_l1_loss);
    m.impl("smooth_l1_loss_backward", &smooth_l1_loss_backward);
    m.impl("huber_loss", &huber_loss);
    m.impl("huber_loss_backward", &huber_loss_backward);
    m.impl("xlogy.Tensor", &vk_xlogy);
    m.impl("xlogy.OutTensor", &xlogy_out);
    m.impl("max", &max_all);
    m.impl("min", &min_all);
    m.impl("max.unary_out", &max_unary_out);
    m.impl("min.unary_out", &min_unary_out);
    m.impl("max.dim", &max_dim);
    m.impl("min.dim", &min_dim);
    m.impl("max.dim_max", &max_dim_out);
    m.impl("min.dim_min", &min_dim_out);
    m.impl("all", &all_full);
    m.impl("any", &any_full);
    m.impl("all.dim", &all_dim);
    m.impl("any.dim", &any_dim);
    m.impl("all.dims", &all_dims_fn);
    m.impl("any.dims", &any_dims_fn);
    m.impl("all.all_out", &all_all_out);
    m.impl("any.all_out", &any_all_out);
    m.impl("all.out", &all_out);
    m.impl("any.out", &any_out);
    m.impl("all.dims_out", &all_dims_out);
    m.impl("any.dims_out", &any_dims_out);
    m.impl("var.correction", &var_correction);
    m.impl("std.correction", &std_correction);
    m.impl("var_mean.correction", &var_mean_correction);
    m.impl("std_mean.correction", &std_mean_correction);
    m.impl("linalg_vector_norm", &vector_norm);
    m.impl("linalg_vector_norm.out", &vector_norm_out);
    m.impl("masked_fill_.Scalar", &masked_fill_scalar_);
    m.impl("masked_fill_.Tensor", &masked_fill_tensor_);
    m.impl("tril", &tril);
    m.impl("triu", &triu);
    m.impl("tril_", &tril_);
    m.impl("triu_", &triu_);
    m.impl("tril.out", &tril_out);
    m.impl("triu.out", &triu_out);
    m.impl("arange.start_out", &arange_out);
    m.impl("linspace.out", &linspace_out);
    m.impl("eye.m_out", &eye_m_out);
    m.impl("eye.out", &eye_out);
    m.impl("mse_loss", &mse_loss);
    m.impl("mse_loss_backward", &mse_loss_backward);
}

}  // namespace tvk_aten
