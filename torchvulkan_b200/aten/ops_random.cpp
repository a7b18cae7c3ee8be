// Random fills and dropout on the "vulkan" device.
//
// Counterparts in the reference: uniform_ / normal_ / bernoulli_ (src/api/ops/random.cpp), native_dropout and its backward
// (src/api/ops/dropout.cpp:10-120). Every launch reserves its offsets from the device's generator state
// (tvk_rng_reserve; torch.manual_seed and torchvulkan.manual_seed reach tvk_rng_set_seed through the generator), so the
// same seed replays the same stream. torch.randn / rand / rand_like / dropout / nn.init.* are composites over these.
// A generator object passed by the caller shares the state of its device.
#include "common.h"

namespace tvk_aten {
namespace {

enum { kUniform = 0, kNormal = 1, kBernoulli = 2 };

at::Tensor& random_fill_(at::Tensor& self, int kind, double a, double b, const char* name) {
    const at::ScalarType st = self.scalar_type();
    const bool mask = st == at::kBool || st == at::kByte;
    if (!is_hot_float(st) && !(mask && kind == kBernoulli)) TVK_NOT_IMPLEMENTED(name, " for dtype ", st, " on the vulkan device");
    if (self.numel() == 0) return self;
    at::Tensor target = self.is_non_overlapping_and_dense() ? self : empty_vulkan(self.sizes(), st, self.device());
    DeviceScope scope(self);
    uint64_t seed = 0, offset = 0;
    const uint64_t* state = nullptr;      // non-null inside a graph capture: the replay's generator state lives on the device
    TVK_CALL(tvk_rng_reserve_state(scope.device, (uint64_t)((target.numel() + 3) / 4), &seed, &offset, &state));
    TVK_CALL(tvk_random_fill(kind, to_tvk_dtype(st), target.data_ptr(), target.numel(), a, b, seed, offset, state, scope.stream));
    if (!target.is_same(self)) self.copy_(target);
    return self;
}
at::Tensor& uniform_(at::Tensor& self, double from, double to, c10::optional<at::Generator>) {
    TORCH_CHECK(from <= to, "uniform_ expects to return a [from, to) range, but found from=", from, " > to=", to);
    return random_fill_(self, kUniform, from, to, "uniform_");
}
at::Tensor& normal_(at::Tensor& self, double mean, double std, c10::optional<at::Generator>) {
    TORCH_CHECK(std >= 0.0, "normal expects std >= 0.0, but found std ", std);
    return random_fill_(self, kNormal, mean, std, "normal_");
}
at::Tensor& bernoulli_float_(at::Tensor& self, double p, c10::optional<at::Generator>) {
    TORCH_CHECK(p >= 0.0 && p <= 1.0, "bernoulli_ expects p to be in [0, 1], but got p=", p);
    return random_fill_(self, kBernoulli, p, 0.0, "bernoulli_");
}
at::Tensor bernoulli_p(const at::Tensor& self, double p, c10::optional<at::Generator> gen) {
    at::Tensor out = at::empty_like(self);
    return bernoulli_float_(out, p, gen);
}

std::tuple<at::Tensor, at::Tensor> native_dropout(const at::Tensor& input, double p, c10::optional<bool> train) {
    if (input.numel() == 0) return {input, at::empty_like(input, input.options().dtype(at::kBool))};
    if (train.has_value() && !*train) {
        at::Tensor ones = at::empty_like(input, input.options().dtype(at::kBool));
        ones.fill_(true);
        return {input.clone(), ones};
    }
    TORCH_CHECK(p >= 0.0 && p <= 1.0, "dropout probability has to be between 0 and 1, but got ", p);
    if (!is_hot_float(input.scalar_type())) TVK_NOT_IMPLEMENTED("dropout for dtype ", input.scalar_type(), " on the vulkan device");
    // elementwise: any dense layout runs as it is, and the outputs keep it
    at::Tensor src = input.is_non_overlapping_and_dense() ? input : contiguous_vulkan(input);
    at::Tensor out = at::empty_strided(src.sizes(), src.strides(), src.options());
    at::Tensor mask = at::empty_strided(src.sizes(), src.strides(), src.options().dtype(at::kBool));
    DeviceScope scope(src);
    uint64_t seed = 0, offset = 0;
    const uint64_t* state = nullptr;
    TVK_CALL(tvk_rng_reserve_state(scope.device, (uint64_t)((src.numel() + 3) / 4), &seed, &offset, &state));
    TVK_CALL(tvk_dropout(to_tvk_dtype(src.scalar_type()), out.data_ptr(), (uint8_t*)mask.data_ptr(), src.data_ptr(), src.numel(), 1.0 - p, seed, offset, state,
                         scope.stream));
    return {out, mask};
}
at::Tensor native_dropout_backward(const at::Tensor& grad, const at::Tensor& mask, double scale) {
    return grad * mask.to(grad.scalar_type()) * scale;
}

// Categorical sampling (the generate() loop of a language model: torch.multinomial(probs, 1)), on the device end to end.
// With replacement (or one sample): inverse CDF - the row's running sum, one uniform number in (0, total] per sample, and
// the index is the count of prefix sums below it (an exact integer sum). Without replacement: the Gumbel top-k trick,
// top-k of log p + Gumbel noise.
at::Tensor multinomial(const at::Tensor& self, int64_t num_samples, bool replacement, c10::optional<at::Generator>) {
    TORCH_CHECK(self.dim() == 1 || self.dim() == 2, "prob_dist must be 1 or 2 dim");
    TORCH_CHECK(at::isFloatingType(self.scalar_type()), "multinomial only supports floating-point dtypes for input, got: ", self.scalar_type());
    const int64_t n = self.size(-1);
    TORCH_CHECK(num_samples > 0 && n > 0, "cannot sample n_sample <= 0 samples");
    TORCH_CHECK(replacement || num_samples <= n, "cannot sample n_sample > prob_dist.size(-1) samples without replacement");
    at::Tensor p = (self.dim() == 1 ? self.unsqueeze(0) : self).to(at::kFloat);
    const int64_t rows = p.size(0);
    at::Tensor u = at::empty({rows, num_samples}, p.options());
    u.uniform_(0.0, 1.0);
    at::Tensor result;
    if (replacement || num_samples == 1) {
        at::Tensor cdf = at::cumsum(p, -1);                                              // [rows, n]
        at::Tensor total = cdf.narrow(-1, n - 1, 1);                                     // [rows, 1]
        at::Tensor target = (1.0 - u) * total;                                           // in (0, total]
        if (n == 1) result = at::zeros({rows, num_samples}, p.options().dtype(at::kLong));
        else result = at::lt(cdf.narrow(-1, 0, n - 1).unsqueeze(1), target.unsqueeze(-1)).sum(at::IntArrayRef({-1}));   // [rows, samples]
    } else {
        at::Tensor gumbel = at::neg(at::log(at::neg(at::log(1.0 - u.narrow(1, 0, 1).expand({rows, n}).clone().uniform_(0.0, 1.0)))));
        result = std::get<1>(at::topk(at::log(p) + gumbel, num_samples, -1, true, true));
    }
    return self.dim() == 1 ? result.squeeze(0) : result;
}

// Integer uniform fills: low + floor(u * (high - low)) with u from the float generator. The range must fit fp32's 24-bit
// integers (class counts, vocabulary sizes, dataset indices); wider ranges raise.
at::Tensor& random_range_(at::Tensor& self, int64_t low, int64_t high, const char* name) {
    TORCH_CHECK(high > low, name, " expects 'from' to be less than 'to', but got from=", low, " >= to=", high);
    if (high - low > (int64_t(1) << 24)) TVK_NOT_IMPLEMENTED(name, " over a range of more than 2^24 values");
    at::Tensor u = at::empty(self.sizes(), self.options().dtype(at::kFloat));
    u.uniform_(0.0, 1.0);
    at::Tensor v = at::floor(u * (double)(high - low));
    v = at::clamp_max(v, (double)(high - low - 1)) + (double)low;          // u * range may round up to the range itself
    self.copy_(v.to(self.scalar_type()));
    return self;
}
at::Tensor& random_from_(at::Tensor& self, int64_t from, c10::optional<int64_t> to, c10::optional<at::Generator>) {
    TORCH_CHECK(to.has_value(), "torchvulkan [NOT IMPLEMENTED]: random_ with an open upper bound");
    return random_range_(self, from, *to, "random_");
}
at::Tensor& random_to_(at::Tensor& self, int64_t to, c10::optional<at::Generator>) { return random_range_(self, 0, to, "random_"); }
// bernoulli with a tensor of probabilities (torch.bernoulli(p)): one uniform draw per element compared with its probability
at::Tensor& bernoulli_tensor_(at::Tensor& self, const at::Tensor& p, c10::optional<at::Generator>) {
    if (self.numel() == 0) return self;
    at::Tensor prob = is_hot_float(p.scalar_type()) ? p : p.to(at::kFloat);
    at::Tensor u = at::empty(self.sizes(), prob.options().dtype(at::kFloat));
    u.uniform_(0.0, 1.0);
    at::Tensor drawn = at::lt(u, prob.to(at::kFloat));
    TORCH_CHECK(drawn.sizes() == self.sizes(), "bernoulli_: the probabilities must broadcast to the shape of self");
    self.copy_(self.scalar_type() == at::kBool ? drawn : drawn.to(self.scalar_type()));
    return self;
}
// exponential_(lambda): -log(1 - u) / lambda with u uniform in [0, 1)
at::Tensor& exponential_(at::Tensor& self, double lambd, c10::optional<at::Generator>) {
    TORCH_CHECK(lambd > 0.0, "exponential_ expects lambda > 0.0, but found lambda=", lambd);
    if (!is_hot_float(self.scalar_type())) TVK_NOT_IMPLEMENTED("exponential_ for dtype ", self.scalar_type(), " on the vulkan device");
    if (self.numel() == 0) return self;
    at::Tensor u = at::empty(self.sizes(), self.options().dtype(at::kFloat));
    u.uniform_(0.0, 1.0);
    // a draw of exactly zero is excluded (its logarithm is taken by gumbel_softmax and the like): floor at half an fp32 epsilon, as ATen does
    at::Tensor v = at::clamp_min(at::neg(at::log1p(at::neg(u))), 5.9604644775390625e-8) * (1.0 / lambd);
    self.copy_(v.to(self.scalar_type()));
    return self;
}
// a random permutation: the order that sorts n uniform numbers
at::Tensor& randperm_out(int64_t n, c10::optional<at::Generator>, at::Tensor& out) {
    TORCH_CHECK(n >= 0, "n must be non-negative, got", n);
    if (out.numel() != n) out.resize_({n});
    if (n == 0) return out;
    at::Tensor u = at::empty({n}, out.options().dtype(at::kFloat));
    u.uniform_(0.0, 1.0);
    out.copy_(std::get<1>(at::sort(u, /*stable=*/true, 0, false)).to(out.scalar_type()));
    return out;
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("bernoulli_.Tensor", &bernoulli_tensor_);
    m.impl("exponential_", &exponential_);
    m.impl("random_.from", &random_from_);
    m.impl("random_.to", &random_to_);
    m.impl("randperm.generator_out", &randperm_out);
    m.impl("multinomial", &multinomial);
    m.impl("uniform_", &uniform_);
    m.impl("normal_", &normal_);
    m.impl("bernoulli_.float", &bernoulli_float_);
    m.impl("bernoulli.p", &bernoulli_p);
    m.impl("native_dropout", &native_dropout);
    m.impl("native_dropout_backward", &native_dropout_backward);
}

}  // namespace tvk_aten
