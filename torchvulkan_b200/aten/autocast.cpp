// torch.autocast("vulkan") and the gradient scaler's two operators.
//
// Counterparts in the reference: src/api/registration.cpp:4-21 (the AutocastPrivateUse1 key) and
// src/api/decompositions.cpp:1625-1626 (_amp_foreach_non_finite_check_and_unscale_, _amp_update_scale_).
// The autocast key needs two things from a backend: a fallthrough for every operator that has no casting policy, and the
// policies themselves - which operators run in the lower-precision type (matmul, convolution, attention ...), which in
// fp32 (softmax-like reductions, losses ...), which promote their inputs. PyTorch ships the operator lists and the wrapper
// templates for exactly this purpose (ATen/autocast_mode.h); a backend instantiates them for its key and adds nothing.
#include "common.h"

#include <ATen/autocast_mode.h>

TORCH_LIBRARY_IMPL(_, AutocastPrivateUse1, m) { m.fallback(torch::CppFunction::makeFallthrough()); }

namespace at::autocast {

#define TVK_AUTOCAST_LOW(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, lower_precision_fp)
#define TVK_AUTOCAST_FP32(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, fp32)
#define TVK_AUTOCAST_FP32_OPT(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, fp32_set_opt_dtype)
#define TVK_AUTOCAST_PROMOTE(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, promote)

TORCH_LIBRARY_IMPL(aten, AutocastPrivateUse1, m) {
    AT_FORALL_LOWER_PRECISION_FP(TVK_AUTOCAST_LOW)
    AT_FORALL_FP32(TVK_AUTOCAST_FP32)
    AT_FORALL_FP32_SET_OPT_DTYPE(TVK_AUTOCAST_FP32_OPT)
    AT_FORALL_DIFFERENT_REDISPATCH_SIGNATURE(KERNEL_DIFFERENT_REDISPATCH_SIGNATURE_PRIVATEUSEONE)
    AT_FORALL_PROMOTE(TVK_AUTOCAST_PROMOTE)
}

}  // namespace at::autocast

namespace tvk_aten {
namespace {

// grads *= inv_scale, and found_inf = 1 where any of them holds a non-finite value (torch.amp.GradScaler.unscale_). A few
// launches per tensor; found_inf stays on the device.
void amp_unscale_(at::TensorList grads, at::Tensor& found_inf, const at::Tensor& inv_scale) {
    TORCH_CHECK(inv_scale.numel() == 1 && found_inf.numel() == 1, "inv_scale and found_inf must be 1-element tensors.");
    for (const at::Tensor& g : grads) {
        if (g.numel() == 0) continue;
        at::Tensor gm = g;
        gm.mul_(inv_scale.to(g.scalar_type()).reshape({}));
        at::Tensor bad = at::logical_not(at::isfinite(g)).any().to(found_inf.scalar_type()).reshape(found_inf.sizes());
        found_inf.copy_(at::maximum(found_inf, bad));
    }
}

// The scaler's update rule, evaluated on the device (no read-back): found_inf -> scale *= backoff, tracker = 0; otherwise
// tracker += 1 and, when it reaches the interval, scale *= growth (unless that overflows) and tracker = 0.
at::Tensor& amp_update_scale_(at::Tensor& scale, at::Tensor& growth_tracker, const at::Tensor& found_inf, double growth_factor, double backoff_factor,
                              int64_t growth_interval) {
    TORCH_CHECK(scale.numel() == 1 && growth_tracker.numel() == 1 && found_inf.numel() == 1, "scale, growth_tracker and found_inf must be 1-element tensors.");
    at::Tensor overflow = at::gt(found_inf.reshape({}), 0);
    at::Tensor s = scale.reshape({});
    at::Tensor tracker = growth_tracker.reshape({}).to(at::kFloat);                  // small counts: exact in fp32
    at::Tensor bumped = tracker + 1;
    at::Tensor grown = s * growth_factor;
    at::Tensor grow = at::logical_and(at::logical_not(overflow), at::logical_and(at::ge(bumped, (double)growth_interval), at::isfinite(grown)));
    at::Tensor zero = at::zeros({}, tracker.options());
    at::Tensor new_scale = at::where(overflow, s * backoff_factor, at::where(grow, grown, s));
    at::Tensor new_tracker = at::where(at::logical_or(overflow, grow), zero, bumped);
    scale.copy_(new_scale.reshape(scale.sizes()));
    growth_tracker.copy_(new_tracker.to(growth_tracker.scalar_type()).reshape(growth_tracker.sizes()));
    return scale;
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("_amp_foreach_non_finite_check_and_unscale_", &amp_unscale_);
    m.impl("_amp_update_scale_", &amp_update_scale_);
}

}  // namespace tvk_aten
