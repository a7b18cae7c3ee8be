// scaled_dot_product_attention on the "vulkan" device: backend choice and the overrideable fused op.
//
// Counterparts in the reference: fused_sdp_choice_vulkan, sdpa_forward_vulkan, sdpa_backward_vulkan
// (src/api/ops/attention.cpp:667-762). F.scaled_dot_product_attention asks the
// _fused_sdp_choice stub which backend to run; answering "overrideable" routes the call to
// _scaled_dot_product_fused_attention_overrideable(+_backward), which receive q/k/v with their
// own head counts (grouped-query attention is resolved inside the kernel, group = Hq / Hk).
// Cases the attention kernels do not cover (an attention mask, fp32, head sizes or key counts that are
// not multiples of 8) run inside the same two operators as a composition of this backend's matmul,
// elementwise and reduction launches in fp32 (scores, mask, softmax with the "no visible key -> 0"
// rule, P.V; the backward recomputes P from the saved log-sum-exp), as the reference's fused path takes
// an additive mask (attention.cpp:698-722). Only dropout answers "math" (attention.cpp:678).
#include "common.h"

#include <ATen/SDPBackend.h>
#include <ATen/native/transformers/attention.h>

#include <cmath>

namespace tvk_aten {
namespace {

bool fused_supported(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const c10::optional<at::Tensor>& mask, double dropout_p) {
    if (mask.has_value() && mask->defined()) return false;
    if (dropout_p != 0.0) return false;
    if (q.dim() != 4 || k.dim() != 4 || v.dim() != 4) return false;
    const auto st = q.scalar_type();
    if (!(st == at::kHalf || st == at::kBFloat16) || k.scalar_type() != st || v.scalar_type() != st) return false;
    if (q.size(-1) != k.size(-1) || k.size(-1) != v.size(-1)) return false;           // one head size
    if (q.size(-1) % 8 != 0 || k.size(2) % 8 != 0) return false;
    if (k.size(1) == 0 || q.size(1) % k.size(1) != 0 || k.size(1) != v.size(1)) return false;
    return true;
}

// what the composed route takes: 4-D q, k, v of one hot floating dtype with matching head sizes, Hq a multiple of Hk
bool composed_supported(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double dropout_p) {
    if (dropout_p != 0.0 || q.dim() != 4 || k.dim() != 4 || v.dim() != 4) return false;
    const auto st = q.scalar_type();
    if (!is_hot_float(st) || k.scalar_type() != st || v.scalar_type() != st) return false;
    if (q.size(-1) != k.size(-1) || k.size(2) != v.size(2)) return false;
    return k.size(1) > 0 && q.size(1) % k.size(1) == 0 && k.size(1) == v.size(1);
}

int64_t fused_sdp_choice(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const c10::optional<at::Tensor>& mask, double dropout_p,
                         bool /*is_causal*/, c10::optional<double> /*scale*/, bool /*enable_gqa*/) {
    const bool ours = fused_supported(q, k, v, mask, dropout_p) || composed_supported(q, k, v, dropout_p);
    return static_cast<int64_t>(ours ? at::SDPBackend::overrideable : at::SDPBackend::math);
}

// ---- the composed route ------------------------------------------------------------------------------------------------
// [B, Hk, S, D] -> [B, Hq, S, D]: query head h reads KV head h / (Hq / Hk)
at::Tensor expand_kv(const at::Tensor& t, int64_t Hq) {
    const int64_t B = t.size(0), Hk = t.size(1), S = t.size(2), D = t.size(3);
    if (Hk == Hq) return t;
    return t.unsqueeze(2).expand({B, Hk, Hq / Hk, S, D}).reshape({B, Hq, S, D});
}
// [B, Hq, S, D] gradient -> [B, Hk, S, D]: the heads of a group add up
at::Tensor reduce_kv(const at::Tensor& t, int64_t Hk) {
    const int64_t B = t.size(0), Hq = t.size(1), S = t.size(2), D = t.size(3);
    if (Hk == Hq) return t;
    return t.reshape({B, Hk, Hq / Hk, S, D}).sum(at::IntArrayRef({2}));
}
at::Tensor scalar_on(const at::Tensor& like, double v) {
    at::Tensor t = empty_vulkan({}, at::kFloat, like.device());
    t.fill_(v);
    return t;
}
// fp32 scores q.k^T * scale + bias, -inf where the causal rule (key j visible to query l when j <= l) or a boolean mask hides a key
at::Tensor masked_scores(const at::Tensor& q32, const at::Tensor& kk32, const at::Tensor& bias, bool causal, double scale) {
    at::Tensor s = at::matmul(q32, kk32.transpose(-2, -1)) * scale;
    const at::Tensor ninf = scalar_on(s, -INFINITY);
    if (bias.defined()) s = bias.scalar_type() == at::kBool ? at::where(bias, s, ninf) : s + bias.to(at::kFloat);
    if (causal) {
        at::Tensor vis = at::ones({q32.size(2), kk32.size(2)}, at::TensorOptions().dtype(at::kBool).device(at::kCPU)).tril().to(s.device());
        s = at::where(vis, s, ninf);
    }
    return s;
}

std::tuple<at::Tensor, at::Tensor> composed_forward(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value, const at::Tensor& bias, bool causal,
                                                    double scale) {
    const int64_t Hq = query.size(1);
    at::Tensor q32 = query.to(at::kFloat), kk = expand_kv(key.to(at::kFloat), Hq), vv = expand_kv(value.to(at::kFloat), Hq);
    at::Tensor s = masked_scores(q32, kk, bias, causal, scale);
    const at::Tensor zero = scalar_on(s, 0.0), pinf = scalar_on(s, INFINITY);
    at::Tensor m = at::amax(s, {-1}, true);
    at::Tensor seen = at::gt(m, -INFINITY);                         // false: the row sees no key -> out 0, lse +inf
    at::Tensor m_safe = at::where(seen, m, zero);
    at::Tensor e = at::exp(s - m_safe);
    at::Tensor sum = e.sum(at::IntArrayRef({-1}), true);
    at::Tensor p = e * at::where(seen, at::reciprocal(sum), zero);
    at::Tensor out = at::matmul(p, vv).to(query.scalar_type());
    at::Tensor lse = at::where(seen, m_safe + at::log(sum), pinf).squeeze(-1);
    return {out, lse};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> composed_backward(const at::Tensor& grad_out, const at::Tensor& query, const at::Tensor& key,
                                                                             const at::Tensor& value, const at::Tensor& bias, const at::Tensor& out,
                                                                             const at::Tensor& lse, bool causal, double scale, bool want_bias) {
    const int64_t Hq = query.size(1), Hk = key.size(1);
    const at::ScalarType st = query.scalar_type();
    at::Tensor q32 = query.to(at::kFloat), kk = expand_kv(key.to(at::kFloat), Hq), vv = expand_kv(value.to(at::kFloat), Hq);
    at::Tensor go = grad_out.to(at::kFloat);
    // P from the saved log-sum-exp: exp(-inf - lse) and exp(s - inf) are both 0, so hidden keys and unseen rows need no special case
    at::Tensor p = at::exp(masked_scores(q32, kk, bias, causal, scale) - lse.to(at::kFloat).unsqueeze(-1));
    at::Tensor dp = at::matmul(go, vv.transpose(-2, -1));
    at::Tensor delta = (go * out.to(at::kFloat)).sum(at::IntArrayRef({-1}), true);
    at::Tensor ds = p * (dp - delta);
    at::Tensor dq = (at::matmul(ds, kk) * scale).to(st);
    at::Tensor dk = reduce_kv(at::matmul(ds.transpose(-2, -1), q32) * scale, Hk).to(st);
    at::Tensor dv = reduce_kv(at::matmul(p.transpose(-2, -1), go), Hk).to(st);
    at::Tensor dbias;
    if (want_bias && bias.defined() && bias.scalar_type() != at::kBool) dbias = ds.sum_to_size(bias.sizes()).to(bias.scalar_type());
    return {dq, dk, dv, dbias};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, c10::SymInt, c10::SymInt, at::Tensor, at::Tensor, at::Tensor> sdpa_forward(
    const at::Tensor& query, const at::Tensor& key, const at::Tensor& value, const c10::optional<at::Tensor>& attn_bias, double dropout_p,
    bool is_causal, bool /*return_debug_mask*/, c10::optional<double> scale) {
    if (!fused_supported(query, key, value, attn_bias, dropout_p)) {
        TORCH_CHECK(composed_supported(query, key, value, dropout_p),
                    "torchvulkan [NOT IMPLEMENTED]: attention needs 4-D fp32/fp16/bf16 q, k, v of one dtype and head size, Hq a multiple of Hk, and no dropout");
        at::Tensor out_c, lse_c;
        std::tie(out_c, lse_c) = composed_forward(query, key, value, attn_bias.has_value() ? *attn_bias : at::Tensor(), is_causal,
                                                  scale.value_or(1.0 / std::sqrt((double)query.size(3))));
        at::Tensor none_c;
        at::Tensor seed_c = at::empty({}, at::TensorOptions().dtype(at::kLong).device(at::kCPU)), offset_c = at::empty({}, seed_c.options());
        seed_c.fill_(0); offset_c.fill_(0);
        return {out_c, lse_c, none_c, none_c, c10::SymInt(query.size(2)), c10::SymInt(key.size(2)), seed_c, offset_c, none_c};
    }
    at::Tensor q = contiguous_vulkan(query), k = contiguous_vulkan(key), v = contiguous_vulkan(value);
    const int64_t B = q.size(0), Hq = q.size(1), L = q.size(2), D = q.size(3), Hk = k.size(1), S = k.size(2);
    TORCH_CHECK(k.size(0) == B && v.size(0) == B && v.size(2) == S, "torchvulkan [ERROR]: attention: q, k, v batch or length mismatch");
    at::Tensor out = empty_vulkan({B, Hq, L, D}, q.scalar_type(), q.device());
    at::Tensor lse = empty_vulkan({B, Hq, L}, at::kFloat, q.device());
    if (out.numel()) {
        DeviceScope scope(q);
        const int dt = to_tvk_dtype(q.scalar_type());
        uint64_t ws_bytes = 0;
        TVK_CALL(tvk_attention_workspace_size(dt, B, Hq, Hk, L, S, D, 0, &ws_bytes));
        Workspace ws(scope.device, ws_bytes);
        const double sc = scale.value_or(1.0 / std::sqrt((double)D));
        TVK_CALL(tvk_attention_forward(dt, out.data_ptr(), (float*)lse.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), B, Hq, Hk, L, S, D, sc,
                                       is_causal ? 1 : 0, ws.ptr, ws.bytes, scope.stream));
    }
    at::Tensor none;
    at::Tensor seed = at::empty({}, at::TensorOptions().dtype(at::kLong).device(at::kCPU)), offset = at::empty({}, seed.options());
    seed.fill_(0); offset.fill_(0);
    return {out, lse, none, none, c10::SymInt(L), c10::SymInt(S), seed, offset, none};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> sdpa_backward(
    const at::Tensor& grad_out, const at::Tensor& query, const at::Tensor& key, const at::Tensor& value, const at::Tensor& attn_bias,
    std::array<bool, 4> grad_input_mask, const at::Tensor& out, const at::Tensor& logsumexp, const at::Tensor& /*cum_seq_q*/,
    const at::Tensor& /*cum_seq_k*/, c10::SymInt /*max_q*/, c10::SymInt /*max_k*/, double dropout_p, bool is_causal, const at::Tensor& /*philox_seed*/,
    const at::Tensor& /*philox_offset*/, c10::optional<double> scale) {
    TORCH_CHECK(dropout_p == 0.0, "torchvulkan [NOT IMPLEMENTED]: attention backward with dropout");
    if (!fused_supported(query, key, value, attn_bias.defined() ? c10::optional<at::Tensor>(attn_bias) : c10::nullopt, dropout_p))
        return composed_backward(grad_out, query, key, value, attn_bias, out, logsumexp, is_causal, scale.value_or(1.0 / std::sqrt((double)query.size(3))),
                                 grad_input_mask[3]);
    at::Tensor q = contiguous_vulkan(query), k = contiguous_vulkan(key), v = contiguous_vulkan(value);
    at::Tensor go = contiguous_vulkan(grad_out.to(q.scalar_type())), o = contiguous_vulkan(out), lse = contiguous_vulkan(logsumexp);
    const int64_t B = q.size(0), Hq = q.size(1), L = q.size(2), D = q.size(3), Hk = k.size(1), S = k.size(2);
    at::Tensor dq = empty_like_contig(q), dk = empty_like_contig(k), dv = empty_like_contig(v);
    if (q.numel() || k.numel()) {
        DeviceScope scope(q);
        const int dt = to_tvk_dtype(q.scalar_type());
        uint64_t ws_bytes = 0;
        TVK_CALL(tvk_attention_workspace_size(dt, B, Hq, Hk, L, S, D, 1, &ws_bytes));
        Workspace ws(scope.device, ws_bytes);
        const double sc = scale.value_or(1.0 / std::sqrt((double)D));
        TVK_CALL(tvk_attention_backward(dt, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), go.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                        o.data_ptr(), (const float*)lse.data_ptr(), B, Hq, Hk, L, S, D, sc, is_causal ? 1 : 0, ws.ptr, ws.bytes,
                                        scope.stream));
    }
    return {dq, dk, dv, at::Tensor()};
}

}  // namespace
}  // namespace tvk_aten

// scaled_dot_product_attention consults this stub, not the _fused_sdp_choice operator
namespace at::native {
REGISTER_PRIVATEUSE1_DISPATCH(_fused_sdp_choice_stub, &tvk_aten::fused_sdp_choice);
}

namespace tvk_aten {
TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("_fused_sdp_choice", &fused_sdp_choice);
    m.impl("_scaled_dot_product_fused_attention_overrideable", &sdpa_forward);
    m.impl("_scaled_dot_product_fused_attention_overrideable_backward", &sdpa_backward);
}
}  // namespace tvk_aten
