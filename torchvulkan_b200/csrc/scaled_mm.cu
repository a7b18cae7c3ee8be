// _scaled_mm: out = cast((A * scale_a) @ (B * scale_b) + bias) for float8 operands.
//
// Replaces scaled_mm_out_vulkan (src/api/ops/matmul.cpp:706-747), which follows torch's CPU emulation: both operands are
// upcast to fp32 and scaled (one scale each, or a row of A by a column of B), multiplied in fp32, the bias added and the
// result cast. Products of float8 values are exact in fp32, and the scales factor out of the sum
// (sum_k (a_ik s_i)(b_kj t_j) = s_i t_j sum_k a_ik b_kj), so the result is acc * (s_i * t_j) + bias with acc the plain
// product accumulated in fp32 - equal to the emulation up to the order of the fp32 additions. Three routes:
//  - operands with k contiguous and 16-byte aligned, fp32/fp16/bf16 output: one launch of the tcgen05 kernel for 1-byte
//    operands (kind::f8f6f4) whose epilogue applies scales, bias and cast;
//  - the same operands with a float8 output (or a bias of another dtype than the output): that kernel leaves the fp32
//    accumulator and one finishing pass applies scales, bias, 1/scale_result and the cast;
//  - any other layout: both operands are widened to fp16, which holds every e4m3 and e5m2 value exactly, multiplied by
//    the fp16 kernel with fp32 accumulation, and finished by the same pass.
#include <cuda_fp8.h>

#include "common.cuh"

namespace tvk {

__device__ __forceinline__ __half fp8_widen(uint8_t v, int kind) {
    const __half_raw r = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)v, kind == TVK_F8_E5M2 ? __NV_E5M2 : __NV_E4M3);
    return __half(r);
}

// out[r * pitch + c] = widen(in[r * rs + c * cs]) for c < cols, 0 for cols <= c < pitch
__global__ void __launch_bounds__(256) fp8_widen_kernel(__half* __restrict__ out, const uint8_t* __restrict__ in, int64_t rows, int64_t cols, int64_t pitch, int64_t rs,
                                                       int64_t cs, int kind) {
    const int64_t total = rows * pitch;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / pitch, c = i - r * pitch;
        out[i] = c < cols ? fp8_widen(in[r * rs + c * cs], kind) : __float2half(0.f);
    }
}
// The same for rows that are contiguous, 8-byte aligned and a multiple of 8 long (pitch == cols): eight values per thread.
__global__ void __launch_bounds__(256) fp8_widen8_kernel(__half* __restrict__ out, const uint8_t* __restrict__ in, int64_t rows, int64_t cols, int64_t rs, int kind) {
    const int64_t per_row = cols / 8, total = rows * per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / per_row, c = (i - r * per_row) * 8;
        const uint2 q = __ldg((const uint2*)(in + r * rs + c));
        const uint32_t w[2] = {q.x, q.y};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __half lo = fp8_widen((uint8_t)(w[j >> 1] >> (16 * (j & 1))), kind), hi = fp8_widen((uint8_t)(w[j >> 1] >> (16 * (j & 1) + 8)), kind);
            o[j] = (uint32_t)__half_as_ushort(lo) | ((uint32_t)__half_as_ushort(hi) << 16);
        }
        *(uint4*)(out + r * cols + c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

template <typename TO> __device__ __forceinline__ TO scaled_cast(float v, int) { return from_f32<TO>(v); }
template <> __device__ __forceinline__ uint8_t scaled_cast<uint8_t>(float v, int kind) {
    // no saturation: an overflow becomes NaN (e4m3) or infinity (e5m2), as a plain cast of the fp32 value does
    return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_NOSAT, kind == TVK_F8_E5M2 ? __NV_E5M2 : __NV_E4M3);
}

// Four adjacent columns of one row per thread (the accumulator's pitch is a multiple of 4, so the 16-byte load is aligned).
template <typename TO, typename TB>
__global__ void __launch_bounds__(256) scaled_mm_finish_kernel(TO* __restrict__ out, const float* __restrict__ acc, int64_t m, int64_t n, int64_t acc_pitch,
                                                              const float* __restrict__ sa, int64_t sa_stride, const float* __restrict__ sb, int64_t sb_stride,
                                                              const TB* __restrict__ bias, const float* __restrict__ scale_result, int out_kind) {
    const int64_t n4 = (n + 3) / 4, total = m * n4;
    const float post = scale_result ? 1.0f / scale_result[0] : 1.0f;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / n4, c0 = (i - r * n4) * 4;
        const float4 q = *(const float4*)(acc + r * acc_pitch + c0);
        const float a4[4] = {q.x, q.y, q.z, q.w};
        const float rsc = sa[r * sa_stride];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t c = c0 + j;
            if (c >= n) break;
            float v = a4[j] * (rsc * sb[c * sb_stride]);
            if (bias) v += to_f32(bias[c]);
            if (scale_result) v *= post;
            out[r * n + c] = scaled_cast<TO>(v, out_kind);
        }
    }
}

static int64_t round_up(int64_t v, int64_t q) { return (v + q - 1) / q * q; }
static unsigned grid_for(int64_t total) {
    int64_t b = (total + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (b > cap) b = cap;
    return (unsigned)(b < 1 ? 1 : b);
}

struct ScaledPlan {
    int64_t kp, np;
    uint64_t a_bytes, b_bytes, acc_bytes, gemm_bytes, total;
};
static ScaledPlan scaled_plan(const tvk_scaled_mm_desc* d) {
    ScaledPlan p;
    p.kp = round_up(d->k > 0 ? d->k : 1, 8);        // 16-byte row pitch of the widened operands
    p.np = round_up(d->n > 0 ? d->n : 1, 4);        // 16-byte row pitch of the fp32 accumulator
    auto a256 = [](uint64_t v) { return (v + 255) / 256 * 256; };
    p.a_bytes = a256((uint64_t)d->m * p.kp * 2);
    p.b_bytes = a256((uint64_t)d->n * p.kp * 2);
    p.acc_bytes = a256((uint64_t)d->m * p.np * 4);
    p.gemm_bytes = 0;
    p.total = p.a_bytes + p.b_bytes + p.acc_bytes;
    return p;
}

static void fill_gemm(tvk_gemm_desc* g, const tvk_scaled_mm_desc* d, const ScaledPlan& p, const void* a16, const void* b16, void* acc) {
    memset(g, 0, sizeof(*g));
    g->dtype = TVK_F16;
    g->activation = TVK_ACT_NONE;
    g->batch = 1; g->m = d->m; g->n = d->n; g->k = p.kp;
    g->a = a16; g->a_rs = p.kp; g->a_cs = 1;
    g->b = b16; g->b_rs = 1; g->b_cs = p.kp;          // widened B is stored [n, kp]: the contraction index is contiguous
    g->c = acc; g->c_rs = p.np;
    g->alpha = 1.f; g->beta = 0.f;
    g->c_f32 = 1;
}

}  // namespace tvk

using namespace tvk;

extern "C" {

static int scaled_finish(const tvk_scaled_mm_desc* d, const float* acc, int64_t acc_pitch, cudaStream_t s) {
    const unsigned blocks = grid_for(d->m * ((d->n + 3) / 4));
#define TVK_SCALED_FINISH(TO, TB)                                                                                                                           \
    scaled_mm_finish_kernel<TO, TB><<<blocks, 256, 0, s>>>((TO*)d->out, acc, d->m, d->n, acc_pitch, d->scale_a, d->sa_stride, d->scale_b, d->sb_stride,          \
                                                          (const TB*)d->bias, fp8_out ? d->scale_result : nullptr, out8_kind)
#define TVK_SCALED_FINISH_OUT(TO)                                                   \
    do {                                                                            \
        if (!d->bias || d->bias_dtype == TVK_F32) { TVK_SCALED_FINISH(TO, float); } \
        else if (d->bias_dtype == TVK_F16) { TVK_SCALED_FINISH(TO, __half); }       \
        else { TVK_SCALED_FINISH(TO, __nv_bfloat16); }                              \
    } while (0)
    // scale_result divides the product only when the output is float8 (matmul.cpp:736-738)
    const bool fp8_out = d->out_kind == TVK_SCALED_OUT_E4M3 || d->out_kind == TVK_SCALED_OUT_E5M2;
    const int out8_kind = d->out_kind == TVK_SCALED_OUT_E5M2 ? TVK_F8_E5M2 : TVK_F8_E4M3;
    switch (d->out_kind) {
        case TVK_SCALED_OUT_F32: TVK_SCALED_FINISH_OUT(float); break;
        case TVK_SCALED_OUT_F16: TVK_SCALED_FINISH_OUT(__half); break;
        case TVK_SCALED_OUT_BF16: TVK_SCALED_FINISH_OUT(__nv_bfloat16); break;
        default: TVK_SCALED_FINISH_OUT(uint8_t); break;
    }
#undef TVK_SCALED_FINISH_OUT
#undef TVK_SCALED_FINISH
    return launch_status("scaled mm finish");
}

static int scaled_validate(const tvk_scaled_mm_desc* d, const char* who) {
    if (!d) return set_error(TVK_ERR_INVALID, "%s: null descriptor", who);
    TVK_REQUIRE(d->m >= 0 && d->n >= 0 && d->k >= 0, "%s: negative extent", who);
    TVK_REQUIRE((d->a_kind == TVK_F8_E4M3 || d->a_kind == TVK_F8_E5M2) && (d->b_kind == TVK_F8_E4M3 || d->b_kind == TVK_F8_E5M2), "%s: unknown float8 kind", who);
    TVK_REQUIRE(d->out_kind == TVK_SCALED_OUT_F32 || d->out_kind == TVK_SCALED_OUT_F16 || d->out_kind == TVK_SCALED_OUT_BF16 || d->out_kind == TVK_SCALED_OUT_E4M3 ||
                    d->out_kind == TVK_SCALED_OUT_E5M2,
                "%s: unknown output kind %d", who, (int)d->out_kind);
    TVK_REQUIRE(d->sa_stride == 0 || d->sa_stride == 1, "%s: scale_a is one value or one per row of A", who);
    TVK_REQUIRE(d->sb_stride == 0 || d->sb_stride == 1, "%s: scale_b is one value or one per column of B", who);
    TVK_REQUIRE(!d->bias || d->bias_dtype == TVK_F32 || d->bias_dtype == TVK_F16 || d->bias_dtype == TVK_BF16, "%s: bias must be fp32, fp16 or bf16", who);
    return TVK_OK;
}

int tvk_scaled_mm_workspace_size(const tvk_scaled_mm_desc* d, uint64_t* bytes) {
    if (!bytes) return set_error(TVK_ERR_INVALID, "tvk_scaled_mm_workspace_size: null output");
    int rc = scaled_validate(d, "tvk_scaled_mm_workspace_size");
    if (rc) return rc;
    ScaledPlan p = scaled_plan(d);
    tvk_gemm_desc g;
    fill_gemm(&g, d, p, nullptr, nullptr, nullptr);
    uint64_t gb = 0;
    if (d->m > 0 && d->n > 0) {
        // the inner GEMM is asked about scratch with placeholder addresses of the alignment it will get
        g.a = (const void*)256; g.b = (const void*)256; g.c = (void*)256;
        rc = tvk_gemm_workspace_size(&g, &gb);
        if (rc) return rc;
    }
    *bytes = p.total + ((gb + 255) / 256 * 256);
    return TVK_OK;
}

int tvk_scaled_mm(const tvk_scaled_mm_desc* d, void* workspace, uint64_t workspace_bytes, void* stream) {
    int rc = scaled_validate(d, "tvk_scaled_mm");
    if (rc) return rc;
    if (d->m == 0 || d->n == 0) return TVK_OK;
    TVK_REQUIRE(d->out && d->scale_a && d->scale_b && (d->k == 0 || (d->a && d->b)), "tvk_scaled_mm: null pointer");
    uint64_t need = 0;
    rc = tvk_scaled_mm_workspace_size(d, &need);
    if (rc) return rc;
    TVK_REQUIRE(workspace && workspace_bytes >= need && ((uintptr_t)workspace & 255) == 0, "tvk_scaled_mm: a 256-byte aligned workspace of %llu bytes is required, %llu given",
                (unsigned long long)need, (unsigned long long)workspace_bytes);
    cudaStream_t s = (cudaStream_t)stream;
    const ScaledPlan p = scaled_plan(d);
    __half* a16 = (__half*)workspace;
    __half* b16 = (__half*)((uint8_t*)workspace + p.a_bytes);
    float* acc = (float*)((uint8_t*)workspace + p.a_bytes + p.b_bytes);
    void* gws = (uint8_t*)workspace + p.total;
    if (f8_product_ok(d->a, d->a_rs, d->a_cs, d->b, d->b_rs, d->b_cs, d->m, d->n, d->k)) {
        // the operands are read in place by the tensor cores (tcgen05.mma kind::f8f6f4); products of float8 values are exact
        // in the fp32 accumulator, as they are in the reference's emulation
        const int out_dtype = d->out_kind == TVK_SCALED_OUT_F32 ? TVK_F32 : d->out_kind == TVK_SCALED_OUT_F16 ? TVK_F16 : d->out_kind == TVK_SCALED_OUT_BF16 ? TVK_BF16 : -1;
        static const bool two_pass = getenv("TORCHVULKAN_SCALED_MM_TWO_PASS") != nullptr;      // keep the separate finishing pass (tests compare the two)
        if (out_dtype >= 0 && (!d->bias || d->bias_dtype == out_dtype) && !two_pass) {
            // scales, bias and cast in the product kernel's epilogue: the same arithmetic as the finishing pass, acc * (sa * sb) + bias
            const F8Epilogue e = {d->scale_a, d->sa_stride, d->scale_b, d->sb_stride, d->bias};
            return f8_product(d->a_kind, d->b_kind, d->a, d->a_rs, d->b, d->b_cs, d->m, d->n, d->k, d->out, out_dtype, d->n, &e, s);
        }
        rc = f8_product(d->a_kind, d->b_kind, d->a, d->a_rs, d->b, d->b_cs, d->m, d->n, d->k, acc, TVK_F32, p.np, nullptr, s);
        if (rc) return rc;
        return scaled_finish(d, acc, p.np, s);
    }
    auto widen = [&](__half* o, const void* in, int64_t rows, int64_t rs, int64_t cs, int kind) {
        if (cs == 1 && d->k == p.kp && rs % 8 == 0 && ((uintptr_t)in & 7) == 0)
            fp8_widen8_kernel<<<grid_for(rows * (p.kp / 8)), 256, 0, s>>>(o, (const uint8_t*)in, rows, p.kp, rs, kind);
        else
            fp8_widen_kernel<<<grid_for(rows * p.kp), 256, 0, s>>>(o, (const uint8_t*)in, rows, d->k, p.kp, rs, cs, kind);
    };
    widen(a16, d->a, d->m, d->a_rs, d->a_cs, d->a_kind);
    // B is read as its transpose: row j of the widened copy is column j of B
    widen(b16, d->b, d->n, d->b_cs, d->b_rs, d->b_kind);
    rc = launch_status("float8 widening");
    if (rc) return rc;
    tvk_gemm_desc g;
    fill_gemm(&g, d, p, a16, b16, acc);
    rc = tvk_gemm(&g, gws, workspace_bytes - p.total, stream);
    if (rc) return rc;
    return scaled_finish(d, acc, p.np, s);
}

}  // extern "C"
