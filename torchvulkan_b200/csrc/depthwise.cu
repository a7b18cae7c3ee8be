// Depthwise 2-D convolution (groups == cin, cout = cin * multiplier): forward, input gradient, weight gradient.
//
// The reference sends these through the same convolution entry as every other grouped convolution
// (convolution_vulkan with groups > 1, src/api/ops/conv.cpp:1088-1117; the `_conv_depthwise2d` / slow aliases at
// conv.cpp:218-230), where each group is an implicit GEMM with K = taps. With one input channel per group there is no
// contraction worth a tensor-core tile: every output element is a dot product of at most kh*kw values, and the op is
// bound by reading x and writing y once. So this is a direct kernel: one thread per output element, the filter taps of
// its channel read through the read-only cache, fp32 accumulation, any stride / padding / dilation, NCHW tensors.
// The weight gradient is one CTA per output channel: each thread keeps the tap sums of the pixels it walks in registers
// and the CTA folds them in a fixed order (no atomics: the result is the same from run to run).
#include "common.cuh"

namespace tvk {

struct DwGeo {
    int64_t N, C, H, W, M, KH, KW, Ho, Wo;      // C input channels, M outputs per input channel
    int sh, sw, ph, pw, dh, dw;
};

constexpr int kDwMaxTaps = 49;     // the weight-gradient kernel keeps one fp32 sum per tap in registers

template <typename T>
__global__ void __launch_bounds__(256) dw_forward_kernel(T* __restrict__ y, const T* __restrict__ x, const T* __restrict__ w, DwGeo g, int64_t total) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t wo = i % g.Wo, ho = (i / g.Wo) % g.Ho, co = (i / (g.Wo * g.Ho)) % (g.C * g.M), n = i / (g.Wo * g.Ho * g.C * g.M);
        const int64_t ci = co / g.M;
        const T* xp = x + (n * g.C + ci) * g.H * g.W;
        const T* wp = w + co * g.KH * g.KW;
        float acc = 0.f;
        for (int kh = 0; kh < g.KH; ++kh) {
            const int64_t h = ho * g.sh - g.ph + (int64_t)kh * g.dh;
            if (h < 0 || h >= g.H) continue;
            for (int kw = 0; kw < g.KW; ++kw) {
                const int64_t ww = wo * g.sw - g.pw + (int64_t)kw * g.dw;
                if (ww < 0 || ww >= g.W) continue;
                acc += to_f32(xp[h * g.W + ww]) * to_f32(wp[kh * g.KW + kw]);
            }
        }
        y[i] = from_f32<T>(acc);
    }
}

// dx[n, ci, h, w] = sum over the M outputs of channel ci and the taps that reach (h, w) of dy * w
template <typename T>
__global__ void __launch_bounds__(256) dw_backward_input_kernel(T* __restrict__ dx, const T* __restrict__ dy, const T* __restrict__ w, DwGeo g,
                                                               int64_t total) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t ww = i % g.W, h = (i / g.W) % g.H, ci = (i / (g.W * g.H)) % g.C, n = i / (g.W * g.H * g.C);
        float acc = 0.f;
        for (int64_t m = 0; m < g.M; ++m) {
            const int64_t co = ci * g.M + m;
            const T* gp = dy + (n * g.C * g.M + co) * g.Ho * g.Wo;
            const T* wp = w + co * g.KH * g.KW;
            for (int kh = 0; kh < g.KH; ++kh) {
                const int64_t th = h + g.ph - (int64_t)kh * g.dh;
                if (th < 0 || th % g.sh != 0) continue;
                const int64_t ho = th / g.sh;
                if (ho >= g.Ho) continue;
                for (int kw = 0; kw < g.KW; ++kw) {
                    const int64_t tw = ww + g.pw - (int64_t)kw * g.dw;
                    if (tw < 0 || tw % g.sw != 0) continue;
                    const int64_t wo = tw / g.sw;
                    if (wo >= g.Wo) continue;
                    acc += to_f32(gp[ho * g.Wo + wo]) * to_f32(wp[kh * g.KW + kw]);
                }
            }
        }
        dx[i] = from_f32<T>(acc);
    }
}

// dw[co, kh, kw] = sum over (n, ho, wo) of dy[n, co, ho, wo] * x[n, ci, ho*s - p + kh*d, wo*s - p + kw*d]. One CTA per co.
template <typename T>
__global__ void __launch_bounds__(256) dw_backward_weight_kernel(T* __restrict__ dwt, const T* __restrict__ dy, const T* __restrict__ x, DwGeo g) {
    __shared__ float smem[33];
    const int64_t co = blockIdx.x, ci = co / g.M;
    const int taps = (int)(g.KH * g.KW);
    float acc[kDwMaxTaps];
#pragma unroll
    for (int t = 0; t < kDwMaxTaps; ++t) acc[t] = 0.f;
    const int64_t plane = g.Ho * g.Wo, total = g.N * plane;
    for (int64_t i = threadIdx.x; i < total; i += blockDim.x) {
        const int64_t n = i / plane, r = i - n * plane, ho = r / g.Wo, wo = r - ho * g.Wo;
        const float gv = to_f32(dy[(n * g.C * g.M + co) * plane + r]);
        const T* xp = x + (n * g.C + ci) * g.H * g.W;
#pragma unroll
        for (int t = 0; t < kDwMaxTaps; ++t) {
            if (t < taps) {
                const int kh = t / (int)g.KW, kw = t - kh * (int)g.KW;
                const int64_t h = ho * g.sh - g.ph + (int64_t)kh * g.dh, ww = wo * g.sw - g.pw + (int64_t)kw * g.dw;
                if (h >= 0 && h < g.H && ww >= 0 && ww < g.W) acc[t] += gv * to_f32(xp[h * g.W + ww]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < kDwMaxTaps; ++t) {
        if (t < taps) {
            const float s = block_sum(acc[t], smem);
            if (threadIdx.x == 0) dwt[co * taps + t] = from_f32<T>(s);
        }
    }
}

static int dw_geo(const tvk_conv2d_desc* d, DwGeo* g, const char* who) {
    if (!d) return set_error(TVK_ERR_INVALID, "%s: null descriptor", who);
    TVK_REQUIRE(d->n >= 0 && d->cin > 0 && d->h > 0 && d->w > 0 && d->cout > 0 && d->kh > 0 && d->kw > 0, "%s: bad extent", who);
    TVK_REQUIRE(d->stride_h > 0 && d->stride_w > 0 && d->dilation_h > 0 && d->dilation_w > 0 && d->pad_h >= 0 && d->pad_w >= 0, "%s: bad stride, dilation or padding", who);
    if (d->groups != d->cin || d->cout % d->cin != 0)
        return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: %s needs groups == cin and cout a multiple of cin (groups %lld, cin %lld, cout %lld)", who,
                         (long long)d->groups, (long long)d->cin, (long long)d->cout);
    if (d->layout != 0) return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: %s on channels-last tensors (pass NCHW)", who);
    g->N = d->n; g->C = d->cin; g->H = d->h; g->W = d->w; g->M = d->cout / d->cin; g->KH = d->kh; g->KW = d->kw;
    g->sh = (int)d->stride_h; g->sw = (int)d->stride_w; g->ph = (int)d->pad_h; g->pw = (int)d->pad_w; g->dh = (int)d->dilation_h; g->dw = (int)d->dilation_w;
    g->Ho = (d->h + 2 * d->pad_h - d->dilation_h * (d->kh - 1) - 1) / d->stride_h + 1;
    g->Wo = (d->w + 2 * d->pad_w - d->dilation_w * (d->kw - 1) - 1) / d->stride_w + 1;
    TVK_REQUIRE(g->Ho > 0 && g->Wo > 0, "%s: the filter does not fit the padded input", who);
    return TVK_OK;
}

static unsigned dw_blocks(int64_t total) {
    int64_t b = (total + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (b > cap) b = cap;
    return (unsigned)(b < 1 ? 1 : b);
}

}  // namespace tvk

using namespace tvk;

extern "C" {

int tvk_depthwise_conv2d_forward(const tvk_conv2d_desc* d, void* y, const void* x, const void* w, void* stream) {
    DwGeo g;
    int rc = dw_geo(d, &g, "tvk_depthwise_conv2d_forward");
    if (rc) return rc;
    const int64_t total = g.N * g.C * g.M * g.Ho * g.Wo;
    if (total == 0) return TVK_OK;
    TVK_REQUIRE(y && x && w, "tvk_depthwise_conv2d_forward: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    TVK_DISPATCH_FLOAT(d->dtype, T, (dw_forward_kernel<T><<<dw_blocks(total), 256, 0, s>>>((T*)y, (const T*)x, (const T*)w, g, total)));
    return launch_status("depthwise conv2d forward");
}

int tvk_depthwise_conv2d_backward_input(const tvk_conv2d_desc* d, void* dx, const void* dy, const void* w, void* stream) {
    DwGeo g;
    int rc = dw_geo(d, &g, "tvk_depthwise_conv2d_backward_input");
    if (rc) return rc;
    const int64_t total = g.N * g.C * g.H * g.W;
    if (total == 0) return TVK_OK;
    TVK_REQUIRE(dx && dy && w, "tvk_depthwise_conv2d_backward_input: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    TVK_DISPATCH_FLOAT(d->dtype, T, (dw_backward_input_kernel<T><<<dw_blocks(total), 256, 0, s>>>((T*)dx, (const T*)dy, (const T*)w, g, total)));
    return launch_status("depthwise conv2d input gradient");
}

int tvk_depthwise_conv2d_backward_weight(const tvk_conv2d_desc* d, void* dw, const void* dy, const void* x, void* stream) {
    DwGeo g;
    int rc = dw_geo(d, &g, "tvk_depthwise_conv2d_backward_weight");
    if (rc) return rc;
    TVK_REQUIRE(dw, "tvk_depthwise_conv2d_backward_weight: null output");
    if (g.KH * g.KW > kDwMaxTaps)
        return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: depthwise weight gradient for filters of more than %d taps", kDwMaxTaps);
    TVK_REQUIRE(g.N == 0 || (dy && x), "tvk_depthwise_conv2d_backward_weight: null pointer");
    TVK_REQUIRE(g.C * g.M <= 0x7fffffffLL, "tvk_depthwise_conv2d_backward_weight: too many channels");
    cudaStream_t s = (cudaStream_t)stream;
    TVK_DISPATCH_FLOAT(d->dtype, T, (dw_backward_weight_kernel<T><<<(unsigned)(g.C * g.M), 256, 0, s>>>((T*)dw, (const T*)dy, (const T*)x, g)));
    return launch_status("depthwise conv2d weight gradient");
}

}  // extern "C"
