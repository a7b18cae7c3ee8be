// 2-D max and average pooling, forward and backward, on NCHW planes.
//
// Replaces the reference's pooling entries (src/api/ops/pool.cpp: max_pool2d_with_indices, avg_pool2d and their
// backward ops, one shader each). Pooling is bound by reading x and writing y once: one thread per output element walks
// its window (a few taps), fp32 arithmetic, any kernel / stride / padding / dilation. The backward kernels are gathers
// - one thread per INPUT element sums the gradients of the windows that selected it (max) or cover it (average) in a
// fixed order - so they need no atomics and give the same bits from run to run. Max pooling keeps ATen's conventions:
// a NaN in the window wins, ties keep the first element in row-major order, and the saved index is h * W + w inside the
// plane.
#include "common.cuh"

namespace tvk {

struct PoolGeo {
    int64_t planes, H, W, Ho, Wo;
    int kh, kw, sh, sw, ph, pw, dh, dw;
    int count_include_pad;
    int64_t divisor_override;
};

template <typename T>
__global__ void __launch_bounds__(256) max_pool_fwd_kernel(T* __restrict__ y, int64_t* __restrict__ idx, const T* __restrict__ x, PoolGeo g, int64_t total) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t wo = i % g.Wo, ho = (i / g.Wo) % g.Ho, p = i / (g.Wo * g.Ho);
        const T* xp = x + p * g.H * g.W;
        float best = -INFINITY;
        int64_t arg = -1;
        for (int a = 0; a < g.kh; ++a) {
            const int64_t h = ho * g.sh - g.ph + (int64_t)a * g.dh;
            if (h < 0 || h >= g.H) continue;
            for (int b = 0; b < g.kw; ++b) {
                const int64_t w = wo * g.sw - g.pw + (int64_t)b * g.dw;
                if (w < 0 || w >= g.W) continue;
                const float v = to_f32(xp[h * g.W + w]);
                if (arg < 0 || v > best || v != v) { best = v; arg = h * g.W + w; }      // (nothing compares greater than a held NaN)
            }
        }
        y[i] = from_f32<T>(best);
        idx[i] = arg < 0 ? 0 : arg;
    }
}

// windows (along one axis) whose taps can touch input coordinate c: output positions lo..hi
__device__ __forceinline__ void covering(int64_t c, int pad, int k, int dil, int stride, int64_t outs, int64_t* lo, int64_t* hi) {
    const int64_t t = c + pad - (int64_t)(k - 1) * dil;
    *lo = t <= 0 ? 0 : (t + stride - 1) / stride;
    *hi = (c + pad) / stride;
    if (*hi > outs - 1) *hi = outs - 1;
}

template <typename T>
__global__ void __launch_bounds__(256) max_pool_bwd_kernel(T* __restrict__ dx, const T* __restrict__ dy, const int64_t* __restrict__ idx, PoolGeo g, int64_t total) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t w = i % g.W, h = (i / g.W) % g.H, p = i / (g.W * g.H);
        const int64_t me = h * g.W + w;
        int64_t ho0, ho1, wo0, wo1;
        covering(h, g.ph, g.kh, g.dh, g.sh, g.Ho, &ho0, &ho1);
        covering(w, g.pw, g.kw, g.dw, g.sw, g.Wo, &wo0, &wo1);
        float acc = 0.f;
        for (int64_t ho = ho0; ho <= ho1; ++ho)
            for (int64_t wo = wo0; wo <= wo1; ++wo) {
                const int64_t o = (p * g.Ho + ho) * g.Wo + wo;
                if (idx[o] == me) acc += to_f32(dy[o]);
            }
        dx[i] = from_f32<T>(acc);
    }
}

// the divisor of output window (ho, wo), as ATen's avg_pool2d defines it
__device__ __forceinline__ float avg_divisor(const PoolGeo& g, int64_t ho, int64_t wo) {
    if (g.divisor_override > 0) return (float)g.divisor_override;
    int64_t hs = ho * g.sh - g.ph, ws = wo * g.sw - g.pw;
    int64_t he = hs + g.kh < g.H + g.ph ? hs + g.kh : g.H + g.ph, we = ws + g.kw < g.W + g.pw ? ws + g.kw : g.W + g.pw;
    const int64_t padded = (he - hs) * (we - ws);
    if (g.count_include_pad) return (float)padded;
    hs = hs < 0 ? 0 : hs; ws = ws < 0 ? 0 : ws;
    he = he > g.H ? g.H : he; we = we > g.W ? g.W : we;
    return (float)((he - hs) * (we - ws));
}

template <typename T>
__global__ void __launch_bounds__(256) avg_pool_fwd_kernel(T* __restrict__ y, const T* __restrict__ x, PoolGeo g, int64_t total) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t wo = i % g.Wo, ho = (i / g.Wo) % g.Ho, p = i / (g.Wo * g.Ho);
        const T* xp = x + p * g.H * g.W;
        float acc = 0.f;
        for (int a = 0; a < g.kh; ++a) {
            const int64_t h = ho * g.sh - g.ph + a;
            if (h < 0 || h >= g.H) continue;
            for (int b = 0; b < g.kw; ++b) {
                const int64_t w = wo * g.sw - g.pw + b;
                if (w < 0 || w >= g.W) continue;
                acc += to_f32(xp[h * g.W + w]);
            }
        }
        y[i] = from_f32<T>(acc / avg_divisor(g, ho, wo));
    }
}

template <typename T>
__global__ void __launch_bounds__(256) avg_pool_bwd_kernel(T* __restrict__ dx, const T* __restrict__ dy, PoolGeo g, int64_t total) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t w = i % g.W, h = (i / g.W) % g.H, p = i / (g.W * g.H);
        int64_t ho0, ho1, wo0, wo1;
        covering(h, g.ph, g.kh, 1, g.sh, g.Ho, &ho0, &ho1);
        covering(w, g.pw, g.kw, 1, g.sw, g.Wo, &wo0, &wo1);
        float acc = 0.f;
        for (int64_t ho = ho0; ho <= ho1; ++ho)
            for (int64_t wo = wo0; wo <= wo1; ++wo) acc += to_f32(dy[(p * g.Ho + ho) * g.Wo + wo]) / avg_divisor(g, ho, wo);
        dx[i] = from_f32<T>(acc);
    }
}

static int pool_geo(const tvk_pool2d_desc* d, PoolGeo* g, bool avg, const char* who) {
    if (!d) return set_error(TVK_ERR_INVALID, "%s: null descriptor", who);
    TVK_REQUIRE(d->planes >= 0 && d->h > 0 && d->w > 0 && d->ho > 0 && d->wo > 0, "%s: bad extent", who);
    TVK_REQUIRE(d->kh > 0 && d->kw > 0 && d->stride_h > 0 && d->stride_w > 0 && d->dilation_h > 0 && d->dilation_w > 0 && d->pad_h >= 0 && d->pad_w >= 0,
                "%s: bad kernel, stride, dilation or padding", who);
    TVK_REQUIRE(2 * d->pad_h <= d->kh && 2 * d->pad_w <= d->kw, "%s: pad should be at most half of the kernel size", who);
    TVK_REQUIRE(!avg || (d->dilation_h == 1 && d->dilation_w == 1), "%s: average pooling has no dilation", who);
    TVK_REQUIRE(d->kh < (1 << 20) && d->kw < (1 << 20) && d->stride_h < (1 << 20) && d->stride_w < (1 << 20), "%s: kernel or stride too large", who);
    g->planes = d->planes; g->H = d->h; g->W = d->w; g->Ho = d->ho; g->Wo = d->wo;
    g->kh = (int)d->kh; g->kw = (int)d->kw; g->sh = (int)d->stride_h; g->sw = (int)d->stride_w; g->ph = (int)d->pad_h; g->pw = (int)d->pad_w;
    g->dh = (int)d->dilation_h; g->dw = (int)d->dilation_w;
    g->count_include_pad = d->count_include_pad ? 1 : 0;
    g->divisor_override = d->divisor_override;
    return TVK_OK;
}

static unsigned pool_blocks(int64_t total) {
    int64_t b = (total + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (b > cap) b = cap;
    return (unsigned)(b < 1 ? 1 : b);
}

}  // namespace tvk

using namespace tvk;

extern "C" {

int tvk_max_pool2d_forward(const tvk_pool2d_desc* d, void* y, int64_t* indices, const void* x, void* stream) {
    PoolGeo g;
    int rc = pool_geo(d, &g, false, "tvk_max_pool2d_forward");
    if (rc) return rc;
    const int64_t total = g.planes * g.Ho * g.Wo;
    if (total == 0) return TVK_OK;
    TVK_REQUIRE(y && indices && x, "tvk_max_pool2d_forward: null pointer");
    TVK_DISPATCH_FLOAT(d->dtype, T, (max_pool_fwd_kernel<T><<<pool_blocks(total), 256, 0, (cudaStream_t)stream>>>((T*)y, indices, (const T*)x, g, total)));
    return launch_status("max pool forward");
}

int tvk_max_pool2d_backward(const tvk_pool2d_desc* d, void* dx, const void* dy, const int64_t* indices, void* stream) {
    PoolGeo g;
    int rc = pool_geo(d, &g, false, "tvk_max_pool2d_backward");
    if (rc) return rc;
    const int64_t total = g.planes * g.H * g.W;
    if (total == 0) return TVK_OK;
    TVK_REQUIRE(dx && dy && indices, "tvk_max_pool2d_backward: null pointer");
    TVK_DISPATCH_FLOAT(d->dtype, T, (max_pool_bwd_kernel<T><<<pool_blocks(total), 256, 0, (cudaStream_t)stream>>>((T*)dx, (const T*)dy, indices, g, total)));
    return launch_status("max pool backward");
}

int tvk_avg_pool2d_forward(const tvk_pool2d_desc* d, void* y, const void* x, void* stream) {
    PoolGeo g;
    int rc = pool_geo(d, &g, true, "tvk_avg_pool2d_forward");
    if (rc) return rc;
    const int64_t total = g.planes * g.Ho * g.Wo;
    if (total == 0) return TVK_OK;
    TVK_REQUIRE(y && x, "tvk_avg_pool2d_forward: null pointer");
    TVK_DISPATCH_FLOAT(d->dtype, T, (avg_pool_fwd_kernel<T><<<pool_blocks(total), 256, 0, (cudaStream_t)stream>>>((T*)y, (const T*)x, g, total)));
    return launch_status("average pool forward");
}

int tvk_avg_pool2d_backward(const tvk_pool2d_desc* d, void* dx, const void* dy, void* stream) {
    PoolGeo g;
    int rc = pool_geo(d, &g, true, "tvk_avg_pool2d_backward");
    if (rc) return rc;
    const int64_t total = g.planes * g.H * g.W;
    if (total == 0) return TVK_OK;
    TVK_REQUIRE(dx && dy, "tvk_avg_pool2d_backward: null pointer");
    TVK_DISPATCH_FLOAT(d->dtype, T, (avg_pool_bwd_kernel<T><<<pool_blocks(total), 256, 0, (cudaStream_t)stream>>>((T*)dx, (const T*)dy, g, total)));
    return launch_status("average pool backward");
}

}  // extern "C"
