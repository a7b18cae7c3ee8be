// conv2d by unfold (im2col) + the tensor-core GEMM of gemm.cu, for all three directions: the route of fp32 tensors and of
// every geometry the implicit-GEMM kernels of conv.cu do not take (dilation, strides above 2, unequal strides).
//
// The fp16/bf16 kernels of conv.cu feed pixels to the tensor cores straight from the activation tensor; fp32 operands
// have to pass through the hi/lo tf32 split anyway (gemm.cu), so here the patches are first written out as rows of a
// [n][Ho*Wo][Ci*taps] matrix and every direction becomes a batched GEMM over the images, as the reference's own
// unfold fallback does (im2col / col2im, src/api/ops/conv.cpp:200-216):
//   forward          y[n]  (Co x P)      = W (Co x K) . cols[n]^T          (or (P x Co) = cols[n] . W^T for channels-last y)
//   input gradient   dcols[n] (P x K)    = dY[n]^T . W, then dx = fold(dcols) as a gather (no atomics)
//   weight gradient  dW = sum over n of dY[n] (Co x P) . cols[n] (P x K): per-image partials + tvk_reduce over n
// The order of k inside a patch follows the filter's memory (ci*taps + tap for OIHW, tap*Ci + ci for a channels-last
// filter), so the filter and its gradient are used in place as Co x K matrices. The matrices have the tensors' dtype
// (fp16/bf16 products accumulate in fp32 on the tensor cores; fold and the sum over images accumulate in fp32).
#include "common.cuh"

namespace tvk {
namespace convunf {

struct Shape {
    int64_t N, Ci, H, W, Co, KH, KW, sh, sw, dh, dw, ph, pw, Ho, Wo;
    int x_cl, y_cl, w_cl, dtype;
    __host__ __device__ int64_t P() const { return Ho * Wo; }
    __host__ __device__ int64_t K() const { return Ci * KH * KW; }
};

// element offset of (n, c, h, w) in a [N, C, H, W] tensor stored plain or channels-last
__device__ __forceinline__ int64_t at4(int cl, int64_t n, int64_t c, int64_t h, int64_t w, int64_t C, int64_t H, int64_t W) {
    return cl ? ((n * H + h) * W + w) * C + c : ((n * C + c) * H + h) * W + w;
}

// cols[n][p][k] = x(n, ci, ho*sh - ph + kh*dh, wo*sw - pw + kw*dw), 0 outside the image
template <typename T>
__global__ void __launch_bounds__(256) unfold_kernel(T* __restrict__ cols, const T* __restrict__ x, Shape g) {
    const int64_t K = g.K(), P = g.P(), taps = g.KH * g.KW, total = g.N * P * K;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t k = i % K, p = (i / K) % P, n = i / (K * P);
        const int64_t ci = g.w_cl ? k % g.Ci : k / taps, tap = g.w_cl ? k / g.Ci : k % taps;
        const int64_t kh = tap / g.KW, kw = tap - kh * g.KW;
        const int64_t ho = p / g.Wo, wo = p - ho * g.Wo;
        const int64_t h = ho * g.sh - g.ph + kh * g.dh, w = wo * g.sw - g.pw + kw * g.dw;
        cols[i] = (h >= 0 && h < g.H && w >= 0 && w < g.W) ? x[at4(g.x_cl, n, ci, h, w, g.Ci, g.H, g.W)] : from_f32<T>(0.f);
    }
}

// dx(n, ci, h, w) = sum over the taps (kh, kw) and output pixels (ho, wo) with ho*sh - ph + kh*dh == h, wo*sw - pw + kw*dw == w
// of dcols[n][ho*Wo + wo][k(ci, tap)]: every input pixel gathers its own contributions in a fixed order, in fp32.
template <typename T>
__global__ void __launch_bounds__(256) fold_kernel(T* __restrict__ dx, const T* __restrict__ dcols, Shape g) {
    const int64_t K = g.K(), P = g.P(), taps = g.KH * g.KW, total = g.N * g.Ci * g.H * g.W;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        // walk the output in its own memory order so that the stores coalesce
        int64_t n, ci, h, w;
        if (g.x_cl) { ci = i % g.Ci; w = (i / g.Ci) % g.W; h = (i / (g.Ci * g.W)) % g.H; n = i / (g.Ci * g.W * g.H); }
        else { w = i % g.W; h = (i / g.W) % g.H; ci = (i / (g.W * g.H)) % g.Ci; n = i / (g.W * g.H * g.Ci); }
        float acc = 0.f;
        for (int64_t kh = 0; kh < g.KH; ++kh) {
            const int64_t hh = h + g.ph - kh * g.dh;
            if (hh < 0 || hh % g.sh != 0) continue;
            const int64_t ho = hh / g.sh;
            if (ho >= g.Ho) continue;
            for (int64_t kw = 0; kw < g.KW; ++kw) {
                const int64_t ww = w + g.pw - kw * g.dw;
                if (ww < 0 || ww % g.sw != 0) continue;
                const int64_t wo = ww / g.sw;
                if (wo >= g.Wo) continue;
                const int64_t tap = kh * g.KW + kw;
                const int64_t k = g.w_cl ? tap * g.Ci + ci : ci * taps + tap;
                acc += to_f32(dcols[(n * P + ho * g.Wo + wo) * K + k]);
            }
        }
        dx[i] = from_f32<T>(acc);
    }
}

static unsigned grid_for(int64_t total) {
    int64_t b = (total + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 32;
    return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

static uint64_t a256(uint64_t v) { return (v + 255) / 256 * 256; }

// The three GEMMs as descriptors. `cols`, `part` may be dummy non-null pointers when only sizes are wanted.
static tvk_gemm_desc gemm_forward(const Shape& g, const void* w, const void* cols, void* y) {
    tvk_gemm_desc d = {};
    d.dtype = g.dtype; d.alpha = 1.f; d.beta = 0.f; d.k = g.K();
    const int64_t P = g.P(), K = g.K();
    if (g.y_cl) {           // all images at once: (N*P x Co) = cols . W^T
        d.batch = 1; d.m = g.N * P; d.n = g.Co;
        d.a = cols; d.a_rs = K; d.a_cs = 1;
        d.b = w; d.b_rs = 1; d.b_cs = K;
        d.c = y; d.c_rs = g.Co;
    } else {                // per image: (Co x P) = W . cols[n]^T, which is NCHW memory
        d.batch = g.N; d.m = g.Co; d.n = P;
        d.a = w; d.a_rs = K; d.a_cs = 1; d.a_bs = 0;
        d.b = cols; d.b_rs = 1; d.b_cs = K; d.b_bs = P * K;
        d.c = y; d.c_rs = P; d.c_bs = g.Co * P;
    }
    return d;
}

static tvk_gemm_desc gemm_dcols(const Shape& g, const void* dy, const void* w, void* dcols) {
    tvk_gemm_desc d = {};
    d.dtype = g.dtype; d.alpha = 1.f; d.beta = 0.f;
    const int64_t P = g.P(), K = g.K();
    d.batch = g.N; d.m = P; d.n = K; d.k = g.Co;
    d.a = dy;               // dY[n]^T: (P x Co)
    if (g.y_cl) { d.a_rs = g.Co; d.a_cs = 1; } else { d.a_rs = 1; d.a_cs = P; }
    d.a_bs = g.Co * P;
    d.b = w; d.b_rs = K; d.b_cs = 1; d.b_bs = 0;
    d.c = dcols; d.c_rs = K; d.c_bs = P * K;
    return d;
}

static tvk_gemm_desc gemm_wgrad(const Shape& g, const void* dy, const void* cols, void* part) {
    tvk_gemm_desc d = {};
    d.dtype = g.dtype; d.alpha = 1.f; d.beta = 0.f;
    const int64_t P = g.P(), K = g.K();
    d.batch = g.N; d.m = g.Co; d.n = K; d.k = P;
    d.a = dy;               // dY[n]: (Co x P)
    if (g.y_cl) { d.a_rs = 1; d.a_cs = g.Co; } else { d.a_rs = P; d.a_cs = 1; }
    d.a_bs = g.Co * P;
    d.b = cols; d.b_rs = K; d.b_cs = 1; d.b_bs = P * K;
    d.c = part; d.c_rs = K; d.c_bs = g.Co * K;
    return d;
}


static int make_shape(const tvk_conv2d_desc* d, Shape* g) {
    TVK_REQUIRE(d->n >= 0 && d->cin > 0 && d->h > 0 && d->w > 0 && d->cout > 0 && d->kh > 0 && d->kw > 0, "tvk_conv2d: bad extent");
    TVK_REQUIRE(d->stride_h >= 1 && d->stride_w >= 1 && d->dilation_h >= 1 && d->dilation_w >= 1, "tvk_conv2d: bad stride or dilation");
    if (d->groups != 1) return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: conv2d with groups (use the depthwise entry points or one call per group)");
    if (!is_float_dtype(d->dtype)) return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: conv2d for dtype %d (fp32, fp16 and bf16 are supported)", d->dtype);
    TVK_REQUIRE(d->pad_h >= 0 && d->pad_w >= 0, "tvk_conv2d: bad padding");
    TVK_REQUIRE(d->layout >= 0 && d->layout <= 7, "tvk_conv2d: unknown layout flags %lld", (long long)d->layout);
    g->N = d->n; g->Ci = d->cin; g->H = d->h; g->W = d->w; g->Co = d->cout; g->KH = d->kh; g->KW = d->kw;
    g->sh = d->stride_h; g->sw = d->stride_w; g->dh = d->dilation_h; g->dw = d->dilation_w; g->dtype = d->dtype;
    g->ph = d->pad_h; g->pw = d->pad_w;
    g->Ho = (d->h + 2 * d->pad_h - d->dilation_h * (d->kh - 1) - 1) / g->sh + 1;
    g->Wo = (d->w + 2 * d->pad_w - d->dilation_w * (d->kw - 1) - 1) / g->sw + 1;
    TVK_REQUIRE(g->Ho > 0 && g->Wo > 0, "tvk_conv2d: the filter does not fit the padded input");
    g->x_cl = (d->layout & TVK_CONV_X_CHANNELS_LAST) ? 1 : 0;
    g->y_cl = (d->layout & TVK_CONV_Y_CHANNELS_LAST) ? 1 : 0;
    g->w_cl = (d->layout & TVK_CONV_W_CHANNELS_LAST) ? 1 : 0;
    return TVK_OK;
}

static int gemm_ws(const tvk_gemm_desc& gd, uint64_t* bytes) {
    *bytes = 0;
    if (gd.batch == 0 || gd.m == 0 || gd.n == 0) return TVK_OK;
    int rc = tvk_gemm_workspace_size(&gd, bytes);
    *bytes = a256(*bytes);
    return rc;
}

// workspace: [cols or dcols][per-image filter-gradient partials (mode 2)][GEMM scratch][reduce scratch (mode 2)]
struct Plan {
    uint64_t cols_b = 0, part_b = 0, gemm_b = 0, red_b = 0;
    uint64_t total() const { return cols_b + part_b + gemm_b + red_b; }
};
static int make_plan(const Shape& g, int mode, Plan* p) {
    void* dummy = (void*)(uintptr_t)256;
    const uint64_t es = dtype_size(g.dtype);
    p->cols_b = a256((uint64_t)g.N * g.P() * g.K() * es);
    int rc;
    if (mode == 0) rc = gemm_ws(gemm_forward(g, dummy, dummy, dummy), &p->gemm_b);
    else if (mode == 1) rc = gemm_ws(gemm_dcols(g, dummy, dummy, dummy), &p->gemm_b);
    else {
        p->part_b = a256((uint64_t)g.N * g.Co * g.K() * es);
        rc = gemm_ws(gemm_wgrad(g, dummy, dummy, dummy), &p->gemm_b);
        if (rc) return rc;
        rc = tvk_reduce_workspace_size(1, g.N, g.Co * g.K(), &p->red_b);
        p->red_b = a256(p->red_b);
    }
    return rc;
}

}  // namespace convunf

int conv2d_unfold_workspace_size(const tvk_conv2d_desc* d, int mode, uint64_t* bytes) {
    convunf::Shape g;
    int rc = convunf::make_shape(d, &g);
    if (rc) return rc;
    if (mode < 0 || mode > 2) return set_error(TVK_ERR_INVALID, "tvk_conv2d_workspace_size: mode must be 0 (forward), 1 (input gradient) or 2 (weight gradient)");
    convunf::Plan p;
    rc = convunf::make_plan(g, mode, &p);
    *bytes = p.total();
    return rc;
}

#define TVK_CONVUNF_PROLOGUE(mode, who)                                                                                         \
    convunf::Shape g;                                                                                                           \
    int rc = convunf::make_shape(d, &g);                                                                                        \
    if (rc) return rc;                                                                                                          \
    convunf::Plan plan;                                                                                                         \
    rc = convunf::make_plan(g, mode, &plan);                                                                                    \
    if (rc) return rc;                                                                                                          \
    TVK_REQUIRE(workspace && workspace_bytes >= plan.total() && ((uintptr_t)workspace & 255) == 0,                              \
                who ": a 256-byte aligned workspace of %llu bytes is required, %llu given", (unsigned long long)plan.total(),   \
                (unsigned long long)workspace_bytes);                                                                           \
    cudaStream_t s = (cudaStream_t)stream;                                                                                      \
    void* cols = workspace;                                                                                                     \
    void* part = (uint8_t*)workspace + plan.cols_b;                                                                             \
    void* gemm_scratch = (uint8_t*)workspace + plan.cols_b + plan.part_b;                                                       \
    void* red_scratch = (uint8_t*)gemm_scratch + plan.gemm_b;                                                                   \
    (void)part; (void)red_scratch

int conv2d_unfold_forward(const tvk_conv2d_desc* d, void* y, const void* x, const void* w, void* workspace, uint64_t workspace_bytes, void* stream) {
    TVK_CONVUNF_PROLOGUE(0, "tvk_conv2d_forward");
    if (g.N == 0) return TVK_OK;
    TVK_DISPATCH_FLOAT(g.dtype, T, (convunf::unfold_kernel<T><<<convunf::grid_for(g.N * g.P() * g.K()), 256, 0, s>>>((T*)cols, (const T*)x, g)));
    rc = launch_status("conv2d unfold");
    if (rc) return rc;
    const tvk_gemm_desc gd = convunf::gemm_forward(g, w, cols, y);
    return tvk_gemm(&gd, plan.gemm_b ? gemm_scratch : nullptr, plan.gemm_b, stream);
}

int conv2d_unfold_backward_input(const tvk_conv2d_desc* d, void* dx, const void* dy, const void* w, void* workspace, uint64_t workspace_bytes, void* stream) {
    TVK_CONVUNF_PROLOGUE(1, "tvk_conv2d_backward_input");
    if (g.N == 0) return TVK_OK;
    const tvk_gemm_desc gd = convunf::gemm_dcols(g, dy, w, cols);
    rc = tvk_gemm(&gd, plan.gemm_b ? gemm_scratch : nullptr, plan.gemm_b, stream);
    if (rc) return rc;
    TVK_DISPATCH_FLOAT(g.dtype, T, (convunf::fold_kernel<T><<<convunf::grid_for(g.N * g.Ci * g.H * g.W), 256, 0, s>>>((T*)dx, (const T*)cols, g)));
    return launch_status("conv2d fold");
}

int conv2d_unfold_backward_weight(const tvk_conv2d_desc* d, void* dw, const void* dy, const void* x, void* workspace, uint64_t workspace_bytes, void* stream) {
    TVK_CONVUNF_PROLOGUE(2, "tvk_conv2d_backward_weight");
    if (g.N == 0) return tvk_fill(g.dtype, dw, 0.0, g.Co * g.K(), stream);
    TVK_DISPATCH_FLOAT(g.dtype, T, (convunf::unfold_kernel<T><<<convunf::grid_for(g.N * g.P() * g.K()), 256, 0, s>>>((T*)cols, (const T*)x, g)));
    rc = launch_status("conv2d unfold");
    if (rc) return rc;
    const tvk_gemm_desc gd = convunf::gemm_wgrad(g, dy, cols, part);
    rc = tvk_gemm(&gd, plan.gemm_b ? gemm_scratch : nullptr, plan.gemm_b, stream);
    if (rc) return rc;
    return tvk_reduce(TVK_R_SUM, g.dtype, g.dtype, dw, part, 1, g.N, g.Co * g.K(), plan.red_b ? red_scratch : nullptr, plan.red_b, stream);
}

}  // namespace tvk
