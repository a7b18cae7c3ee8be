// conv2d forward, input gradient and weight gradient as implicit GEMM on tcgen05 / TMEM, fed by TMA.
//
// Replaces convolution_vulkan / convolution_backward_vulkan and dispatch_conv_shader
// (src/api/ops/conv.cpp:661-685, 1014-1172) and the conv_coop / conv_simd / winograd shaders
// (src/shaders/ops/conv_coop.slang, src/shaders/helpers/conv.slang). The three modes are the
// reference's (conv.cpp:241-245): FORWARD, GRAD_INPUT (stride 2 as four output phases, each a small
// stride-1 convolution over dY, like its sub-pixel phase split conv.cpp:364-382) and GRAD_WEIGHT
// (pixel range split over CTAs into fp32 partials, conv.cpp:1034-1060). Winograd is not used: on
// tcgen05 the direct form is faster at fp16 and has no transform error.
//
// The public tensors are NCHW / OIHW like the reference's (conv.cpp:1106-1108), or channels-last. The kernels read
// channels-last operands (see conv_kernels.cuh for why that layout makes every filter tap a plain TMA box): an NCHW
// input is transposed into the caller's workspace first (16-byte packets through shared memory); outputs are written
// by the epilogue in the caller's layout, NCHW included, with no staged copy. tvk_conv2d_backward transposes an NCHW
// dy once for both gradients.
#include "conv_kernels.cuh"
#include "conv_halo.cuh"

#include <mutex>

namespace tvk {
namespace conv {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
        else
            cudaGetLastError();
    });
    return fn;
}

// Channels-last activation [N, H, W, Cp] as a 4-D map {C, W, H, N}; box {64, bw, bh, bn} walked with `stride` on W and H.
static int encode_nhwc(CUtensorMap* map, int dtype, const void* ptr, int64_t N, int64_t H, int64_t W, int64_t Cp, int bw, int bh, int bn, int stride) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return set_error(TVK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const CUtensorMapDataType dt = dtype == TVK_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    cuuint64_t dims[4] = {(cuuint64_t)Cp, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
    cuuint64_t strides[3] = {(cuuint64_t)Cp * 2, (cuuint64_t)W * Cp * 2, (cuuint64_t)H * W * Cp * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)(bw * stride), (cuuint32_t)(bh * stride), (cuuint32_t)bn};
    cuuint32_t es[4] = {1, (cuuint32_t)stride, (cuuint32_t)stride, 1};
    CUresult r = fn(map, dt, 4, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return set_error(TVK_ERR_CUDA, "cuTensorMapEncodeTiled (activation %lldx%lldx%lldx%lld, box %dx%dx%d, stride %d) failed with code %d", (long long)N,
                         (long long)H, (long long)W, (long long)Cp, bn, bh, bw, stride, (int)r);
    return TVK_OK;
}

// Packed filter [rows, K] (K contiguous) as a 2-D map; box {64, bn}.
static int encode_filter(CUtensorMap* map, int dtype, const void* ptr, int64_t rows, int64_t K, int bn) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return set_error(TVK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const CUtensorMapDataType dt = dtype == TVK_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)bn};
    cuuint32_t es[2] = {1, 1};
    CUresult r = fn(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(TVK_ERR_CUDA, "cuTensorMapEncodeTiled (filter %lld x %lld) failed with code %d", (long long)rows, (long long)K, (int)r);
    return TVK_OK;
}

static int pow2ceil(int64_t v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}
static int64_t pad64(int64_t c) { return (c + 63) / 64 * 64; }
static uint64_t a256(uint64_t v) { return (v + 255) / 256 * 256; }

struct Geo {
    int64_t N, Ci, H, W, Co, KH, KW, s, ph, pw, Ho, Wo, Cip, Cop;
    int taps() const { return (int)(KH * KW); }
};

#define TVK_CONV_SUPPORTED(cond, ...)                                                  \
    do {                                                                               \
        if (!(cond)) return set_error(TVK_ERR_UNSUPPORTED, __VA_ARGS__);               \
    } while (0)

static int make_geo(const tvk_conv2d_desc* d, Geo* g) {
    if (!d) return set_error(TVK_ERR_INVALID, "tvk_conv2d: null descriptor");
    TVK_CONV_SUPPORTED(d->dtype == TVK_F16 || d->dtype == TVK_BF16, "torchvulkan [NOT IMPLEMENTED]: conv2d for dtype %d (fp32, fp16 and bf16 are supported)", d->dtype);
    TVK_REQUIRE(d->n >= 0 && d->cin > 0 && d->h > 0 && d->w > 0 && d->cout > 0 && d->kh > 0 && d->kw > 0, "tvk_conv2d: bad extent");
    TVK_CONV_SUPPORTED(d->stride_h == d->stride_w && (d->stride_h == 1 || d->stride_h == 2), "torchvulkan [NOT IMPLEMENTED]: conv2d stride (%lld, %lld); 1 and 2 are supported",
                (long long)d->stride_h, (long long)d->stride_w);
    TVK_CONV_SUPPORTED(d->dilation_h == 1 && d->dilation_w == 1 && d->groups == 1, "torchvulkan [NOT IMPLEMENTED]: conv2d with dilation or groups");
    TVK_CONV_SUPPORTED(d->kh * d->kw <= kMaxTaps && d->kh <= 64 && d->kw <= 64, "torchvulkan [NOT IMPLEMENTED]: conv2d filter %lld x %lld", (long long)d->kh, (long long)d->kw);
    TVK_REQUIRE(d->pad_h >= 0 && d->pad_w >= 0 && d->pad_h < 64 && d->pad_w < 64, "tvk_conv2d: bad padding");
    TVK_REQUIRE(d->layout >= 0 && d->layout <= 7, "tvk_conv2d: unknown layout flags %lld", (long long)d->layout);
    g->N = d->n; g->Ci = d->cin; g->H = d->h; g->W = d->w; g->Co = d->cout; g->KH = d->kh; g->KW = d->kw; g->s = d->stride_h;
    g->ph = d->pad_h; g->pw = d->pad_w;
    g->Ho = (d->h + 2 * d->pad_h - d->kh) / g->s + 1;
    g->Wo = (d->w + 2 * d->pad_w - d->kw) / g->s + 1;
    TVK_REQUIRE(g->Ho > 0 && g->Wo > 0, "tvk_conv2d: the filter does not fit the padded input");
    TVK_CONV_SUPPORTED(d->n <= 65535 && d->h * d->w < (1 << 30), "torchvulkan [NOT IMPLEMENTED]: conv2d batch above 65535");
    g->Cip = pad64(g->Ci);
    g->Cop = pad64(g->Co);
    return TVK_OK;
}

template <typename T>
static void to_nhwc(T* dst, const T* src, int64_t N, int64_t C, int64_t HW, int64_t Cp, cudaStream_t s) {
    if (sizeof(T) == 2 && HW % 8 == 0 && Cp % 8 == 0 && (((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
        dim3 grid((unsigned)((HW + 63) / 64), (unsigned)((Cp + 63) / 64), (unsigned)N);
        nchw_to_nhwc_packet_kernel<<<grid, 256, 0, s>>>((uint16_t*)dst, (const uint16_t*)src, (int)C, (int)HW, (int)Cp);
        return;
    }
    dim3 grid((unsigned)((HW + 31) / 32), (unsigned)((Cp + 31) / 32), (unsigned)N), block(32, 8);
    nchw_to_nhwc_kernel<T><<<grid, block, 0, s>>>(dst, src, (int)C, (int)HW, (int)Cp);
}
// The channels-last tensor the kernels read, and its channel pitch: the caller's own buffer when it is already
// channels-last with a pitch the TMA accepts (a multiple of 16 bytes), else a copy in `stage` with the channels
// padded to `Cpad` (from NCHW: a transpose; from a narrow channels-last tensor: zero channels appended).
static const uint16_t* stage_act(bool channels_last, const void* src, uint16_t* stage, int64_t N, int64_t C, int64_t HW, int64_t Cpad, int64_t* pitch,
                                 cudaStream_t s) {
    if (channels_last && C % 8 == 0 && ((uintptr_t)src & 15) == 0) {
        *pitch = C;
        return (const uint16_t*)src;
    }
    // the staged copy needs a 16-byte multiple as its channel pitch only: the TMA zero-fills the rest of a 64-channel block
    const int64_t Cs = (C + 7) / 8 * 8;
    (void)Cpad;
    *pitch = Cs;
    if (channels_last) {
        int64_t blocks = (N * HW * Cs + 255) / 256;
        if (blocks > (int64_t)sm_count() * 16) blocks = (int64_t)sm_count() * 16;
        pad_channels_kernel<uint16_t><<<(unsigned)blocks, 256, 0, s>>>(stage, (const uint16_t*)src, N * HW, (int)C, (int)Cs);
    } else {
        to_nhwc<uint16_t>(stage, (const uint16_t*)src, N, C, HW, Cs, s);
    }
    return stage;
}

static int pick_bn(int64_t channels) { return channels <= 64 ? 64 : (channels <= 128 ? 128 : 256); }

template <int BN>
static int launch_fwd(const CUtensorMap& mx, const CUtensorMap& mw, const FwdParams& p, cudaStream_t s) {
    using Cfg = tc::Config<BN>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        TVK_CUDA_CHECK(cudaFuncSetAttribute(conv_fwd_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        attr_set[dev] = true;
    }
    const int64_t grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
    conv_fwd_kernel<BN><<<(unsigned)grid, tc::kThreads, Cfg::kSmemBytes, s>>>(mx, mw, p);
    return launch_status("conv2d implicit GEMM");
}

template <int BN>
static int launch_wgrad(const CUtensorMap& mdy, const CUtensorMap& mx, const WgradParams& p, cudaStream_t s) {
    using Cfg = tc::Config<BN>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        TVK_CUDA_CHECK(cudaFuncSetAttribute(conv_wgrad_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        attr_set[dev] = true;
    }
    const int64_t grid = p.total_items < sm_count() ? p.total_items : sm_count();
    conv_wgrad_kernel<BN><<<(unsigned)grid, tc::kThreads, Cfg::kSmemBytes, s>>>(mdy, mx, p);
    return launch_status("conv2d weight gradient");
}

// Runs conv_fwd_kernel over the pixel grid (Nimg, Ho, Wo) of `p` (tile counts are filled in here).
static int run_fwd(int dtype, const void* act, int64_t N, int64_t H, int64_t W, int64_t Cp, const void* filt, int64_t frows, int64_t fK, FwdParams p,
                   cudaStream_t s) {
    p.tw = pow2ceil(p.Wo) < 128 ? pow2ceil(p.Wo) : 128;
    p.th = pow2ceil(p.Ho) < 128 / p.tw ? pow2ceil(p.Ho) : 128 / p.tw;
    p.tn = 128 / (p.tw * p.th);
    const int bn = pick_bn(p.Cout);
    p.tiles_w = (p.Wo + p.tw - 1) / p.tw;
    p.tiles_h = (p.Ho + p.th - 1) / p.th;
    p.tiles_n = (p.Nimg + p.tn - 1) / p.tn;
    p.tiles_c = (p.Cout + bn - 1) / bn;
    p.total_tiles = (int64_t)p.tiles_w * p.tiles_h * p.tiles_n * p.tiles_c;
    p.dtype = dtype;
    p.status = device_status_word();
    const uint32_t fmt = dtype == TVK_F16 ? 0u : 1u;
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(tc::BM >> 4) << 24);
    CUtensorMap mx, mw;
    int rc = encode_nhwc(&mx, dtype, act, N, H, W, Cp, p.tw, p.th, p.tn, p.in_stride);
    if (rc) return rc;
    rc = encode_filter(&mw, dtype, filt, frows, fK, bn);
    if (rc) return rc;
    switch (bn) {
        case 64: return launch_fwd<64>(mx, mw, p, s);
        case 128: return launch_fwd<128>(mx, mw, p, s);
        default: return launch_fwd<256>(mx, mw, p, s);
    }
}

// The 3x3 / stride 1 / padding 1 kernel with resident filters (conv_halo.cuh) applies when one 64-channel block
// covers the contraction and one 64-column tile the output channels.
static bool halo_eligible(const Geo& g, int64_t in_channels_padded, int64_t out_channels) {
    static const bool off = getenv("TORCHVULKAN_CONV_NO_HALO") != nullptr;
    return !off && g.KH == 3 && g.KW == 3 && g.s == 1 && g.ph == 1 && g.pw == 1 && in_channels_padded == 64 && out_channels <= 64;
}

static int run_halo(int dtype, const void* act, int64_t N, int64_t H, int64_t W, int64_t pitch, const void* filt, int64_t frows, HaloParams p,
                    cudaStream_t s) {
    p.N = (int)N; p.H = (int)H; p.W = (int)W;
    p.tiles_w = (int)((W + kHaloW - 1) / kHaloW);
    p.tiles_h = (int)((H + kHaloH - 1) / kHaloH);
    p.total_tiles = (int64_t)p.tiles_w * p.tiles_h * N;
    p.dtype = dtype;
    p.status = device_status_word();
    const uint32_t fmt = dtype == TVK_F16 ? 0u : 1u;
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(tc::BM >> 4) << 24);
    CUtensorMap mx, mw;
    int rc = encode_nhwc(&mx, dtype, act, N, H, W, pitch, kHaloW + 2, kHaloH + 2, 1, 1);
    if (rc) return rc;
    rc = encode_filter(&mw, dtype, filt, frows, 9 * 64, 64);
    if (rc) return rc;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        TVK_CUDA_CHECK(cudaFuncSetAttribute(conv3x3_halo_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kHaloSmemBytes));
        attr_set[dev] = true;
    }
    const int64_t grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
    conv3x3_halo_kernel<<<(unsigned)grid, tc::kThreads, kHaloSmemBytes, s>>>(mx, mw, p);
    return launch_status("conv2d 3x3 halo kernel");
}

struct HaloWgradPlan {
    int blocks_w, blocks_h, splits;
    int64_t kblocks, kb_per_split;
};
static HaloWgradPlan plan_halo_wgrad(const Geo& g) {
    HaloWgradPlan w;
    w.blocks_w = (int)((g.W + 7) / 8);
    w.blocks_h = (int)((g.H + 7) / 8);
    w.kblocks = (int64_t)w.blocks_w * w.blocks_h * g.N;
    int64_t splits = (2 * (int64_t)sm_count() + 2) / 3;          // three filter rows per split: about two items per SM
    if (splits > w.kblocks) splits = w.kblocks;
    if (splits < 1) splits = 1;
    w.kb_per_split = (w.kblocks + splits - 1) / splits;
    if (w.kb_per_split < 1) w.kb_per_split = 1;
    w.splits = (int)((w.kblocks + w.kb_per_split - 1) / w.kb_per_split);
    if (w.splits < 1) w.splits = 1;
    return w;
}

static int run_halo_wgrad(int dtype, const void* dya, int64_t dy_pitch, const void* xa, int64_t x_pitch, const Geo& g, float* partial, cudaStream_t s) {
    const HaloWgradPlan w = plan_halo_wgrad(g);
    HaloWgradParams p = {};
    p.N = (int)g.N; p.H = (int)g.H; p.W = (int)g.W;
    p.blocks_w = w.blocks_w; p.blocks_h = w.blocks_h; p.kblocks = w.kblocks;
    p.splits = w.splits; p.kb_per_split = w.kb_per_split; p.total_items = 3 * w.splits;
    p.O = (int)g.Co;
    p.partial = partial;
    p.status = device_status_word();
    const uint32_t fmt = dtype == TVK_F16 ? 0u : 1u;
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(192 >> 3) << 17) | ((uint32_t)(tc::BM >> 4) << 24);
    CUtensorMap mdy, mx;
    int rc = encode_nhwc(&mdy, dtype, dya, g.N, g.Ho, g.Wo, dy_pitch, 8, 8, 1, 1);
    if (rc) return rc;
    rc = encode_nhwc(&mx, dtype, xa, g.N, g.H, g.W, x_pitch, 10, 8, 1, 1);
    if (rc) return rc;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        TVK_CUDA_CHECK(cudaFuncSetAttribute(conv3x3_wgrad_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWgSmemBytes));
        attr_set[dev] = true;
    }
    const int grid = p.total_items < sm_count() ? p.total_items : sm_count();
    conv3x3_wgrad_rows_kernel<<<(unsigned)grid, tc::kThreads, kWgSmemBytes, s>>>(mdy, mx, p);
    return launch_status("conv2d 3x3 weight gradient");
}

struct WgradPlan {
    int tn, th, tw, blocks_w, blocks_h, blocks_n, splits, bn, tiles_o, tiles_i;
    int64_t kblocks, kb_per_split;
};
static WgradPlan plan_wgrad(const Geo& g) {
    WgradPlan w;
    w.tw = pow2ceil(g.Wo) < 64 ? pow2ceil(g.Wo) : 64;
    w.th = pow2ceil(g.Ho) < 64 / w.tw ? pow2ceil(g.Ho) : 64 / w.tw;
    w.tn = 64 / (w.tw * w.th);
    w.blocks_w = (int)((g.Wo + w.tw - 1) / w.tw);
    w.blocks_h = (int)((g.Ho + w.th - 1) / w.th);
    w.blocks_n = (int)((g.N + w.tn - 1) / w.tn);
    w.kblocks = (int64_t)w.blocks_w * w.blocks_h * w.blocks_n;
    w.bn = pick_bn(g.Cip);
    w.tiles_o = (int)((g.Co + 127) / 128);
    w.tiles_i = (int)((g.Cip + w.bn - 1) / w.bn);
    const int64_t items = (int64_t)g.taps() * w.tiles_o * w.tiles_i;
    // One work item per SM: every extra split is another fp32 copy of the filter gradient to write and to fold (two items
    // per SM measured 1 % slower on the ResNet step for twice the partial traffic).
    int64_t splits = (int64_t)sm_count() / items;
    if (splits > w.kblocks) splits = w.kblocks;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    w.kb_per_split = (w.kblocks + splits - 1) / splits;
    if (w.kb_per_split < 1) w.kb_per_split = 1;
    w.splits = (int)((w.kblocks + w.kb_per_split - 1) / w.kb_per_split);
    if (w.splits < 1) w.splits = 1;
    return w;
}

}  // namespace conv
}  // namespace tvk

namespace tvk {
// fp32 tensors and the geometries the kernels of this file do not take: unfold + GEMM (conv_unfold.cu)
int conv2d_unfold_workspace_size(const tvk_conv2d_desc* d, int mode, uint64_t* bytes);
int conv2d_unfold_forward(const tvk_conv2d_desc* d, void* y, const void* x, const void* w, void* workspace, uint64_t workspace_bytes, void* stream);
int conv2d_unfold_backward_input(const tvk_conv2d_desc* d, void* dx, const void* dy, const void* w, void* workspace, uint64_t workspace_bytes, void* stream);
int conv2d_unfold_backward_weight(const tvk_conv2d_desc* d, void* dw, const void* dy, const void* x, void* workspace, uint64_t workspace_bytes, void* stream);
}  // namespace tvk

using namespace tvk;
using namespace tvk::conv;

// fp32 tensors, and half tensors with dilation, a stride above 2, unequal strides or a filter of more taps than the
// implicit-GEMM kernels walk, take the unfold route
static bool unfold_route(const tvk_conv2d_desc* d) {
    if (!d) return false;
    if (d->dtype == TVK_F32) return true;
    if (d->dtype != TVK_F16 && d->dtype != TVK_BF16) return false;
    if (d->groups != 1 || d->stride_h < 1 || d->stride_w < 1 || d->dilation_h < 1 || d->dilation_w < 1 || d->kh < 1 || d->kw < 1) return false;
    return d->stride_h != d->stride_w || d->stride_h > 2 || d->dilation_h != 1 || d->dilation_w != 1 || d->kh * d->kw > kMaxTaps || d->kh > 64 || d->kw > 64 ||
           d->pad_h >= 64 || d->pad_w >= 64;
}

extern "C" {

int tvk_conv2d_workspace_size(const tvk_conv2d_desc* d, int mode, uint64_t* bytes) {
    if (!bytes) return set_error(TVK_ERR_INVALID, "tvk_conv2d_workspace_size: null output");
    if (unfold_route(d)) {
        if (mode != 3) return conv2d_unfold_workspace_size(d, mode, bytes);
        uint64_t b1 = 0, b2 = 0;      // both gradients: the two products run one after the other in the same workspace
        int rc1 = conv2d_unfold_workspace_size(d, 1, &b1);
        if (rc1) return rc1;
        rc1 = conv2d_unfold_workspace_size(d, 2, &b2);
        if (rc1) return rc1;
        *bytes = b1 > b2 ? b1 : b2;
        return TVK_OK;
    }
    Geo g;
    int rc = make_geo(d, &g);
    if (rc) return rc;
    const uint64_t x_b = a256((uint64_t)g.N * g.H * g.W * g.Cip * 2), dy_b = a256((uint64_t)g.N * g.Ho * g.Wo * g.Cop * 2);
    const uint64_t w_b = a256((uint64_t)g.Cop * g.taps() * g.Cip * 2);   // covers [O, taps, Ip] and [I, taps, Op]
    if (mode == 0) *bytes = x_b + w_b;          // staged input and packed filter; the output is written in place
    else if (mode == 1) *bytes = dy_b + w_b;
    else if (mode == 2) {
        const WgradPlan w = plan_wgrad(g);
        uint64_t splits = (uint64_t)w.splits;
        if (halo_eligible(g, g.Cip, g.Co) && (uint64_t)plan_halo_wgrad(g).splits > splits) splits = (uint64_t)plan_halo_wgrad(g).splits;
        *bytes = x_b + dy_b + a256(splits * g.taps() * g.Co * g.Cip * 4);
    } else if (mode == 3) {
        // both gradients in one call: dy staged channels-last once, then the larger of the two workspaces
        tvk_conv2d_desc d2 = *d;
        d2.layout |= TVK_CONV_Y_CHANNELS_LAST;
        uint64_t b1 = 0, b2 = 0;
        int rc1 = tvk_conv2d_workspace_size(&d2, 1, &b1);
        if (rc1) return rc1;
        rc1 = tvk_conv2d_workspace_size(&d2, 2, &b2);
        if (rc1) return rc1;
        *bytes = dy_b + (b1 > b2 ? b1 : b2);
    } else return set_error(TVK_ERR_INVALID, "tvk_conv2d_workspace_size: mode must be 0 (forward), 1 (input gradient), 2 (weight gradient) or 3 (both gradients)");
    return TVK_OK;
}

#define TVK_CONV_WS_CHECK(mode, who)                                                                                        \
    uint64_t need = 0;                                                                                                      \
    tvk_conv2d_workspace_size(d, mode, &need);                                                                              \
    TVK_REQUIRE(workspace && workspace_bytes >= need && ((uintptr_t)workspace & 255) == 0,                                  \
                who ": a 256-byte aligned workspace of %llu bytes is required, %llu given", (unsigned long long)need,       \
                (unsigned long long)workspace_bytes)

int tvk_conv2d_forward(const tvk_conv2d_desc* d, void* y, const void* x, const void* w, void* workspace, uint64_t workspace_bytes, void* stream) {
    if (unfold_route(d)) {
        TVK_REQUIRE(d->n == 0 || (y && x && w), "tvk_conv2d_forward: null pointer");
        return conv2d_unfold_forward(d, y, x, w, workspace, workspace_bytes, stream);
    }
    Geo g;
    int rc = make_geo(d, &g);
    if (rc) return rc;
    if (g.N == 0) return TVK_OK;
    TVK_REQUIRE(y && x && w, "tvk_conv2d_forward: null pointer");
    TVK_CONV_WS_CHECK(0, "tvk_conv2d_forward");
    cudaStream_t s = (cudaStream_t)stream;
    uint16_t* xs = (uint16_t*)workspace;
    uint16_t* wp = (uint16_t*)((uint8_t*)xs + a256((uint64_t)g.N * g.H * g.W * g.Cip * 2));
    uint16_t* ys = nullptr;
    int64_t x_pitch = 0;
    const uint16_t* xa = stage_act((d->layout & TVK_CONV_X_CHANNELS_LAST) != 0, x, xs, g.N, g.Ci, g.H * g.W, g.Cip, &x_pitch, s);
    if ((d->layout & TVK_CONV_W_CHANNELS_LAST) && g.Cip == g.Ci && ((uintptr_t)w & 15) == 0) {
        // a channels-last filter [O, taps, I] with whole 64-channel blocks IS the packed forward operand: read it in place
        wp = (uint16_t*)w;
    } else {
        pack_filter_kernel<uint16_t><<<sm_count() * 2, 256, 0, s>>>(wp, (const uint16_t*)w, (int)g.Co, (int)g.Ci, g.taps(), (int)g.Cip, 0,
                                                                    (d->layout & TVK_CONV_W_CHANNELS_LAST) ? 1 : 0);
    }
    // the kernels write the caller's tensor themselves in either layout (their native channels-last rows, or NCHW planes
    // from the epilogue: a lane is a pixel, so a channel's stores run along the plane)
    const int y_nchw = (d->layout & TVK_CONV_Y_CHANNELS_LAST) ? 0 : 1;
    ys = (uint16_t*)y;
    if (halo_eligible(g, g.Cip, g.Co)) {
        HaloParams hp = {};
        for (int t = 0; t < 9; ++t) { hp.dh[t] = (int8_t)(t / 3 - 1); hp.dw[t] = (int8_t)(t % 3 - 1); hp.wtap[t] = (int16_t)t; }
        hp.OC = (int)g.Co; hp.Cout = (int)g.Co; hp.out = ys; hp.out_nchw = y_nchw;
        rc = run_halo(d->dtype, xa, g.N, g.H, g.W, x_pitch, wp, g.Co, hp, s);
        if (rc) return rc;
        return launch_status("conv2d forward");
    }
    FwdParams p = {};
    p.Nimg = (int)g.N; p.Ho = (int)g.Ho; p.Wo = (int)g.Wo;
    p.in_stride = (int)g.s;
    p.ntaps = g.taps(); p.cblocks = (int)(g.Cip / 64);
    for (int kh = 0; kh < g.KH; ++kh)
        for (int kw = 0; kw < g.KW; ++kw) {
            const int t = kh * (int)g.KW + kw;
            p.dh[t] = (int8_t)(kh - g.ph); p.dw[t] = (int8_t)(kw - g.pw); p.wtap[t] = (int16_t)t;
        }
    p.OH = (int)g.Ho; p.OW = (int)g.Wo; p.os = 1; p.oh0 = 0; p.ow0 = 0; p.OC = (int)g.Co; p.Cout = (int)g.Co;
    p.out = ys; p.out_nchw = y_nchw;
    rc = run_fwd(d->dtype, xa, g.N, g.H, g.W, x_pitch, wp, g.Co, (int64_t)g.taps() * g.Cip, p, s);
    if (rc) return rc;
    return launch_status("conv2d forward");
}

int tvk_conv2d_backward_input(const tvk_conv2d_desc* d, void* dx, const void* dy, const void* w, void* workspace, uint64_t workspace_bytes,
                              void* stream) {
    if (unfold_route(d)) {
        TVK_REQUIRE(d->n == 0 || (dx && dy && w), "tvk_conv2d_backward_input: null pointer");
        return conv2d_unfold_backward_input(d, dx, dy, w, workspace, workspace_bytes, stream);
    }
    Geo g;
    int rc = make_geo(d, &g);
    if (rc) return rc;
    if (g.N == 0) return TVK_OK;
    TVK_REQUIRE(dx && dy && w, "tvk_conv2d_backward_input: null pointer");
    TVK_CONV_WS_CHECK(1, "tvk_conv2d_backward_input");
    cudaStream_t s = (cudaStream_t)stream;
    uint16_t* dys = (uint16_t*)workspace;
    uint16_t* wp = (uint16_t*)((uint8_t*)dys + a256((uint64_t)g.N * g.Ho * g.Wo * g.Cop * 2));
    uint16_t* dxs = nullptr;
    int64_t dy_pitch = 0;
    const uint16_t* dya = stage_act((d->layout & TVK_CONV_Y_CHANNELS_LAST) != 0, dy, dys, g.N, g.Co, g.Ho * g.Wo, g.Cop, &dy_pitch, s);
    pack_filter_kernel<uint16_t><<<sm_count() * 2, 256, 0, s>>>(wp, (const uint16_t*)w, (int)g.Co, (int)g.Ci, g.taps(), (int)g.Cop, 1,
                                                                (d->layout & TVK_CONV_W_CHANNELS_LAST) ? 1 : 0);
    const int dx_nchw = (d->layout & TVK_CONV_X_CHANNELS_LAST) ? 0 : 1;
    dxs = (uint16_t*)dx;
    if (halo_eligible(g, g.Cop, g.Ci)) {
        // dx[h, w] = sum over taps of dy[h + 1 - kh, w + 1 - kw] * w[:, :, kh, kw]^T
        HaloParams hp = {};
        for (int t = 0; t < 9; ++t) { hp.dh[t] = (int8_t)(1 - t / 3); hp.dw[t] = (int8_t)(1 - t % 3); hp.wtap[t] = (int16_t)t; }
        hp.OC = (int)g.Ci; hp.Cout = (int)g.Ci; hp.out = dxs; hp.out_nchw = dx_nchw;
        rc = run_halo(d->dtype, dya, g.N, g.Ho, g.Wo, dy_pitch, wp, g.Ci, hp, s);
        if (rc) return rc;
        return launch_status("conv2d input gradient");
    }
    const int S = (int)g.s;
    bool zero_first = false;
    // Output rows/columns that no dY element reaches (the filter does not tile the padded input exactly) and
    // phases without any tap are zero: clear the staging buffer once when either can happen.
    for (int php = 0; php < S; ++php) {
        int nh = 0, nw = 0;
        for (int kh = 0; kh < g.KH; ++kh) nh += ((php + g.ph - kh) % S == 0);
        for (int kw = 0; kw < g.KW; ++kw) nw += ((php + g.pw - kw) % S == 0);
        if (nh == 0 || nw == 0) zero_first = true;
    }
    if (zero_first) TVK_CUDA_CHECK(cudaMemsetAsync(dxs, 0, (size_t)g.N * g.H * g.W * g.Ci * 2, s));
    for (int php = 0; php < S; ++php) {
        for (int pwp = 0; pwp < S; ++pwp) {
            FwdParams p = {};
            p.Nimg = (int)g.N;
            p.Ho = (int)((g.H - php + S - 1) / S);
            p.Wo = (int)((g.W - pwp + S - 1) / S);
            if (p.Ho <= 0 || p.Wo <= 0) continue;
            p.in_stride = 1;
            p.cblocks = (int)(g.Cop / 64);
            int nt = 0;
            for (int kh = 0; kh < g.KH; ++kh) {
                const int eh = php + (int)g.ph - kh;
                if (((eh % S) + S) % S != 0) continue;
                for (int kw = 0; kw < g.KW; ++kw) {
                    const int ew = pwp + (int)g.pw - kw;
                    if (((ew % S) + S) % S != 0) continue;
                    // dY row = (S*hh + php + pad - kh) / S = hh + eh / S  (eh is a multiple of S, possibly negative)
                    p.dh[nt] = (int8_t)(eh / S); p.dw[nt] = (int8_t)(ew / S); p.wtap[nt] = (int16_t)(kh * g.KW + kw);
                    ++nt;
                }
            }
            if (nt == 0) continue;
            p.ntaps = nt;
            p.OH = (int)g.H; p.OW = (int)g.W; p.os = S; p.oh0 = php; p.ow0 = pwp; p.OC = (int)g.Ci; p.Cout = (int)g.Ci;
            p.out = dxs; p.out_nchw = dx_nchw;
            rc = run_fwd(d->dtype, dya, g.N, g.Ho, g.Wo, dy_pitch, wp, g.Ci, (int64_t)g.taps() * g.Cop, p, s);
            if (rc) return rc;
        }
    }
    return launch_status("conv2d input gradient");
}

int tvk_conv2d_backward_weight(const tvk_conv2d_desc* d, void* dw, const void* dy, const void* x, void* workspace, uint64_t workspace_bytes,
                               void* stream) {
    if (unfold_route(d)) {
        TVK_REQUIRE(dw && (d->n == 0 || (dy && x)), "tvk_conv2d_backward_weight: null pointer");
        return conv2d_unfold_backward_weight(d, dw, dy, x, workspace, workspace_bytes, stream);
    }
    Geo g;
    int rc = make_geo(d, &g);
    if (rc) return rc;
    TVK_REQUIRE(dw, "tvk_conv2d_backward_weight: null output");
    if (g.N == 0) return tvk_fill(d->dtype, dw, 0.0, g.Co * g.Ci * g.taps(), stream);
    TVK_REQUIRE(dy && x, "tvk_conv2d_backward_weight: null pointer");
    TVK_CONV_WS_CHECK(2, "tvk_conv2d_backward_weight");
    cudaStream_t s = (cudaStream_t)stream;
    const WgradPlan wpn = plan_wgrad(g);
    uint16_t* xs = (uint16_t*)workspace;
    uint16_t* dys = (uint16_t*)((uint8_t*)xs + a256((uint64_t)g.N * g.H * g.W * g.Cip * 2));
    float* partial = (float*)((uint8_t*)dys + a256((uint64_t)g.N * g.Ho * g.Wo * g.Cop * 2));
    int64_t x_pitch = 0, dy_pitch = 0;
    const uint16_t* xa = stage_act((d->layout & TVK_CONV_X_CHANNELS_LAST) != 0, x, xs, g.N, g.Ci, g.H * g.W, g.Cip, &x_pitch, s);
    const uint16_t* dya = stage_act((d->layout & TVK_CONV_Y_CHANNELS_LAST) != 0, dy, dys, g.N, g.Co, g.Ho * g.Wo, g.Cop, &dy_pitch, s);
    if (halo_eligible(g, g.Cip, g.Co)) {
        rc = run_halo_wgrad(d->dtype, dya, dy_pitch, xa, x_pitch, g, partial, s);
        if (rc) return rc;
        const int64_t total = g.Co * g.Ci * 9;
        int64_t blocks = (total + 255) / 256;
        if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
        const int hsplits = plan_halo_wgrad(g).splits, cl = (d->layout & TVK_CONV_W_CHANNELS_LAST) ? 1 : 0;
        if (d->dtype == TVK_F16) wgrad_finalize_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>((__half*)dw, partial, hsplits, 9, (int)g.Co, (int)g.Ci, 64, cl);
        else wgrad_finalize_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>((__nv_bfloat16*)dw, partial, hsplits, 9, (int)g.Co, (int)g.Ci, 64, cl);
        return launch_status("conv2d weight gradient");
    }
    WgradParams p = {};
    p.tn = wpn.tn; p.th = wpn.th; p.tw = wpn.tw;
    p.blocks_w = wpn.blocks_w; p.blocks_h = wpn.blocks_h; p.blocks_n = wpn.blocks_n; p.kblocks = wpn.kblocks;
    p.splits = wpn.splits; p.kb_per_split = wpn.kb_per_split;
    p.ntaps = g.taps(); p.tiles_o = wpn.tiles_o; p.tiles_i = wpn.tiles_i;
    p.total_items = (int64_t)p.ntaps * p.tiles_o * p.tiles_i * p.splits;
    p.in_stride = (int)g.s;
    for (int kh = 0; kh < g.KH; ++kh)
        for (int kw = 0; kw < g.KW; ++kw) {
            const int t = kh * (int)g.KW + kw;
            p.dh[t] = (int8_t)(kh - g.ph); p.dw[t] = (int8_t)(kw - g.pw);
        }
    p.O = (int)g.Co; p.I = (int)g.Ci; p.Ip = (int)g.Cip;
    p.partial = partial;
    p.status = device_status_word();
    const uint32_t fmt = d->dtype == TVK_F16 ? 0u : 1u;
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(wpn.bn >> 3) << 17) | ((uint32_t)(tc::BM >> 4) << 24);
    CUtensorMap mdy, mx;
    rc = encode_nhwc(&mdy, d->dtype, dya, g.N, g.Ho, g.Wo, dy_pitch, p.tw, p.th, p.tn, 1);
    if (rc) return rc;
    rc = encode_nhwc(&mx, d->dtype, xa, g.N, g.H, g.W, x_pitch, p.tw, p.th, p.tn, (int)g.s);
    if (rc) return rc;
    switch (wpn.bn) {
        case 64: rc = launch_wgrad<64>(mdy, mx, p, s); break;
        case 128: rc = launch_wgrad<128>(mdy, mx, p, s); break;
        default: rc = launch_wgrad<256>(mdy, mx, p, s); break;
    }
    if (rc) return rc;
    const int64_t total = g.Co * g.Ci * g.taps();
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
    const int dw_cl = (d->layout & TVK_CONV_W_CHANNELS_LAST) ? 1 : 0;
    if (d->dtype == TVK_F16) wgrad_finalize_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>((__half*)dw, partial, p.splits, p.ntaps, p.O, p.I, p.Ip, dw_cl);
    else wgrad_finalize_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>((__nv_bfloat16*)dw, partial, p.splits, p.ntaps, p.O, p.I, p.Ip, dw_cl);
    return launch_status("conv2d weight gradient");
}

int tvk_conv2d_backward(const tvk_conv2d_desc* d, void* dx, void* dw, const void* dy, const void* x, const void* w, void* workspace,
                        uint64_t workspace_bytes, void* stream) {
    if (!d) return set_error(TVK_ERR_INVALID, "tvk_conv2d_backward: null descriptor");
    TVK_REQUIRE(dx || dw, "tvk_conv2d_backward: neither gradient requested");
    tvk_conv2d_desc d2 = *d;
    const void* dy_used = dy;
    uint8_t* ws = (uint8_t*)workspace;
    uint64_t left = workspace_bytes;
    if (!unfold_route(d)) {
        Geo g;
        int rc = make_geo(d, &g);
        if (rc) return rc;
        TVK_CONV_WS_CHECK(3, "tvk_conv2d_backward");
        // an NCHW dy would be transposed by each of the two kernels' staging: do it once here and hand both the channels-last copy
        if (dx && dw && g.N > 0 && dy && !(d->layout & TVK_CONV_Y_CHANNELS_LAST) && g.Co % 8 == 0) {
            to_nhwc<uint16_t>((uint16_t*)ws, (const uint16_t*)dy, g.N, g.Co, g.Ho * g.Wo, g.Co, (cudaStream_t)stream);
            dy_used = ws;
            d2.layout |= TVK_CONV_Y_CHANNELS_LAST;
        }
        const uint64_t dy_b = a256((uint64_t)g.N * g.Ho * g.Wo * g.Cop * 2);
        ws += dy_b;
        left -= dy_b;
    }
    if (dx) {
        int rc = tvk_conv2d_backward_input(&d2, dx, dy_used, w, ws, left, stream);
        if (rc) return rc;
    }
    if (dw) {
        int rc = tvk_conv2d_backward_weight(&d2, dw, dy_used, x, ws, left, stream);
        if (rc) return rc;
    }
    return TVK_OK;
}

}  // extern "C"
