// Scaled dot-product attention, forward and backward: causal or full, grouped-query heads.
//
// Replaces sdpa_forward_vulkan / sdpa_backward_vulkan (src/api/ops/attention.cpp:395-480, 641-749)
// and the attention_coop / attention_simd shaders (src/shaders/ops/attention_coop.slang:117-301).
// Semantics kept from the reference: fp32 log-sum-exp output; probabilities are rounded to the
// input dtype before the P.V product (attention_coop.slang:164-175); a query row without any
// unmasked key yields out = 0 and lse = +inf, and backward treats lse = +inf as p = 0
// (attention_coop.slang:203-222, 299-301); K/V heads are shared by Hq/Hk query heads
// (kvh = h / GROUP); backward = delta (sum dO*O), then dV, dK, dQ from saved LSE
// (attention.cpp:641-665).
//
// Structure here: the contractions run on the tcgen05 GEMM of gemm.cu and the softmax on row
// kernels. All query heads of one KV group are folded into the M dimension: for tensors laid
// out [B, H, L, D] the rows (g, l) of a group are adjacent, so Q_group is a plain
// [G*L, D] matrix, scores are [G*L, S] and the K/V gradients come out of one GEMM per (b, kvh)
// whose contraction runs over all G*L rows — no per-head loop and no atomics. Scores are kept
// in fp32 between the QK^T product and the softmax.
#include "common.cuh"
#include "attention_fused.cuh"
#include "attention_fused_bwd.cuh"

#include <cuda.h>
#include <mutex>

namespace tvk {

// One CTA of 128 threads per score row. scores: fp32 [rows, S] (raw q.k); writes P (T) and lse.
template <typename T>
__global__ void __launch_bounds__(128) attn_softmax_kernel(T* __restrict__ P, float* __restrict__ lse, const float* __restrict__ scores, int64_t L,
                                                          int64_t S, float scale, int causal) {
    __shared__ float smem[33];
    const int64_t row = blockIdx.x;
    const int64_t l = row % L;
    // causal mask aligned to the top-left corner (key j is visible when j <= l), as the reference masks key > row
    // (src/api/ops/attention.cpp:107-112, src/shaders/ops/attention_coop.slang:53-56)
    const int64_t limit = causal ? (l + 1) : S;
    const int64_t nvis = limit < 0 ? 0 : (limit > S ? S : limit);
    const float* s = scores + row * S;
    T* p = P + row * S;
    float m = -INFINITY;
    for (int64_t j = threadIdx.x; j < nvis; j += blockDim.x) m = fmaxf(m, s[j] * scale);
    m = block_max(m, smem);
    float sum = 0.f;
    for (int64_t j = threadIdx.x; j < nvis; j += blockDim.x) sum += expf(s[j] * scale - m);
    sum = block_sum(sum, smem);
    if (nvis == 0) {
        for (int64_t j = threadIdx.x; j < S; j += blockDim.x) p[j] = from_f32<T>(0.f);
        if (threadIdx.x == 0) lse[row] = INFINITY;
        return;
    }
    const float inv = 1.0f / sum;
    for (int64_t j = threadIdx.x; j < S; j += blockDim.x) p[j] = from_f32<T>(j < nvis ? expf(s[j] * scale - m) * inv : 0.f);
    if (threadIdx.x == 0) lse[row] = m + logf(sum);
}

// delta[row] = sum_d dO[row, d] * O[row, d] for two-byte types with 16-byte aligned rows: eight lanes per row, a 16-byte
// packet of both tensors per lane and step, so a warp covers four rows and every load instruction moves 512 bytes.
template <typename T>
__global__ void __launch_bounds__(256) attn_delta_vec_kernel(float* __restrict__ delta, const T* __restrict__ dO, const T* __restrict__ O, int64_t rows, int D) {
    const int64_t row = ((int64_t)blockIdx.x * 256 + threadIdx.x) >> 3;
    const int sub = threadIdx.x & 7;
    float acc = 0.f;
    if (row < rows) {
        constexpr int N = 16 / (int)sizeof(T);       // elements per 16-byte packet
        for (int d = sub * N; d < D; d += 8 * N) {
            const uint4 a = __ldcs((const uint4*)(dO + row * D + d)), b = __ldcs((const uint4*)(O + row * D + d));
            const T* pa = (const T*)&a;
            const T* pb = (const T*)&b;
#pragma unroll
            for (int e = 0; e < N; ++e) acc += to_f32(pa[e]) * to_f32(pb[e]);
        }
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    if (row < rows && sub == 0) delta[row] = acc;
}

// delta[row] = sum_d dO[row, d] * O[row, d]; one warp per row.
template <typename T>
__global__ void __launch_bounds__(128) attn_delta_kernel(float* __restrict__ delta, const T* __restrict__ dO, const T* __restrict__ O, int64_t rows, int64_t D) {
    const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    float acc = 0.f;
    for (int64_t d = lane; d < D; d += 32) acc += to_f32(dO[row * D + d]) * to_f32(O[row * D + d]);
    acc = warp_sum(acc);
    if (lane == 0) delta[row] = acc;
}

constexpr float kDsScale = 1024.f;

// Recomputes p = exp(s*scale - lse) and forms dS = p * (dP - delta) * scale. Writes P and dS (T).
template <typename T>
__global__ void __launch_bounds__(128) attn_dsoftmax_kernel(T* __restrict__ P, T* __restrict__ dS, const float* __restrict__ scores, const float* __restrict__ dP,
                                                           const float* __restrict__ lse, const float* __restrict__ delta, int64_t L, int64_t S,
                                                           float scale, int causal) {
    const int64_t row = blockIdx.x;
    const int64_t l = row % L;
    const int64_t limit = causal ? (l + 1) : S;
    const int64_t nvis = limit < 0 ? 0 : (limit > S ? S : limit);
    const float ls = lse[row], dl = delta[row];
    const bool dead = !(ls < INFINITY);   // +inf (or NaN): the row attended to nothing
    const float* s = scores + row * S;
    const float* g = dP + row * S;
    for (int64_t j = threadIdx.x; j < S; j += blockDim.x) {
        float p = 0.f;
        if (!dead && j < nvis) p = expf(s[j] * scale - ls);
        // the forward pass multiplied V by the rounded probabilities: differentiate that function
        const float pr = to_f32(from_f32<T>(p));
        P[row * S + j] = from_f32<T>(p);
        // dS is tiny next to the probabilities (it carries the upstream gradient): it is stored scaled by
        // kDsScale so that it does not fall into fp16's subnormal range; the dQ/dK products undo the scale.
        float ds = pr * (g[j] - dl) * scale * kDsScale;
        ds = fminf(fmaxf(ds, -60000.f), 60000.f);
        dS[row * S + j] = from_f32<T>(ds);
    }
}

// ---- the same two row kernels for S <= 1024, S % 4 == 0: one warp per row, the row in registers, 128-bit loads ----
template <typename T> __device__ __forceinline__ uint2 pack4(float a, float b, float c, float d);
template <> __device__ __forceinline__ uint2 pack4<__half>(float a, float b, float c, float d) {
    __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
    return make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
}
template <> __device__ __forceinline__ uint2 pack4<__nv_bfloat16>(float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    return make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
}
template <> __device__ __forceinline__ uint2 pack4<float>(float, float, float, float) { return make_uint2(0, 0); }   // not instantiated at run time

template <typename T>
__global__ void __launch_bounds__(256) attn_softmax_warp_kernel(T* __restrict__ P, float* __restrict__ lse, const float* __restrict__ scores, int64_t rows,
                                                               int64_t L, int S, float scale, int causal) {
    constexpr int MAXV = 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + warp;
    if (row >= rows) return;
    const int64_t l = row % L;
    const int64_t limit = causal ? (l + 1) : S;
    const int nvis = (int)(limit < 0 ? 0 : (limit > S ? S : limit));
    const float4* s4 = (const float4*)(scores + row * S);
    uint2* p2 = (uint2*)(P + row * S);
    const int nv = S >> 2;
    float v[MAXV][4];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int idx = i * 32 + lane;
        if (idx < nv) {
            const float4 t = __ldcs(s4 + idx);
            v[i][0] = t.x * scale; v[i][1] = t.y * scale; v[i][2] = t.z * scale; v[i][3] = t.w * scale;
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (idx * 4 + e < nvis) m = fmaxf(m, v[i][e]);
        }
    }
    m = warp_max(m);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int idx = i * 32 + lane;
        if (idx < nv) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                v[i][e] = (idx * 4 + e < nvis) ? expf(v[i][e] - m) : 0.f;
                sum += v[i][e];
            }
        }
    }
    sum = warp_sum(sum);
    const float inv = nvis > 0 ? 1.0f / sum : 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int idx = i * 32 + lane;
        if (idx < nv) p2[idx] = pack4<T>(v[i][0] * inv, v[i][1] * inv, v[i][2] * inv, v[i][3] * inv);
    }
    if (lane == 0) lse[row] = nvis > 0 ? m + logf(sum) : INFINITY;
}

template <typename T>
__global__ void __launch_bounds__(256) attn_dsoftmax_vec_kernel(T* __restrict__ P, T* __restrict__ dS, const float* __restrict__ scores,
                                                               const float* __restrict__ dP, const float* __restrict__ lse, const float* __restrict__ delta,
                                                               int64_t rows, int64_t L, int S, float scale, int causal) {
    const int nv = S >> 2;
    const int64_t total = rows * nv;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / nv;
        const int j0 = (int)(i - row * nv) * 4;
        const int64_t l = row % L;
        const int64_t limit = causal ? (l + 1) : S;
        const int nvis = (int)(limit < 0 ? 0 : (limit > S ? S : limit));
        const float ls = lse[row], dl = delta[row];
        const bool dead = !(ls < INFINITY);
        const float4 s = __ldcs((const float4*)scores + i), g = __ldcs((const float4*)dP + i);
        const float sv[4] = {s.x, s.y, s.z, s.w}, gv[4] = {g.x, g.y, g.z, g.w};
        float p[4], ds[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            p[e] = (!dead && j0 + e < nvis) ? expf(sv[e] * scale - ls) : 0.f;
            const float pr = to_f32(from_f32<T>(p[e]));
            ds[e] = fminf(fmaxf(pr * (gv[e] - dl) * scale * kDsScale, -60000.f), 60000.f);
        }
        ((uint2*)P)[i] = pack4<T>(p[0], p[1], p[2], p[3]);
        ((uint2*)dS)[i] = pack4<T>(ds[0], ds[1], ds[2], ds[3]);
    }
}

static uint64_t a256(uint64_t v) { return (v + 255) / 256 * 256; }

// ---- fused forward (attention_fused.cuh) ----------------------------------------------------------------
typedef CUresult (*AttnEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static AttnEncodeFn attn_encode_fn() {
    static AttnEncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (AttnEncodeFn)p;
        else cudaGetLastError();
    });
    return fn;
}
// [rows, 64] matrix of 2-byte elements as a 2-D map with a {64, box_rows} box.
static int encode_rows64(CUtensorMap* map, int dtype, const void* ptr, int64_t rows, int box_rows) {
    AttnEncodeFn fn = attn_encode_fn();
    if (!fn) return set_error(TVK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {64, (cuuint64_t)rows};
    cuuint64_t strides[1] = {128};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t es[2] = {1, 1};
    CUresult r = fn(map, dtype == TVK_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                    box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(TVK_ERR_CUDA, "cuTensorMapEncodeTiled (attention operand, %lld rows) failed with code %d", (long long)rows, (int)r);
    return TVK_OK;
}

static bool fused_forward_ok(int64_t Hq, int64_t Hk, int64_t L, int64_t S, int64_t D, const void* out, const void* q, const void* k, const void* v) {
    static const bool off = getenv("TORCHVULKAN_ATTENTION_NO_FUSED") != nullptr;
    return !off && D == 64 && S >= 1 && S <= attn::kFusedS && ((Hq / Hk) * L) % 128 == 0 && aligned16(out) && aligned16(q) && aligned16(k) && aligned16(v);
}

static int run_fused_forward(int dtype, void* out, float* lse, const void* q, const void* k, const void* v, int64_t B, int64_t Hq, int64_t Hk, int64_t L,
                             int64_t S, double scale, int causal, cudaStream_t s) {
    const int64_t G = Hq / Hk, GL = G * L, groups = B * Hk;
    attn::FusedParams p = {};
    p.L = (int)L; p.S = (int)S;
    p.rows_per_group = (int)GL;
    p.tiles_per_group = (int)(GL / 128);
    p.scale = (float)scale;
    p.scale_log2e = (float)(scale * 1.4426950408889634);
    p.causal = causal;
    p.out = out; p.lse = lse; p.dtype = dtype;
    p.status = device_status_word();
    const uint32_t fmt = dtype == TVK_F16 ? 0u : 1u;
    p.idesc_qk = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    p.idesc_pv = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    CUtensorMap mq, mk, mv;
    int rc = encode_rows64(&mq, dtype, q, groups * GL, 128);
    if (rc) return rc;
    rc = encode_rows64(&mk, dtype, k, groups * S, attn::kFusedS);
    if (rc) return rc;
    rc = encode_rows64(&mv, dtype, v, groups * S, attn::kFusedS);
    if (rc) return rc;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        TVK_CUDA_CHECK(cudaFuncSetAttribute(attn::attn_fwd_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, attn::kFusedSmemBytes));
        attr_set[dev] = true;
    }
    const int64_t ctas = groups * p.tiles_per_group;
    TVK_REQUIRE(ctas <= 0x7fffffffLL && groups * GL <= 0x7fffffffLL, "torchvulkan [NOT IMPLEMENTED]: attention with %lld query rows", (long long)(groups * GL));
    attn::attn_fwd_fused_kernel<<<(unsigned)ctas, attn::kFusedThreads, attn::kFusedSmemBytes, s>>>(mq, mk, mv, p);
    return launch_status("fused attention forward");
}

static bool fused_backward_ok(int64_t Hq, int64_t Hk, int64_t L, int64_t S, int64_t D, const void* dq, const void* dk, const void* dv, const void* dout,
                              const void* q, const void* k, const void* v) {
    static const bool off = getenv("TORCHVULKAN_ATTENTION_NO_FUSED_BWD") != nullptr;
    return !off && D == 64 && S >= 128 && S % 128 == 0 && S <= 1024 && ((Hq / Hk) * L) % 128 == 0 && aligned16(dq) && aligned16(dk) && aligned16(dv) &&
           aligned16(dout) && aligned16(q) && aligned16(k) && aligned16(v);
}

// delta must already hold sum(dO * O) per row; dq_part is scratch of (S / 128) * rows * 64 floats.
static int run_fused_backward(int dtype, void* dq, void* dk, void* dv, const void* dout, const void* q, const void* k, const void* v, const float* lse,
                              const float* delta, float* dq_part, int64_t B, int64_t Hq, int64_t Hk, int64_t L, int64_t S, double scale, int causal,
                              cudaStream_t s) {
    const int64_t G = Hq / Hk, GL = G * L, groups = B * Hk, rows = groups * GL;
    attn::BwdParams p = {};
    p.L = (int)L; p.S = (int)S;
    p.rows_per_group = (int)GL;
    p.tiles_per_group = (int)(GL / 128);
    p.kblocks = (int)(S / 128);
    p.scale = (float)scale;
    p.scale_log2e = (float)(scale * 1.4426950408889634);
    p.causal = causal;
    p.lse = lse; p.delta = delta; p.dq_part = dq_part; p.total_rows = rows;
    p.dk = dk; p.dv = dv; p.dtype = dtype;
    p.status = device_status_word();
    const uint32_t fmt = dtype == TVK_F16 ? 0u : 1u;
    const uint32_t base = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(128 >> 4) << 24);
    p.idesc_s = base | ((uint32_t)(128 >> 3) << 17);
    p.idesc_t = base | (1u << 15) | (1u << 16) | ((uint32_t)(64 >> 3) << 17);
    p.idesc_q = base | (1u << 16) | ((uint32_t)(64 >> 3) << 17);
    TVK_REQUIRE(rows <= 0x7fffffffLL && groups * S <= 0x7fffffffLL && groups * p.kblocks <= 0x7fffffffLL,
                "torchvulkan [NOT IMPLEMENTED]: attention backward with %lld query rows", (long long)rows);
    CUtensorMap mq, mdo, mk, mv;
    int rc = encode_rows64(&mq, dtype, q, rows, 128);
    if (rc) return rc;
    rc = encode_rows64(&mdo, dtype, dout, rows, 128);
    if (rc) return rc;
    rc = encode_rows64(&mk, dtype, k, groups * S, 128);
    if (rc) return rc;
    rc = encode_rows64(&mv, dtype, v, groups * S, 128);
    if (rc) return rc;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        TVK_CUDA_CHECK(cudaFuncSetAttribute(attn::attn_bwd_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, attn::kBwdSmemBytes));
        attr_set[dev] = true;
    }
    attn::attn_bwd_fused_kernel<<<(unsigned)(groups * p.kblocks), attn::kBwdThreads, attn::kBwdSmemBytes, s>>>(mq, mdo, mk, mv, p);
    rc = launch_status("fused attention backward");
    if (rc) return rc;
    const int64_t threads = rows * 16;
    TVK_DISPATCH_FLOAT(dtype, T, (attn::attn_dq_finalize_kernel<T><<<(unsigned)((threads + 255) / 256), 256, 0, s>>>((T*)dq, dq_part, rows, (int)GL, p.kblocks, (int)L, (int)S, causal)));
    return launch_status("attention backward dQ");
}

struct AttnShape {
    int64_t B, Hq, Hk, L, S, D;
    int64_t G() const { return Hq / Hk; }
    int64_t rows() const { return B * Hq * L; }
};

static int check_shape(const AttnShape& a, int dtype, const char* who) {
    TVK_REQUIRE(dtype == TVK_F16 || dtype == TVK_BF16, "torchvulkan [NOT IMPLEMENTED]: %s for dtype %d (fp16 and bf16 are supported)", who, dtype);
    TVK_REQUIRE(a.B >= 0 && a.Hq > 0 && a.Hk > 0 && a.L >= 0 && a.S >= 0 && a.D > 0, "%s: bad extent", who);
    TVK_REQUIRE(a.Hq % a.Hk == 0, "%s: %lld query heads are not a multiple of %lld key/value heads", who, (long long)a.Hq, (long long)a.Hk);
    TVK_REQUIRE(a.D % 8 == 0 && a.S % 8 == 0, "torchvulkan [NOT IMPLEMENTED]: %s needs head_dim and key length to be multiples of 8 (got %lld, %lld)", who,
                (long long)a.D, (long long)a.S);
    TVK_REQUIRE(a.rows() <= 0x7fffffffLL, "%s: too many rows", who);
    return TVK_OK;
}

// One batched GEMM over (b, kvh) groups. a: [M, K] view, b: [K, N] view, given by strides.
static int group_gemm(int dtype, int64_t batch, int64_t m, int64_t n, int64_t k, const void* a, int64_t a_rs, int64_t a_cs, int64_t a_bs, const void* b,
                      int64_t b_rs, int64_t b_cs, int64_t b_bs, void* c, int64_t c_bs, int c_f32, cudaStream_t s, float alpha = 1.f) {
    tvk_gemm_desc d = {};
    d.dtype = dtype;
    d.batch = batch; d.m = m; d.n = n; d.k = k;
    d.a = a; d.a_rs = a_rs; d.a_cs = a_cs; d.a_bs = a_bs;
    d.b = b; d.b_rs = b_rs; d.b_cs = b_cs; d.b_bs = b_bs;
    d.c = c; d.c_rs = n; d.c_bs = c_bs;
    d.alpha = alpha; d.beta = 0.f;
    d.force_path = 1;
    d.c_f32 = c_f32;
    return tvk_gemm(&d, nullptr, 0, (void*)s);
}

}  // namespace tvk

using namespace tvk;

extern "C" {

int tvk_attention_workspace_size(int dtype, int64_t B, int64_t Hq, int64_t Hk, int64_t L, int64_t S, int64_t D, int backward, uint64_t* bytes) {
    if (!bytes) return set_error(TVK_ERR_INVALID, "tvk_attention_workspace_size: null output");
    AttnShape a = {B, Hq, Hk, L, S, D};
    int rc = check_shape(a, dtype, "attention");
    if (rc) return rc;
    const uint64_t ls = (uint64_t)a.rows() * (uint64_t)S;
    uint64_t need = a256(ls * 4) + a256(ls * 2);                       // scores fp32, P
    if (backward) need += a256(ls * 4) + a256(ls * 2) + a256((uint64_t)a.rows() * 4);   // dP fp32, dS, delta
    *bytes = need;
    return TVK_OK;
}

int tvk_attention_forward(int dtype, void* out, float* lse, const void* q, const void* k, const void* v, int64_t B, int64_t Hq, int64_t Hk,
                          int64_t L, int64_t S, int64_t D, double scale, int causal, void* workspace, uint64_t workspace_bytes, void* stream) {
    AttnShape a = {B, Hq, Hk, L, S, D};
    int rc = check_shape(a, dtype, "attention forward");
    if (rc) return rc;
    if (a.rows() == 0) return TVK_OK;
    TVK_REQUIRE(out && lse && q, "tvk_attention_forward: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    if (S == 0) {
        // nothing to attend to: out = 0, lse = +inf
        rc = tvk_fill(dtype, out, 0.0, a.rows() * D, stream);
        if (rc) return rc;
        return tvk_fill(TVK_F32, lse, (double)INFINITY, a.rows(), stream);
    }
    TVK_REQUIRE(k && v, "tvk_attention_forward: null pointer");
    uint64_t need = 0;
    tvk_attention_workspace_size(dtype, B, Hq, Hk, L, S, D, 0, &need);
    TVK_REQUIRE(workspace && workspace_bytes >= need && ((uintptr_t)workspace & 255) == 0,
                "tvk_attention_forward: a 256-byte aligned workspace of %llu bytes is required, %llu given", (unsigned long long)need,
                (unsigned long long)workspace_bytes);
    if (fused_forward_ok(Hq, Hk, L, S, D, out, q, k, v)) return run_fused_forward(dtype, out, lse, q, k, v, B, Hq, Hk, L, S, scale, causal, s);
    const uint64_t ls = (uint64_t)a.rows() * (uint64_t)S;
    float* scores = (float*)workspace;
    void* P = (uint8_t*)workspace + a256(ls * 4);
    const int64_t G = a.G(), GL = G * L, groups = B * Hk;
    // scores[b, kvh] = Q_group [G*L, D] @ K[b, kvh]^T [D, S]   (fp32 out)
    rc = group_gemm(dtype, groups, GL, S, D, q, D, 1, GL * D, k, 1, D, S * D, scores, GL * S, 1, s);
    if (rc) return rc;
    if (S % 4 == 0 && S <= 1024) {
        TVK_DISPATCH_FLOAT(dtype, T, (attn_softmax_warp_kernel<T><<<(unsigned)((a.rows() + 7) / 8), 256, 0, s>>>((T*)P, lse, scores, a.rows(), L, (int)S, (float)scale, causal)));
    } else {
        TVK_DISPATCH_FLOAT(dtype, T, (attn_softmax_kernel<T><<<(unsigned)a.rows(), 128, 0, s>>>((T*)P, lse, scores, L, S, (float)scale, causal)));
    }
    rc = launch_status("attention softmax");
    if (rc) return rc;
    // out_group [G*L, D] = P_group [G*L, S] @ V[b, kvh] [S, D]
    return group_gemm(dtype, groups, GL, D, S, P, S, 1, GL * S, v, D, 1, S * D, out, GL * D, 0, s);
}

int tvk_attention_backward(int dtype, void* dq, void* dk, void* dv, const void* dout, const void* q, const void* k, const void* v, const void* out,
                           const float* lse, int64_t B, int64_t Hq, int64_t Hk, int64_t L, int64_t S, int64_t D, double scale, int causal,
                           void* workspace, uint64_t workspace_bytes, void* stream) {
    AttnShape a = {B, Hq, Hk, L, S, D};
    int rc = check_shape(a, dtype, "attention backward");
    if (rc) return rc;
    if (a.rows() == 0 || S == 0) {
        if (dk && B * Hk * S * D) { rc = tvk_fill(dtype, dk, 0.0, B * Hk * S * D, stream); if (rc) return rc; }
        if (dv && B * Hk * S * D) { rc = tvk_fill(dtype, dv, 0.0, B * Hk * S * D, stream); if (rc) return rc; }
        if (dq && a.rows() * D) { rc = tvk_fill(dtype, dq, 0.0, a.rows() * D, stream); if (rc) return rc; }
        return TVK_OK;
    }
    TVK_REQUIRE(dq && dk && dv && dout && q && k && v && out && lse, "tvk_attention_backward: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    uint64_t need = 0;
    tvk_attention_workspace_size(dtype, B, Hq, Hk, L, S, D, 1, &need);
    TVK_REQUIRE(workspace && workspace_bytes >= need && ((uintptr_t)workspace & 255) == 0,
                "tvk_attention_backward: a 256-byte aligned workspace of %llu bytes is required, %llu given", (unsigned long long)need,
                (unsigned long long)workspace_bytes);
    const uint64_t ls = (uint64_t)a.rows() * (uint64_t)S;
    uint8_t* w = (uint8_t*)workspace;
    float* scores = (float*)w;                 w += a256(ls * 4);
    void* P = w;                               w += a256(ls * 2);
    float* dP = (float*)w;                     w += a256(ls * 4);
    void* dS = w;                              w += a256(ls * 2);
    float* delta = (float*)w;
    const int64_t G = a.G(), GL = G * L, groups = B * Hk;
    if (aligned16(dout) && aligned16(out) && D <= (1 << 20)) {     // D is a multiple of 8 (check_shape), so rows stay 16-byte aligned
        TVK_DISPATCH_FLOAT(dtype, T, (attn_delta_vec_kernel<T><<<(unsigned)((a.rows() * 8 + 255) / 256), 256, 0, s>>>(delta, (const T*)dout, (const T*)out, a.rows(), (int)D)));
    } else {
        TVK_DISPATCH_FLOAT(dtype, T, (attn_delta_kernel<T><<<(unsigned)((a.rows() + 3) / 4), 128, 0, s>>>(delta, (const T*)dout, (const T*)out, a.rows(), D)));
    }
    if (fused_backward_ok(Hq, Hk, L, S, D, dq, dk, dv, dout, q, k, v)) {
        // the scores region (rows * S floats) is more than the (S / 128) * rows * 64 floats of dQ partials
        return run_fused_backward(dtype, dq, dk, dv, dout, q, k, v, lse, delta, scores, B, Hq, Hk, L, S, scale, causal, s);
    }
    // scores = Q_group @ K^T, dP = dO_group @ V^T   (both fp32)
    rc = group_gemm(dtype, groups, GL, S, D, q, D, 1, GL * D, k, 1, D, S * D, scores, GL * S, 1, s);
    if (rc) return rc;
    rc = group_gemm(dtype, groups, GL, S, D, dout, D, 1, GL * D, v, 1, D, S * D, dP, GL * S, 1, s);
    if (rc) return rc;
    if (S % 4 == 0 && S <= (1 << 20)) {
        int64_t blocks = (a.rows() * (S / 4) + 255) / 256;
        if (blocks > (int64_t)sm_count() * 16) blocks = (int64_t)sm_count() * 16;
        TVK_DISPATCH_FLOAT(dtype, T, (attn_dsoftmax_vec_kernel<T><<<(unsigned)blocks, 256, 0, s>>>((T*)P, (T*)dS, scores, dP, lse, delta, a.rows(), L, (int)S, (float)scale, causal)));
    } else {
        TVK_DISPATCH_FLOAT(dtype, T, (attn_dsoftmax_kernel<T><<<(unsigned)a.rows(), 128, 0, s>>>((T*)P, (T*)dS, scores, dP, lse, delta, L, S, (float)scale, causal)));
    }
    rc = launch_status("attention backward softmax");
    if (rc) return rc;
    // dV[b, kvh] [S, D] = P_group^T [S, G*L] @ dO_group [G*L, D]
    rc = group_gemm(dtype, groups, S, D, GL, P, 1, S, GL * S, dout, D, 1, GL * D, dv, S * D, 0, s);
    if (rc) return rc;
    // dK[b, kvh] [S, D] = dS_group^T [S, G*L] @ Q_group [G*L, D]
    rc = group_gemm(dtype, groups, S, D, GL, dS, 1, S, GL * S, q, D, 1, GL * D, dk, S * D, 0, s, 1.f / kDsScale);
    if (rc) return rc;
    // dQ_group [G*L, D] = dS_group [G*L, S] @ K[b, kvh] [S, D]
    return group_gemm(dtype, groups, GL, D, S, dS, S, 1, GL * S, k, D, 1, S * D, dq, GL * D, 0, s, 1.f / kDsScale);
}

}  // extern "C"
