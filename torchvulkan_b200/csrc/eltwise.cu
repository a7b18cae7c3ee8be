// Elementwise maps: unary, binary (+scalar operand), compare, ternary, fill, cast, strided copy.
//
// Replaces the reference's binary/unary/compare/where/addc/fill/copy/cast shaders
// (src/shaders/ops/{binary,unary,compare,where,addc,fill,copy,cast}.slang) and their hosts
// (src/api/ops/unary.cpp:76-135, binary.cpp:60-131, 711-771, src/api/tensor/cast.cpp:8-55,
// src/api/tensor/transfer.cpp:16-56). The reference's contiguous path moves VEC elements per
// thread with per-element loads (binary.slang:166-183); here every thread moves 16-byte packets
// and several packets are in flight per thread so HBM3e stays saturated. Half/bf16 math runs
// in fp32 and rounds once (core/dtype.slang:256-283).
#include "common.cuh"

namespace tvk {

// ---- op definitions ---------------------------------------------------------
template <int OP> __device__ __forceinline__ float unary_apply(float x) {
    if constexpr (OP == TVK_U_NEG) return -x;
    else if constexpr (OP == TVK_U_EXP) return expf(x);
    else if constexpr (OP == TVK_U_LOG) return logf(x);
    else if constexpr (OP == TVK_U_SQRT) return sqrtf(x);
    else if constexpr (OP == TVK_U_RSQRT) return 1.0f / sqrtf(x);
    else if constexpr (OP == TVK_U_SIGMOID) return 1.0f / (1.0f + expf(-x));
    else if constexpr (OP == TVK_U_RELU) return (x != x) ? x : fmaxf(x, 0.0f);
    else if constexpr (OP == TVK_U_GELU) return 0.5f * x * (1.0f + erff(x * 0.7071067811865476f));
    else if constexpr (OP == TVK_U_GELU_TANH) return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    else if constexpr (OP == TVK_U_TANH) return tanhf(x);
    else if constexpr (OP == TVK_U_ABS) return fabsf(x);
    else if constexpr (OP == TVK_U_SILU) return x / (1.0f + expf(-x));
    else if constexpr (OP == TVK_U_RECIPROCAL) return 1.0f / x;
    else if constexpr (OP == TVK_U_SQUARE) return x * x;
    else if constexpr (OP == TVK_U_SIN) return sinf(x);
    else if constexpr (OP == TVK_U_COS) return cosf(x);
    else if constexpr (OP == TVK_U_FLOOR) return floorf(x);
    else if constexpr (OP == TVK_U_CEIL) return ceilf(x);
    else if constexpr (OP == TVK_U_ROUND) return rintf(x);
    else if constexpr (OP == TVK_U_TRUNC) return truncf(x);
    else if constexpr (OP == TVK_U_SIGN) return (float)((x > 0.f) - (x < 0.f));
    else if constexpr (OP == TVK_U_LOG2) return log2f(x);
    else if constexpr (OP == TVK_U_LOG10) return log10f(x);
    else if constexpr (OP == TVK_U_LOG1P) return log1pf(x);
    else if constexpr (OP == TVK_U_EXPM1) return expm1f(x);
    else if constexpr (OP == TVK_U_EXP2) return exp2f(x);
    else if constexpr (OP == TVK_U_TAN) return tanf(x);
    else if constexpr (OP == TVK_U_SINH) return sinhf(x);
    else if constexpr (OP == TVK_U_COSH) return coshf(x);
    else if constexpr (OP == TVK_U_ASIN) return asinf(x);
    else if constexpr (OP == TVK_U_ACOS) return acosf(x);
    else if constexpr (OP == TVK_U_ATAN) return atanf(x);
    else if constexpr (OP == TVK_U_ERF) return erff(x);
    else if constexpr (OP == TVK_U_ERFC) return erfcf(x);
    else if constexpr (OP == TVK_U_HARDSIGMOID) return fminf(fmaxf(x + 3.0f, 0.0f), 6.0f) / 6.0f;
    else if constexpr (OP == TVK_U_HARDSWISH) return x * fminf(fmaxf(x + 3.0f, 0.0f), 6.0f) / 6.0f;
    else if constexpr (OP == TVK_U_MISH) return x * tanhf(x > 20.0f ? x : log1pf(expf(x)));
    else if constexpr (OP == TVK_U_LOGSIGMOID) return fminf(x, 0.0f) - log1pf(expf(-fabsf(x)));
    else if constexpr (OP == TVK_U_ASINH) return asinhf(x);
    else if constexpr (OP == TVK_U_ACOSH) return acoshf(x);
    else if constexpr (OP == TVK_U_ATANH) return atanhf(x);
    else if constexpr (OP == TVK_U_ERFINV) return erfinvf(x);
    else if constexpr (OP == TVK_U_LGAMMA) return lgammaf(x);
    else if constexpr (OP == TVK_U_FRAC) return x - truncf(x);
    else if constexpr (OP == TVK_U_SINC) return x == 0.0f ? 1.0f : sinpif(x) / (3.14159265358979323846f * x);
    else return x;
}

template <int OP> __device__ __forceinline__ float binary_apply(float a, float b, float alpha) {
    if constexpr (OP == TVK_B_ADD) return a + alpha * b;
    else if constexpr (OP == TVK_B_ADD_RELU) { const float v = a + alpha * b; return (v != v) ? v : fmaxf(v, 0.f); }
    else if constexpr (OP == TVK_B_SUB) return a - alpha * b;
    else if constexpr (OP == TVK_B_MUL) return a * b;
    else if constexpr (OP == TVK_B_DIV) return a / b;
    else if constexpr (OP == TVK_B_MAXIMUM) return nan_max(a, b);
    else if constexpr (OP == TVK_B_MINIMUM) return nan_min(a, b);
    else if constexpr (OP == TVK_B_POW) return (b == 2.0f) ? a * a : powf(a, b);
    else if constexpr (OP == TVK_B_GELU_BACKWARD) {
        const float cdf = 0.5f * (1.0f + erff(b * 0.7071067811865476f));
        const float pdf = expf(-0.5f * b * b) * 0.3989422804014327f;
        return a * (cdf + b * pdf);
    } else if constexpr (OP == TVK_B_GELU_TANH_BACKWARD) {
        const float x2 = b * b;
        const float t = tanhf(0.7978845608028654f * (b + 0.044715f * x2 * b));
        const float dinner = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * x2);
        return a * (0.5f * (1.0f + t) + 0.5f * b * (1.0f - t * t) * dinner);
    } else if constexpr (OP == TVK_B_THRESHOLD_BACKWARD) return (b <= alpha) ? 0.0f : a;
    else if constexpr (OP == TVK_B_SILU_BACKWARD) {
        const float s = 1.0f / (1.0f + expf(-b));
        return a * s * (1.0f + b * (1.0f - s));
    } else if constexpr (OP == TVK_B_SIGMOID_BACKWARD) return a * (1.0f - b) * b;
    else if constexpr (OP == TVK_B_TANH_BACKWARD) return a * (1.0f - b * b);
    else if constexpr (OP == TVK_B_FMOD) return fmodf(a, b);
    else if constexpr (OP == TVK_B_REMAINDER) {
        float r = fmodf(a, b);
        if (r != 0.0f && ((r < 0.0f) != (b < 0.0f))) r += b;
        return r;
    } else if constexpr (OP == TVK_B_ATAN2) return atan2f(a, b);
    else if constexpr (OP == TVK_B_FLOOR_DIVIDE) {
        if (b == 0.0f) return a / b;
        const float mod = fmodf(a, b);
        float div = (a - mod) / b;
        if (mod != 0.0f && ((b < 0.0f) != (mod < 0.0f))) div -= 1.0f;
        if (div == 0.0f) return copysignf(0.0f, a / b);
        float fl = floorf(div);
        if (div - fl > 0.5f) fl += 1.0f;
        return fl;
    } else if constexpr (OP == TVK_B_CLAMP) return (a != a) ? a : fminf(fmaxf(a, alpha), b);
    else if constexpr (OP == TVK_B_LEAKY_RELU) return a > 0.0f ? a : a * b;
    else if constexpr (OP == TVK_B_ELU) return a > 0.0f ? a : alpha * expm1f(a);
    else if constexpr (OP == TVK_B_SOFTPLUS) return (a * alpha > b) ? a : log1pf(expf(a * alpha)) / alpha;
    else if constexpr (OP == TVK_B_LEAKY_RELU_BACKWARD) return b > 0.0f ? a : a * alpha;
    else if constexpr (OP == TVK_B_ELU_BACKWARD) return b > 0.0f ? a : a * alpha * expf(b);
    else if constexpr (OP == TVK_B_HARDSWISH_BACKWARD) return b < -3.0f ? 0.0f : (b <= 3.0f ? a * (b / 3.0f + 0.5f) : a);
    else if constexpr (OP == TVK_B_HARDSIGMOID_BACKWARD) return (b > -3.0f && b < 3.0f) ? a * (1.0f / 6.0f) : 0.0f;
    else if constexpr (OP == TVK_B_MISH_BACKWARD) {
        const float sp = b > 20.0f ? b : log1pf(expf(b)), t = tanhf(sp), sg = 1.0f / (1.0f + expf(-b));
        return a * (t + b * sg * (1.0f - t * t));
    } else if constexpr (OP == TVK_B_LOGSIGMOID_BACKWARD) return a / (1.0f + expf(b));
    else if constexpr (OP == TVK_B_SOFTPLUS_BACKWARD) {
        const float z = expf(b * alpha);
        return (b * alpha > 20.0f) ? a : a * z / (z + 1.0f);
    } else if constexpr (OP == TVK_B_HYPOT) return hypotf(a, b);
    else if constexpr (OP == TVK_B_COPYSIGN) return copysignf(a, b);
    else if constexpr (OP == TVK_B_LOGADDEXP) {
        if (isinf(a) && a == b) return a;                            // inf - inf would be NaN
        const float mx = fmaxf(a, b), mn = fminf(a, b);
        return (a != a || b != b) ? a + b : mx + log1pf(expf(mn - mx));
    } else if constexpr (OP == TVK_B_LOGADDEXP2) {
        if (isinf(a) && a == b) return a;
        const float mx = fmaxf(a, b), mn = fminf(a, b);
        return (a != a || b != b) ? a + b : mx + log1pf(exp2f(mn - mx)) * 1.4426950408889634f;
    } else if constexpr (OP == TVK_B_FMAX) return fmaxf(a, b);
    else if constexpr (OP == TVK_B_FMIN) return fminf(a, b);
    else if constexpr (OP == TVK_B_HEAVISIDE) return (a != a) ? a : (a < 0.0f ? 0.0f : (a > 0.0f ? 1.0f : b));
    else return a;
}

template <typename T> struct CmpVal { using type = float; static __device__ __forceinline__ float get(T v) { return to_f32(v); } };
template <> struct CmpVal<int64_t> { using type = int64_t; static __device__ __forceinline__ int64_t get(int64_t v) { return v; } };
template <> struct CmpVal<int32_t> { using type = int64_t; static __device__ __forceinline__ int64_t get(int32_t v) { return v; } };
template <> struct CmpVal<uint8_t> { using type = int64_t; static __device__ __forceinline__ int64_t get(uint8_t v) { return v; } };
#define TVK_DISPATCH_CMP(dtype, T, ...)                                                        \
    switch (dtype) {                                                                           \
        case TVK_F32: { using T = float; __VA_ARGS__; break; }                                 \
        case TVK_F16: { using T = __half; __VA_ARGS__; break; }                                \
        case TVK_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }                        \
        case TVK_I64: { using T = int64_t; __VA_ARGS__; break; }                               \
        case TVK_I32: { using T = int32_t; __VA_ARGS__; break; }                               \
        case TVK_U8: { using T = uint8_t; __VA_ARGS__; break; }                                \
        default: return ::tvk::set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: comparison of dtype %d", (int)(dtype)); \
    }

template <int OP, typename V> __device__ __forceinline__ bool compare_apply(V a, V b) {
    if constexpr (OP == TVK_C_EQ) return a == b;
    else if constexpr (OP == TVK_C_NE) return a != b;
    else if constexpr (OP == TVK_C_LT) return a < b;
    else if constexpr (OP == TVK_C_LE) return a <= b;
    else if constexpr (OP == TVK_C_GT) return a > b;
    else return a >= b;
}

template <int OP> __device__ __forceinline__ float ternary_apply(float a, float b, float c, float value) {
    if constexpr (OP == TVK_T_ADDCMUL) return a + value * b * c;
    else if constexpr (OP == TVK_T_ADDCDIV) return a + value * (b / c);
    else return a + value * (b - a);  // LERP
}

// ---- contiguous kernels -------------------------------------------------------
constexpr int kThreads = 256;
constexpr int kUnroll = 4;  // 16-byte packets in flight per thread per operand

static inline int grid_for(int64_t packets) {
    int64_t per_block = (int64_t)kThreads * kUnroll;
    int64_t blocks = (packets + per_block - 1) / per_block;
    int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

// One-input map over packets; F maps float -> float.
template <typename T, typename F>
__global__ void __launch_bounds__(kThreads) map1_vec_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t npackets, F f) {
    constexpr int N = Vec16<T>::N;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    for (; i + (kUnroll - 1) * stride < npackets; i += kUnroll * stride) {
        Vec16<T> v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) v[u] = load16_stream(in + (i + u * stride) * N);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
            for (int j = 0; j < N; ++j) v[u].v[j] = from_f32<T>(f(to_f32(v[u].v[j])));
            store16_stream(out + (i + u * stride) * N, v[u]);
        }
    }
    for (; i < npackets; i += stride) {
        Vec16<T> v = load16_stream(in + i * N);
#pragma unroll
        for (int j = 0; j < N; ++j) v.v[j] = from_f32<T>(f(to_f32(v.v[j])));
        store16_stream(out + i * N, v);
    }
}

template <typename T, typename F>
__global__ void __launch_bounds__(kThreads) map2_vec_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, int64_t npackets, F f) {
    constexpr int N = Vec16<T>::N;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    for (; i + (kUnroll - 1) * stride < npackets; i += kUnroll * stride) {
        Vec16<T> va[kUnroll], vb[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            va[u] = load16_stream(a + (i + u * stride) * N);
            vb[u] = load16_stream(b + (i + u * stride) * N);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
            for (int j = 0; j < N; ++j) va[u].v[j] = from_f32<T>(f(to_f32(va[u].v[j]), to_f32(vb[u].v[j])));
            store16_stream(out + (i + u * stride) * N, va[u]);
        }
    }
    for (; i < npackets; i += stride) {
        Vec16<T> va = load16_stream(a + i * N), vb = load16_stream(b + i * N);
#pragma unroll
        for (int j = 0; j < N; ++j) va.v[j] = from_f32<T>(f(to_f32(va.v[j]), to_f32(vb.v[j])));
        store16_stream(out + i * N, va);
    }
}

template <typename T, typename F>
__global__ void __launch_bounds__(kThreads) map3_vec_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ c, int64_t npackets, F f) {
    constexpr int N = Vec16<T>::N;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < npackets; i += stride) {
        Vec16<T> va = load16_stream(a + i * N), vb = load16_stream(b + i * N), vc = load16_stream(c + i * N);
#pragma unroll
        for (int j = 0; j < N; ++j) va.v[j] = from_f32<T>(f(to_f32(va.v[j]), to_f32(vb.v[j]), to_f32(vc.v[j])));
        store16_stream(out + i * N, va);
    }
}

// Scalar kernels: unaligned pointers and the tail after the last whole packet.
template <typename T, typename F>
__global__ void map1_scalar_kernel(T* out, const T* in, int64_t begin, int64_t n, F f) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = from_f32<T>(f(to_f32(in[i])));
}
template <typename T, typename F>
__global__ void map2_scalar_kernel(T* out, const T* a, const T* b, int64_t begin, int64_t n, F f) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = from_f32<T>(f(to_f32(a[i]), to_f32(b[i])));
}
template <typename T, typename F>
__global__ void map3_scalar_kernel(T* out, const T* a, const T* b, const T* c, int64_t begin, int64_t n, F f) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = from_f32<T>(f(to_f32(a[i]), to_f32(b[i]), to_f32(c[i])));
}

static inline int scalar_grid(int64_t n) {
    int64_t blocks = (n + 255) / 256;
    int64_t cap = (int64_t)sm_count() * 16;
    return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

template <typename T, typename F>
static int launch_map1(T* out, const T* in, int64_t n, F f, cudaStream_t s) {
    constexpr int N = Vec16<T>::N;
    int64_t done = 0;
    if (aligned16(out) && aligned16(in) && n >= N) {
        const int64_t packets = n / N;
        map1_vec_kernel<T, F><<<grid_for(packets), kThreads, 0, s>>>(out, in, packets, f);
        done = packets * N;
    }
    if (done < n) map1_scalar_kernel<T, F><<<scalar_grid(n - done), 256, 0, s>>>(out, in, done, n, f);
    return launch_status("elementwise map");
}
template <typename T, typename F>
static int launch_map2(T* out, const T* a, const T* b, int64_t n, F f, cudaStream_t s) {
    constexpr int N = Vec16<T>::N;
    int64_t done = 0;
    if (aligned16(out) && aligned16(a) && aligned16(b) && n >= N) {
        const int64_t packets = n / N;
        map2_vec_kernel<T, F><<<grid_for(packets), kThreads, 0, s>>>(out, a, b, packets, f);
        done = packets * N;
    }
    if (done < n) map2_scalar_kernel<T, F><<<scalar_grid(n - done), 256, 0, s>>>(out, a, b, done, n, f);
    return launch_status("elementwise map");
}
template <typename T, typename F>
static int launch_map3(T* out, const T* a, const T* b, const T* c, int64_t n, F f, cudaStream_t s) {
    constexpr int N = Vec16<T>::N;
    int64_t done = 0;
    if (aligned16(out) && aligned16(a) && aligned16(b) && aligned16(c) && n >= N) {
        const int64_t packets = n / N;
        map3_vec_kernel<T, F><<<grid_for(packets), kThreads, 0, s>>>(out, a, b, c, packets, f);
        done = packets * N;
    }
    if (done < n) map3_scalar_kernel<T, F><<<scalar_grid(n - done), 256, 0, s>>>(out, a, b, c, done, n, f);
    return launch_status("elementwise map");
}

// ---- functors ---------------------------------------------------------------
template <int OP> struct UnaryF { __device__ __forceinline__ float operator()(float x) const { return unary_apply<OP>(x); } };
template <int OP> struct BinaryF {
    float alpha;
    __device__ __forceinline__ float operator()(float a, float b) const { return binary_apply<OP>(a, b, alpha); }
};
template <int OP> struct BinaryScalarF {  // b is a scalar
    float alpha, b;
    __device__ __forceinline__ float operator()(float a) const { return binary_apply<OP>(a, b, alpha); }
};
template <int OP> struct TernaryF {
    float value;
    __device__ __forceinline__ float operator()(float a, float b, float c) const { return ternary_apply<OP>(a, b, c, value); }
};
template <int OP> struct Ternary2F {  // lerp: c unused
    float value;
    __device__ __forceinline__ float operator()(float a, float b) const { return ternary_apply<OP>(a, b, 0.f, value); }
};

template <int OP> static int unary_op(int dtype, void* out, const void* in, int64_t n, cudaStream_t s) {
    int rc = TVK_OK;
    TVK_DISPATCH_FLOAT(dtype, T, rc = launch_map1<T>((T*)out, (const T*)in, n, UnaryF<OP>{}, s));
    return rc;
}
template <int OP> static int binary_op(int dtype, void* out, const void* a, const void* b, float bs, float alpha, int64_t n, cudaStream_t s) {
    int rc = TVK_OK;
    if (b) {
        TVK_DISPATCH_FLOAT(dtype, T, rc = launch_map2<T>((T*)out, (const T*)a, (const T*)b, n, BinaryF<OP>{alpha}, s));
    } else {
        TVK_DISPATCH_FLOAT(dtype, T, rc = launch_map1<T>((T*)out, (const T*)a, n, BinaryScalarF<OP>{alpha, bs}, s));
    }
    return rc;
}

// ---- compare (output u8) and where (u8 condition) ----------------------------------
template <typename T, int OP>
__global__ void compare_kernel(uint8_t* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, typename CmpVal<T>::type bs, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = compare_apply<OP>(CmpVal<T>::get(a[i]), b ? CmpVal<T>::get(b[i]) : bs) ? 1 : 0;
}
// and / or / xor / not on boolean bytes (any non-zero byte is true; the result is 0 or 1)
__global__ void logical_kernel(uint8_t* __restrict__ out, const uint8_t* __restrict__ a, const uint8_t* __restrict__ b, int op, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const bool x = a[i] != 0, y = b ? b[i] != 0 : false;
        out[i] = op == TVK_L_AND ? (x && y) : op == TVK_L_OR ? (x || y) : op == TVK_L_XOR ? (x != y) : !x;
    }
}
template <typename T>
__global__ void where_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, const uint8_t* __restrict__ c, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = c[i] ? a[i] : b[i];
}

// ---- fill / cast ----------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads) fill_vec_kernel(T* __restrict__ out, T value, int64_t npackets) {
    constexpr int N = Vec16<T>::N;
    Vec16<T> v;
#pragma unroll
    for (int j = 0; j < N; ++j) v.v[j] = value;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < npackets; i += stride) store16_stream(out + i * N, v);
}
template <typename T>
__global__ void fill_scalar_kernel(T* out, T value, int64_t begin, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = begin + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = value;
}
template <typename T> static int fill_impl(T* out, T value, int64_t n, cudaStream_t s) {
    constexpr int N = Vec16<T>::N;
    int64_t done = 0;
    if (aligned16(out) && n >= N) {
        const int64_t packets = n / N;
        fill_vec_kernel<T><<<grid_for(packets), kThreads, 0, s>>>(out, value, packets);
        done = packets * N;
    }
    if (done < n) fill_scalar_kernel<T><<<scalar_grid(n - done), 256, 0, s>>>(out, value, done, n);
    return launch_status("fill");
}

// Generic scalar value conversions used by cast / strided copy (through double for the
// integer and f64 types, through float for the half types).
template <typename T> __device__ __forceinline__ double to_f64(T v) { return (double)v; }
template <> __device__ __forceinline__ double to_f64<__half>(__half v) { return (double)__half2float(v); }
template <> __device__ __forceinline__ double to_f64<__nv_bfloat16>(__nv_bfloat16 v) { return (double)__bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f64(double v) { return (T)v; }
template <> __device__ __forceinline__ __half from_f64<__half>(double v) { return __float2half_rn((float)v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f64<__nv_bfloat16>(double v) { return __float2bfloat16_rn((float)v); }
template <> __device__ __forceinline__ uint8_t from_f64<uint8_t>(double v) { return (uint8_t)(long long)v; }

template <typename D, typename S> __device__ __forceinline__ D convert(S v) {
    if constexpr (sizeof(S) == 8 && sizeof(D) == 8 && !(sizeof(D) == 8 && false)) {
        return (D)v;  // i64 <-> f64 directly, no rounding through a narrower type
    } else if constexpr ((sizeof(S) <= 4 && sizeof(D) <= 4) &&
                         !(std::is_same<S, int32_t>::value || std::is_same<D, int32_t>::value)) {
        return from_f32<D>(to_f32<S>(v));
    } else {
        return from_f64<D>(to_f64<S>(v));
    }
}
template <> __device__ __forceinline__ float to_f32<uint8_t>(uint8_t v) { return (float)v; }
template <> __device__ __forceinline__ uint8_t from_f32<uint8_t>(float v) { return (uint8_t)(int)v; }

template <typename D, typename S>
__global__ void __launch_bounds__(kThreads) cast_kernel(D* __restrict__ dst, const S* __restrict__ src, int64_t n) {
    // Each thread converts 8 consecutive elements so both sides see wide accesses.
    const int64_t stride = (int64_t)gridDim.x * kThreads * 8;
    for (int64_t base = ((int64_t)blockIdx.x * kThreads + threadIdx.x) * 8; base < n; base += stride) {
        if (base + 8 <= n) {
            S tmp[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) tmp[j] = src[base + j];
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[base + j] = convert<D, S>(tmp[j]);
        } else {
            for (int64_t i = base; i < n; ++i) dst[i] = convert<D, S>(src[i]);
        }
    }
}

#define TVK_DISPATCH_ALL(dtype, T, ...)                                                        \
    switch (dtype) {                                                                           \
        case TVK_F32: { using T = float; __VA_ARGS__; break; }                                 \
        case TVK_F16: { using T = __half; __VA_ARGS__; break; }                                \
        case TVK_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }                        \
        case TVK_I64: { using T = int64_t; __VA_ARGS__; break; }                               \
        case TVK_I32: { using T = int32_t; __VA_ARGS__; break; }                               \
        case TVK_U8: { using T = uint8_t; __VA_ARGS__; break; }                                \
        case TVK_F64: { using T = double; __VA_ARGS__; break; }                                \
        default: return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: unknown dtype %d", (int)(dtype)); \
    }

// ---- strided iteration --------------------------------------------------------------
struct IterArgs {
    int ndim;
    int64_t total;
    int64_t sizes[TVK_MAX_DIMS];
    int64_t strides[4][TVK_MAX_DIMS];
};

// Drops size-1 dims and merges neighbouring dims that are contiguous for every operand.
static int make_iter(const tvk_iter* it, int nops, IterArgs* out) {
    if (!it) return set_error(TVK_ERR_INVALID, "null iteration descriptor");
    if (it->ndim < 0 || it->ndim > TVK_MAX_DIMS) return set_error(TVK_ERR_INVALID, "iteration rank %d out of range", it->ndim);
    IterArgs r = {};
    int64_t total = 1;
    int nd = 0;
    // The elements are independent, so the dims may be walked in any order: take them by increasing output stride
    // (ties: innermost first). A channels-last or otherwise permuted output then has its contiguous dim innermost,
    // which is what the packet kernels need.
    int order[TVK_MAX_DIMS];
    for (int i = 0; i < it->ndim; ++i) order[i] = it->ndim - 1 - i;
    for (int i = 1; i < it->ndim; ++i)
        for (int j = i; j > 0; --j) {
            const int64_t sa = it->strides[0][order[j - 1]], sb = it->strides[0][order[j]];
            if ((sa < 0 ? -sa : sa) <= (sb < 0 ? -sb : sb)) break;
            const int tmp = order[j]; order[j] = order[j - 1]; order[j - 1] = tmp;
        }
    for (int oi = 0; oi < it->ndim; ++oi) {
        const int d = order[oi];
        const int64_t sz = it->sizes[d];
        if (sz < 0) return set_error(TVK_ERR_INVALID, "negative size in iteration descriptor");
        total *= sz;
        if (sz == 1) continue;
        bool merged = false;
        if (nd > 0) {
            bool can = true;
            for (int o = 0; o < nops; ++o)
                if (it->strides[o][d] != r.strides[o][nd - 1] * r.sizes[nd - 1]) { can = false; break; }
            if (can) { r.sizes[nd - 1] *= sz; merged = true; }
        }
        if (!merged) {
            r.sizes[nd] = sz;
            for (int o = 0; o < nops; ++o) r.strides[o][nd] = it->strides[o][d];
            ++nd;
        }
    }
    r.ndim = nd;
    r.total = total;
    *out = r;
    return TVK_OK;
}

template <int NOPS> __device__ __forceinline__ void iter_offsets(const IterArgs& it, int64_t linear, int64_t* off) {
#pragma unroll
    for (int o = 0; o < NOPS; ++o) off[o] = 0;
    for (int d = 0; d < it.ndim; ++d) {
        const int64_t q = linear / it.sizes[d];
        const int64_t r = linear - q * it.sizes[d];
        linear = q;
#pragma unroll
        for (int o = 0; o < NOPS; ++o) off[o] += r * it.strides[o][d];
    }
}

template <typename T, typename F>
__global__ void strided1_kernel(T* out, const T* in, IterArgs it, F f) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < it.total; i += stride) {
        int64_t off[2];
        iter_offsets<2>(it, i, off);
        out[off[0]] = from_f32<T>(f(to_f32(in[off[1]])));
    }
}
template <typename T, typename F>
__global__ void strided2_kernel(T* out, const T* a, const T* b, IterArgs it, F f) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < it.total; i += stride) {
        int64_t off[3];
        iter_offsets<3>(it, i, off);
        out[off[0]] = from_f32<T>(f(to_f32(a[off[1]]), to_f32(b[off[2]])));
    }
}
template <typename T, typename F>
__global__ void strided3_kernel(T* out, const T* a, const T* b, const T* c, IterArgs it, F f) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < it.total; i += stride) {
        int64_t off[4];
        iter_offsets<4>(it, i, off);
        out[off[0]] = from_f32<T>(f(to_f32(a[off[1]]), to_f32(b[off[2]]), to_f32(c[off[3]])));
    }
}
// ---- strided iteration, 16 bytes at a time ----------------------------------------------------
// Most non-contiguous operands still have a contiguous innermost dimension (a slice of the last
// dim, a permutation of outer dims, a broadcast table): then the innermost dim is walked in 16-byte
// packets, the index arithmetic is paid once per packet, and every access is a 128-bit one.
// Operands whose innermost stride is 0 (broadcast along the row) are read as one scalar per packet.

// Rewrites `ia` into packet space if every operand allows it. ptrs[o] / es[o] are the base pointer and element
// size of operand o (operand 0 is the output). Returns false (ia untouched) when the scalar kernels must run.
static bool vectorize_iter(IterArgs* ia, int nops, const void* const* ptrs, const size_t* es, int* bcast_mask) {
    if (ia->ndim == 0 || ia->total == 0) return false;
    size_t max_es = 0;
    for (int o = 0; o < nops; ++o) max_es = es[o] > max_es ? es[o] : max_es;
    const int64_t vec = (int64_t)(16 / max_es);            // elements per packet (of the widest operand)
    if (vec <= 1 || ia->sizes[0] % vec != 0) return false;
    int mask = 0;
    for (int o = 0; o < nops; ++o) {
        const int64_t s0 = ia->strides[o][0];
        if (s0 == 0 && o > 0) { mask |= 1 << o; continue; }
        if (s0 != 1) return false;
        const size_t packet_bytes = (size_t)vec * es[o];   // 16 for the widest type, less for narrower ones
        if ((uintptr_t)ptrs[o] % packet_bytes != 0) return false;
        for (int d = 1; d < ia->ndim; ++d)
            if ((ia->strides[o][d] * (int64_t)es[o]) % (int64_t)packet_bytes != 0) return false;
    }
    ia->sizes[0] /= vec;
    ia->total /= vec;
    for (int o = 0; o < nops; ++o) ia->strides[o][0] *= vec;
    *bcast_mask = mask;
    return true;
}

template <typename T> __device__ __forceinline__ Vec16<T> load_or_splat(const T* p, bool splat) {
    if (!splat) return load16(p);
    Vec16<T> r;
    const T s = *p;
#pragma unroll
    for (int j = 0; j < Vec16<T>::N; ++j) r.v[j] = s;
    return r;
}

template <typename T, typename F>
__global__ void __launch_bounds__(256) strided1_vec_kernel(T* out, const T* in, IterArgs it, F f) {
    constexpr int N = Vec16<T>::N;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < it.total; i += stride) {
        int64_t off[2];
        iter_offsets<2>(it, i, off);
        Vec16<T> v = load16(in + off[1]);
#pragma unroll
        for (int j = 0; j < N; ++j) v.v[j] = from_f32<T>(f(to_f32(v.v[j])));
        store16(out + off[0], v);
    }
}
template <typename T, typename F>
__global__ void __launch_bounds__(256) strided2_vec_kernel(T* out, const T* a, const T* b, IterArgs it, int bcast, F f) {
    constexpr int N = Vec16<T>::N;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < it.total; i += stride) {
        int64_t off[3];
        iter_offsets<3>(it, i, off);
        Vec16<T> va = load_or_splat(a + off[1], bcast & 2), vb = load_or_splat(b + off[2], bcast & 4);
#pragma unroll
        for (int j = 0; j < N; ++j) va.v[j] = from_f32<T>(f(to_f32(va.v[j]), to_f32(vb.v[j])));
        store16(out + off[0], va);
    }
}
template <typename T, typename F>
__global__ void __launch_bounds__(256) strided3_vec_kernel(T* out, const T* a, const T* b, const T* c, IterArgs it, int bcast, F f) {
    constexpr int N = Vec16<T>::N;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < it.total; i += stride) {
        int64_t off[4];
        iter_offsets<4>(it, i, off);
        Vec16<T> va = load_or_splat(a + off[1], bcast & 2), vb = load_or_splat(b + off[2], bcast & 4), vc = load_or_splat(c + off[3], bcast & 8);
#pragma unroll
        for (int j = 0; j < N; ++j) va.v[j] = from_f32<T>(f(to_f32(va.v[j]), to_f32(vb.v[j]), to_f32(vc.v[j])));
        store16(out + off[0], va);
    }
}
// Same-type copy of `packet` bytes per step (16 when dst and src are both 16-byte steppable).
__global__ void __launch_bounds__(256) strided_copy_vec_kernel(uint4* dst, const uint4* src, IterArgs it) {
    // offsets are in elements of the packet-space iteration: strides were pre-divided to packets by the host
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < it.total; i += stride) {
        int64_t off[2];
        iter_offsets<2>(it, i, off);
        dst[off[0]] = src[off[1]];
    }
}

template <typename T, int OP>
__global__ void strided_compare_kernel(uint8_t* out, const T* a, const T* b, IterArgs it) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < it.total; i += stride) {
        int64_t off[3];
        iter_offsets<3>(it, i, off);
        out[off[0]] = compare_apply<OP>(CmpVal<T>::get(a[off[1]]), CmpVal<T>::get(b[off[2]])) ? 1 : 0;
    }
}
template <typename T>
__global__ void strided_where_kernel(T* out, const T* a, const T* b, const uint8_t* c, IterArgs it) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < it.total; i += stride) {
        int64_t off[4];
        iter_offsets<4>(it, i, off);
        out[off[0]] = c[off[3]] ? a[off[1]] : b[off[2]];
    }
}
template <typename D, typename S>
__global__ void strided_copy_kernel(D* dst, const S* src, IterArgs it) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < it.total; i += stride) {
        int64_t off[2];
        iter_offsets<2>(it, i, off);
        dst[off[0]] = convert<D, S>(src[off[1]]);
    }
}

// 2-D transposing copy through shared memory for the common "inner dim of the source is the
// outer dim of the destination" case (e.g. .t().contiguous()), same dtype.
template <typename T>
__global__ void transpose_copy_kernel(T* __restrict__ dst, const T* __restrict__ src, int64_t rows, int64_t cols,
                                      int64_t dst_rs, int64_t src_cs, int64_t batch_dst, int64_t batch_src) {
    // dst[r*dst_rs + c] = src[c*src_cs + r]; r < rows, c < cols.
    __shared__ T tile[32][33];
    dst += (int64_t)blockIdx.z * batch_dst;
    src += (int64_t)blockIdx.z * batch_src;
    const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int64_t c = c0 + j, r = r0 + threadIdx.x;
        if (c < cols && r < rows) tile[j][threadIdx.x] = src[c * src_cs + r];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int64_t r = r0 + j, c = c0 + threadIdx.x;
        if (c < cols && r < rows) dst[r * dst_rs + c] = tile[threadIdx.x][j];
    }
}

template <typename F> static int dispatch_unary_op(int op, F&& f) {
    switch (op) {
#define C(OPV) case OPV: return f(std::integral_constant<int, OPV>{});
        C(TVK_U_NEG) C(TVK_U_EXP) C(TVK_U_LOG) C(TVK_U_SQRT) C(TVK_U_RSQRT) C(TVK_U_SIGMOID) C(TVK_U_RELU)
        C(TVK_U_GELU) C(TVK_U_TANH) C(TVK_U_ABS) C(TVK_U_SILU) C(TVK_U_RECIPROCAL) C(TVK_U_SQUARE) C(TVK_U_SIN) C(TVK_U_COS)
        C(TVK_U_GELU_TANH)
        C(TVK_U_FLOOR) C(TVK_U_CEIL) C(TVK_U_ROUND) C(TVK_U_TRUNC) C(TVK_U_SIGN) C(TVK_U_LOG2) C(TVK_U_LOG10) C(TVK_U_LOG1P) C(TVK_U_EXPM1) C(TVK_U_EXP2)
        C(TVK_U_TAN) C(TVK_U_SINH) C(TVK_U_COSH) C(TVK_U_ASIN) C(TVK_U_ACOS) C(TVK_U_ATAN) C(TVK_U_ERF) C(TVK_U_ERFC)
        C(TVK_U_HARDSIGMOID) C(TVK_U_HARDSWISH) C(TVK_U_MISH) C(TVK_U_LOGSIGMOID)
        C(TVK_U_ASINH) C(TVK_U_ACOSH) C(TVK_U_ATANH) C(TVK_U_ERFINV) C(TVK_U_LGAMMA) C(TVK_U_FRAC) C(TVK_U_SINC)
#undef C
        default: return set_error(TVK_ERR_INVALID, "unknown unary op %d", op);
    }
}
template <typename F> static int dispatch_binary_op(int op, F&& f) {
    switch (op) {
#define C(OPV) case OPV: return f(std::integral_constant<int, OPV>{});
        C(TVK_B_ADD) C(TVK_B_SUB) C(TVK_B_MUL) C(TVK_B_DIV) C(TVK_B_MAXIMUM) C(TVK_B_MINIMUM) C(TVK_B_POW)
        C(TVK_B_GELU_BACKWARD) C(TVK_B_THRESHOLD_BACKWARD) C(TVK_B_SILU_BACKWARD) C(TVK_B_SIGMOID_BACKWARD) C(TVK_B_TANH_BACKWARD)
        C(TVK_B_GELU_TANH_BACKWARD) C(TVK_B_ADD_RELU)
        C(TVK_B_FMOD) C(TVK_B_REMAINDER) C(TVK_B_ATAN2) C(TVK_B_FLOOR_DIVIDE) C(TVK_B_CLAMP) C(TVK_B_LEAKY_RELU) C(TVK_B_ELU) C(TVK_B_SOFTPLUS)
        C(TVK_B_LEAKY_RELU_BACKWARD) C(TVK_B_ELU_BACKWARD) C(TVK_B_HARDSWISH_BACKWARD) C(TVK_B_HARDSIGMOID_BACKWARD) C(TVK_B_MISH_BACKWARD)
        C(TVK_B_LOGSIGMOID_BACKWARD) C(TVK_B_SOFTPLUS_BACKWARD)
        C(TVK_B_HYPOT) C(TVK_B_COPYSIGN) C(TVK_B_LOGADDEXP) C(TVK_B_LOGADDEXP2) C(TVK_B_FMAX) C(TVK_B_FMIN) C(TVK_B_HEAVISIDE)
#undef C
        default: return set_error(TVK_ERR_INVALID, "unknown binary op %d", op);
    }
}
template <typename F> static int dispatch_compare_op(int op, F&& f) {
    switch (op) {
#define C(OPV) case OPV: return f(std::integral_constant<int, OPV>{});
        C(TVK_C_EQ) C(TVK_C_NE) C(TVK_C_LT) C(TVK_C_LE) C(TVK_C_GT) C(TVK_C_GE)
#undef C
        default: return set_error(TVK_ERR_INVALID, "unknown compare op %d", op);
    }
}

// Integer arithmetic (counters such as BatchNorm's num_batches_tracked, class indices and position ids live on the
// device): add / sub / mul, maximum / minimum, floor division and the two remainders, exactly, in the tensor's own width.
// Division by zero gives 0 (ATen's CUDA kernels leave it undefined; the CPU raises).
__host__ __device__ inline bool int_op_supported(int op) {
    return op == TVK_B_ADD || op == TVK_B_SUB || op == TVK_B_MUL || op == TVK_B_MAXIMUM || op == TVK_B_MINIMUM || op == TVK_B_FLOOR_DIVIDE ||
           op == TVK_B_REMAINDER || op == TVK_B_FMOD;
}
template <typename T> __device__ __forceinline__ T int_apply(int op, T x, T y, T alpha) {
    switch (op) {
        case TVK_B_ADD: return x + alpha * y;
        case TVK_B_SUB: return x - alpha * y;
        case TVK_B_MUL: return x * y;
        case TVK_B_MAXIMUM: return x > y ? x : y;
        case TVK_B_MINIMUM: return x < y ? x : y;
        case TVK_B_FLOOR_DIVIDE: {
            if (y == 0) return 0;
            T q = x / y;
            if ((x % y != 0) && ((x < 0) != (y < 0))) --q;
            return q;
        }
        case TVK_B_REMAINDER: {
            if (y == 0) return 0;
            T r = x % y;
            if (r != 0 && ((r < 0) != (y < 0))) r += y;
            return r;
        }
        default: return y == 0 ? 0 : x % y;      // TVK_B_FMOD: the sign of x
    }
}
template <typename T>
__global__ void int_binary_kernel(T* out, const T* a, const T* b, T bs, T alpha, int op, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = int_apply<T>(op, a[i], b ? b[i] : bs, alpha);
}
template <typename T>
__global__ void int_binary_strided_kernel(T* out, const T* a, const T* b, T alpha, int op, IterArgs it) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < it.total; i += stride) {
        int64_t off[3];
        iter_offsets<3>(it, i, off);
        out[off[0]] = int_apply<T>(op, a[off[1]], b[off[2]], alpha);
    }
}

}  // namespace tvk

using namespace tvk;

extern "C" {

int tvk_unary(int op, int dtype, void* out, const void* in, int64_t n, void* stream) {
    if (n == 0) return TVK_OK;
    TVK_REQUIRE(out && in && n > 0, "tvk_unary: null pointer or negative size");
    cudaStream_t s = (cudaStream_t)stream;
    return dispatch_unary_op(op, [&](auto opc) { return unary_op<decltype(opc)::value>(dtype, out, in, n, s); });
}

int tvk_binary(int op, int dtype, void* out, const void* a, const void* b, double b_scalar, double alpha, int64_t n,
               void* stream) {
    if (n == 0) return TVK_OK;
    TVK_REQUIRE(out && a && n > 0, "tvk_binary: null pointer or negative size");
    cudaStream_t s = (cudaStream_t)stream;
    if ((dtype == TVK_I64 || dtype == TVK_I32) && int_op_supported(op)) {
        if (dtype == TVK_I64) int_binary_kernel<int64_t><<<scalar_grid(n), 256, 0, s>>>((int64_t*)out, (const int64_t*)a, (const int64_t*)b, (int64_t)b_scalar, (int64_t)alpha, op, n);
        else int_binary_kernel<int32_t><<<scalar_grid(n), 256, 0, s>>>((int32_t*)out, (const int32_t*)a, (const int32_t*)b, (int32_t)b_scalar, (int32_t)alpha, op, n);
        return launch_status("integer binary");
    }
    return dispatch_binary_op(op, [&](auto opc) {
        return binary_op<decltype(opc)::value>(dtype, out, a, b, (float)b_scalar, (float)alpha, n, s);
    });
}

int tvk_compare(int op, int dtype, uint8_t* out, const void* a, const void* b, double b_scalar, int64_t n, void* stream) {
    if (n == 0) return TVK_OK;
    TVK_REQUIRE(out && a && n > 0, "tvk_compare: null pointer or negative size");
    cudaStream_t s = (cudaStream_t)stream;
    return dispatch_compare_op(op, [&](auto opc) {
        constexpr int OP = decltype(opc)::value;
        TVK_DISPATCH_CMP(dtype, T, (compare_kernel<T, OP><<<scalar_grid(n), 256, 0, s>>>(out, (const T*)a, (const T*)b, (typename CmpVal<T>::type)b_scalar, n)));
        return launch_status("compare");
    });
}

int tvk_logical(int op, uint8_t* out, const uint8_t* a, const uint8_t* b, int64_t n, void* stream) {
    if (n == 0) return TVK_OK;
    TVK_REQUIRE(op >= 0 && op < TVK_L_COUNT_, "tvk_logical: unknown op %d", op);
    TVK_REQUIRE(out && a && (b || op == TVK_L_NOT) && n > 0, "tvk_logical: null pointer or negative size");
    logical_kernel<<<scalar_grid(n), 256, 0, (cudaStream_t)stream>>>(out, a, op == TVK_L_NOT ? nullptr : b, op, n);
    return launch_status("logical op");
}

int tvk_ternary(int op, int dtype, void* out, const void* a, const void* b, const void* c, double value, int64_t n,
                void* stream) {
    if (n == 0) return TVK_OK;
    TVK_REQUIRE(out && a && b && n > 0, "tvk_ternary: null pointer or negative size");
    cudaStream_t s = (cudaStream_t)stream;
    int rc = TVK_OK;
    switch (op) {
        case TVK_T_ADDCMUL:
            TVK_REQUIRE(c, "tvk_ternary: addcmul needs three inputs");
            TVK_DISPATCH_FLOAT(dtype, T, rc = launch_map3<T>((T*)out, (const T*)a, (const T*)b, (const T*)c, n, TernaryF<TVK_T_ADDCMUL>{(float)value}, s));
            return rc;
        case TVK_T_ADDCDIV:
            TVK_REQUIRE(c, "tvk_ternary: addcdiv needs three inputs");
            TVK_DISPATCH_FLOAT(dtype, T, rc = launch_map3<T>((T*)out, (const T*)a, (const T*)b, (const T*)c, n, TernaryF<TVK_T_ADDCDIV>{(float)value}, s));
            return rc;
        case TVK_T_LERP:
            TVK_DISPATCH_FLOAT(dtype, T, rc = launch_map2<T>((T*)out, (const T*)a, (const T*)b, n, Ternary2F<TVK_T_LERP>{(float)value}, s));
            return rc;
        case TVK_T_WHERE:
            TVK_REQUIRE(c, "tvk_ternary: where needs a condition");
            TVK_DISPATCH_ALL(dtype, T, (where_kernel<T><<<scalar_grid(n), 256, 0, s>>>((T*)out, (const T*)a, (const T*)b, (const uint8_t*)c, n)));
            return launch_status("where");
        default:
            return set_error(TVK_ERR_INVALID, "unknown ternary op %d", op);
    }
}

int tvk_unary_strided(int op, int dtype, void* out, const void* in, const tvk_iter* it, void* stream) {
    IterArgs ia;
    int rc = make_iter(it, 2, &ia);
    if (rc) return rc;
    if (ia.total == 0) return TVK_OK;
    TVK_REQUIRE(out && in, "tvk_unary_strided: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    const void* ptrs[2] = {out, in};
    const size_t es[2] = {dtype_size(dtype), dtype_size(dtype)};
    int bcast = 0;
    const bool vec = (dtype == TVK_F32 || dtype == TVK_F16 || dtype == TVK_BF16) && vectorize_iter(&ia, 2, ptrs, es, &bcast) && bcast == 0;
    return dispatch_unary_op(op, [&](auto opc) {
        constexpr int OP = decltype(opc)::value;
        if (vec) {
            TVK_DISPATCH_FLOAT(dtype, T, (strided1_vec_kernel<T><<<scalar_grid(ia.total), 256, 0, s>>>((T*)out, (const T*)in, ia, UnaryF<OP>{})));
        } else {
            TVK_DISPATCH_FLOAT(dtype, T, (strided1_kernel<T><<<scalar_grid(ia.total), 256, 0, s>>>((T*)out, (const T*)in, ia, UnaryF<OP>{})));
        }
        return launch_status("strided unary");
    });
}

int tvk_binary_strided(int op, int dtype, void* out, const void* a, const void* b, double alpha, const tvk_iter* it,
                       void* stream) {
    IterArgs ia;
    int rc = make_iter(it, 3, &ia);
    if (rc) return rc;
    if (ia.total == 0) return TVK_OK;
    TVK_REQUIRE(out && a && b, "tvk_binary_strided: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    if ((dtype == TVK_I64 || dtype == TVK_I32) && int_op_supported(op)) {
        if (dtype == TVK_I64) int_binary_strided_kernel<int64_t><<<scalar_grid(ia.total), 256, 0, s>>>((int64_t*)out, (const int64_t*)a, (const int64_t*)b, (int64_t)alpha, op, ia);
        else int_binary_strided_kernel<int32_t><<<scalar_grid(ia.total), 256, 0, s>>>((int32_t*)out, (const int32_t*)a, (const int32_t*)b, (int32_t)alpha, op, ia);
        return launch_status("integer binary");
    }
    const void* ptrs[3] = {out, a, b};
    const size_t es[3] = {dtype_size(dtype), dtype_size(dtype), dtype_size(dtype)};
    int bcast = 0;
    const bool vec = vectorize_iter(&ia, 3, ptrs, es, &bcast);
    return dispatch_binary_op(op, [&](auto opc) {
        constexpr int OP = decltype(opc)::value;
        if (vec) {
            TVK_DISPATCH_FLOAT(dtype, T, (strided2_vec_kernel<T><<<scalar_grid(ia.total), 256, 0, s>>>((T*)out, (const T*)a, (const T*)b, ia, bcast, BinaryF<OP>{(float)alpha})));
        } else {
            TVK_DISPATCH_FLOAT(dtype, T, (strided2_kernel<T><<<scalar_grid(ia.total), 256, 0, s>>>((T*)out, (const T*)a, (const T*)b, ia, BinaryF<OP>{(float)alpha})));
        }
        return launch_status("strided binary");
    });
}

int tvk_compare_strided(int op, int dtype, uint8_t* out, const void* a, const void* b, const tvk_iter* it, void* stream) {
    IterArgs ia;
    int rc = make_iter(it, 3, &ia);
    if (rc) return rc;
    if (ia.total == 0) return TVK_OK;
    TVK_REQUIRE(out && a && b, "tvk_compare_strided: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    return dispatch_compare_op(op, [&](auto opc) {
        constexpr int OP = decltype(opc)::value;
        TVK_DISPATCH_CMP(dtype, T, (strided_compare_kernel<T, OP><<<scalar_grid(ia.total), 256, 0, s>>>(out, (const T*)a, (const T*)b, ia)));
        return launch_status("strided compare");
    });
}

int tvk_ternary_strided(int op, int dtype, void* out, const void* a, const void* b, const void* c, double value,
                        const tvk_iter* it, void* stream) {
    IterArgs ia;
    int rc = make_iter(it, 4, &ia);
    if (rc) return rc;
    if (ia.total == 0) return TVK_OK;
    TVK_REQUIRE(out && a && b, "tvk_ternary_strided: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    int bcast = 0;
    bool vec = false;
    if (op == TVK_T_ADDCMUL || op == TVK_T_ADDCDIV) {
        TVK_REQUIRE(c, "addcmul / addcdiv need three inputs");
        const void* ptrs[4] = {out, a, b, c};
        const size_t es[4] = {dtype_size(dtype), dtype_size(dtype), dtype_size(dtype), dtype_size(dtype)};
        vec = (dtype == TVK_F32 || dtype == TVK_F16 || dtype == TVK_BF16) && vectorize_iter(&ia, 4, ptrs, es, &bcast);
    }
    const int g = scalar_grid(ia.total);
    switch (op) {
        case TVK_T_ADDCMUL:
            if (vec) { TVK_DISPATCH_FLOAT(dtype, T, (strided3_vec_kernel<T><<<g, 256, 0, s>>>((T*)out, (const T*)a, (const T*)b, (const T*)c, ia, bcast, TernaryF<TVK_T_ADDCMUL>{(float)value}))); }
            else { TVK_DISPATCH_FLOAT(dtype, T, (strided3_kernel<T><<<g, 256, 0, s>>>((T*)out, (const T*)a, (const T*)b, (const T*)c, ia, TernaryF<TVK_T_ADDCMUL>{(float)value}))); }
            break;
        case TVK_T_ADDCDIV:
            if (vec) { TVK_DISPATCH_FLOAT(dtype, T, (strided3_vec_kernel<T><<<g, 256, 0, s>>>((T*)out, (const T*)a, (const T*)b, (const T*)c, ia, bcast, TernaryF<TVK_T_ADDCDIV>{(float)value}))); }
            else { TVK_DISPATCH_FLOAT(dtype, T, (strided3_kernel<T><<<g, 256, 0, s>>>((T*)out, (const T*)a, (const T*)b, (const T*)c, ia, TernaryF<TVK_T_ADDCDIV>{(float)value}))); }
            break;
        case TVK_T_LERP:
            TVK_DISPATCH_FLOAT(dtype, T, (strided2_kernel<T><<<g, 256, 0, s>>>((T*)out, (const T*)a, (const T*)b, ia, Ternary2F<TVK_T_LERP>{(float)value})));
            break;
        case TVK_T_WHERE:
            TVK_REQUIRE(c, "where needs a condition");
            TVK_DISPATCH_ALL(dtype, T, (strided_where_kernel<T><<<g, 256, 0, s>>>((T*)out, (const T*)a, (const T*)b, (const uint8_t*)c, ia)));
            break;
        default:
            return set_error(TVK_ERR_INVALID, "unknown ternary op %d", op);
    }
    return launch_status("strided ternary");
}

int tvk_fill(int dtype, void* out, double value, int64_t n, void* stream) {
    if (n == 0) return TVK_OK;
    TVK_REQUIRE(out && n > 0, "tvk_fill: null pointer or negative size");
    cudaStream_t s = (cudaStream_t)stream;
    int rc = TVK_OK;
    switch (dtype) {
        case TVK_F32: rc = fill_impl<float>((float*)out, (float)value, n, s); break;
        case TVK_F16: rc = fill_impl<__half>((__half*)out, __float2half_rn((float)value), n, s); break;
        case TVK_BF16: rc = fill_impl<__nv_bfloat16>((__nv_bfloat16*)out, __float2bfloat16_rn((float)value), n, s); break;
        case TVK_I64: rc = fill_impl<int64_t>((int64_t*)out, (int64_t)value, n, s); break;
        case TVK_I32: rc = fill_impl<int32_t>((int32_t*)out, (int32_t)value, n, s); break;
        case TVK_U8: rc = fill_impl<uint8_t>((uint8_t*)out, (uint8_t)(int64_t)value, n, s); break;
        case TVK_F64: rc = fill_impl<double>((double*)out, value, n, s); break;
        default: return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: fill of dtype %d", dtype);
    }
    return rc;
}

int tvk_cast(int dst_dtype, void* dst, int src_dtype, const void* src, int64_t n, void* stream) {
    if (n == 0) return TVK_OK;
    TVK_REQUIRE(dst && src && n > 0, "tvk_cast: null pointer or negative size");
    cudaStream_t s = (cudaStream_t)stream;
    if (dst_dtype == src_dtype) {
        TVK_CUDA_CHECK(cudaMemcpyAsync(dst, src, (size_t)n * dtype_size(dst_dtype), cudaMemcpyDeviceToDevice, s));
        return TVK_OK;
    }
    int64_t blocks = (n + (int64_t)kThreads * 8 - 1) / ((int64_t)kThreads * 8);
    int64_t cap = (int64_t)sm_count() * 16;
    const int g = (int)(blocks > cap ? cap : blocks);
    TVK_DISPATCH_ALL(dst_dtype, D, TVK_DISPATCH_ALL(src_dtype, S, (cast_kernel<D, S><<<g, kThreads, 0, s>>>((D*)dst, (const S*)src, n))));
    return launch_status("cast");
}

int tvk_copy_strided(int dst_dtype, void* dst, int src_dtype, const void* src, const tvk_iter* it, void* stream) {
    IterArgs ia;
    int rc = make_iter(it, 2, &ia);
    if (rc) return rc;
    if (ia.total == 0) return TVK_OK;
    TVK_REQUIRE(dst && src, "tvk_copy_strided: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    // Transposing copies go through shared memory so both sides stay coalesced.
    if (dst_dtype == src_dtype && (ia.ndim == 2 || ia.ndim == 3) && ia.strides[0][0] == 1 && ia.strides[1][1] == 1 &&
        ia.strides[1][0] != 1 && ia.sizes[0] >= 16 && ia.sizes[1] >= 16 && (ia.ndim == 2 || ia.sizes[2] <= 65535)) {
        // innermost (d=0): dst contiguous, src strided by strides[1][0]; next (d=1): src contiguous.
        const int64_t cols = ia.sizes[0], rows = ia.sizes[1];
        const int64_t nb = ia.ndim == 3 ? ia.sizes[2] : 1;
        dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32), (unsigned)nb);
        if (grid.y <= 65535) {
            dim3 block(32, 8);
            const int64_t bd = ia.ndim == 3 ? ia.strides[0][2] : 0, bs = ia.ndim == 3 ? ia.strides[1][2] : 0;
            switch (dtype_size(dst_dtype)) {
                case 2: transpose_copy_kernel<uint16_t><<<grid, block, 0, s>>>((uint16_t*)dst, (const uint16_t*)src, rows, cols, ia.strides[0][1], ia.strides[1][0], bd, bs); break;
                case 4: transpose_copy_kernel<uint32_t><<<grid, block, 0, s>>>((uint32_t*)dst, (const uint32_t*)src, rows, cols, ia.strides[0][1], ia.strides[1][0], bd, bs); break;
                case 8: transpose_copy_kernel<uint64_t><<<grid, block, 0, s>>>((uint64_t*)dst, (const uint64_t*)src, rows, cols, ia.strides[0][1], ia.strides[1][0], bd, bs); break;
                case 1: transpose_copy_kernel<uint8_t><<<grid, block, 0, s>>>((uint8_t*)dst, (const uint8_t*)src, rows, cols, ia.strides[0][1], ia.strides[1][0], bd, bs); break;
                default: return set_error(TVK_ERR_UNSUPPORTED, "unknown dtype %d", dst_dtype);
            }
            return launch_status("transpose copy");
        }
    }
    if (dst_dtype == src_dtype) {
        // contiguous innermost runs on both sides: move them as 16-byte packets
        const void* ptrs[2] = {dst, src};
        const size_t es[2] = {dtype_size(dst_dtype), dtype_size(dst_dtype)};
        int bcast = 0;
        IterArgs va = ia;
        if (es[0] < 16 && vectorize_iter(&va, 2, ptrs, es, &bcast) && bcast == 0) {
            const int64_t vec = (int64_t)(16 / es[0]);
            for (int o = 0; o < 2; ++o)
                for (int d = 0; d < va.ndim; ++d) va.strides[o][d] /= vec;   // element strides -> packet strides
            strided_copy_vec_kernel<<<scalar_grid(va.total), 256, 0, s>>>((uint4*)dst, (const uint4*)src, va);
            return launch_status("strided copy");
        }
    }
    const int g = scalar_grid(ia.total);
    TVK_DISPATCH_ALL(dst_dtype, D, TVK_DISPATCH_ALL(src_dtype, S, (strided_copy_kernel<D, S><<<g, 256, 0, s>>>((D*)dst, (const S*)src, ia))));
    return launch_status("strided copy");
}

}  // extern "C"
