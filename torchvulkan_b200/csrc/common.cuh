// Shared host/device helpers for the tvk kernels: status reporting, dtype traits,
// 128-bit vector access, warp/block reductions.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdarg.h>
#include <stdio.h>

#include "../../include/tvk.h"

namespace tvk {

// ---- host-side status -------------------------------------------------------
int set_error(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
void clear_error();
// Device status word of the current device (device pointer, 4 ints). Kernels with bounded
// waits or index checks record a non-zero code there; tvk_check_device_status reads it.
int* device_status_word();

#define TVK_CUDA_CHECK(expr)                                                                   \
    do {                                                                                       \
        cudaError_t _e = (expr);                                                               \
        if (_e != cudaSuccess)                                                                 \
            return ::tvk::set_error(TVK_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,             \
                                    cudaGetErrorString(_e), __FILE__, __LINE__);               \
    } while (0)

#define TVK_REQUIRE(cond, ...)                                                                 \
    do {                                                                                       \
        if (!(cond)) return ::tvk::set_error(TVK_ERR_INVALID, __VA_ARGS__);                    \
    } while (0)


// Runs the statement(s) with `T` bound to the C++ type of a floating tvk_dtype.
#define TVK_DISPATCH_FLOAT(dtype, T, ...)                                                      \
    switch (dtype) {                                                                           \
        case TVK_F32: { using T = float; __VA_ARGS__; break; }                                 \
        case TVK_F16: { using T = __half; __VA_ARGS__; break; }                                \
        case TVK_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }                        \
        default: return ::tvk::set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: dtype %d is not a floating type handled by this kernel", (int)(dtype)); \
    }

inline int launch_status(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return set_error(TVK_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return TVK_OK;
}

// Number of SMs of the current device (cached per device).
int sm_count();

inline size_t dtype_size(int dt) {
    switch (dt) {
        case TVK_F32: case TVK_I32: return 4;
        case TVK_F16: case TVK_BF16: return 2;
        case TVK_I64: case TVK_F64: return 8;
        case TVK_U8: return 1;
        default: return 0;
    }
}
inline bool is_float_dtype(int dt) { return dt == TVK_F32 || dt == TVK_F16 || dt == TVK_BF16; }

// ---- device-side conversions ------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// A 16-byte packet of T.
template <typename T> struct Vec16 {
    static constexpr int N = 16 / sizeof(T);
    union { uint4 raw; T v[N]; };
};

template <typename T> __device__ __forceinline__ Vec16<T> load16(const T* p) {
    Vec16<T> r; r.raw = *reinterpret_cast<const uint4*>(p); return r;
}
template <typename T> __device__ __forceinline__ void store16(T* p, const Vec16<T>& v) {
    *reinterpret_cast<uint4*>(p) = v.raw;
}
// Streaming variants: data touched once, keep it out of the way of L1.
template <typename T> __device__ __forceinline__ Vec16<T> load16_stream(const T* p) {
    Vec16<T> r; r.raw = __ldcs(reinterpret_cast<const uint4*>(p)); return r;
}
template <typename T> __device__ __forceinline__ void store16_stream(T* p, const Vec16<T>& v) {
    __stcs(reinterpret_cast<uint4*>(p), v.raw);
}

// exp for row kernels that read 16-bit data: the hardware exponential (its error is far below half a unit of a 16-bit
// result); fp32 data keeps expf.
template <typename T> __device__ __forceinline__ float exp_for(float x) { return sizeof(T) == 2 ? __expf(x) : expf(x); }
// 2^x by the hardware unit alone (about two units in the last place of fp32 for the small |x| used here).
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// exp(x - m) for row kernels: 16-bit data folds the subtraction and the change of base into one fused multiply-add
// (m_log2e = m * log2(e)) ahead of the hardware exponential; fp32 data keeps expf(x - m).
constexpr float kLog2e = 1.4426950408889634f;
template <typename T> __device__ __forceinline__ float exp_shifted(float x, float m, float m_log2e) {
    return sizeof(T) == 2 ? ex2_approx(fmaf(x, kLog2e, -m_log2e)) : expf(x - m);
}
// float8 product on the tensor cores (gemm.cu), for scaled_mm.cu: see the definitions for the operand rules
bool f8_product_ok(const void* a, int64_t a_rs, int64_t a_cs, const void* b, int64_t b_rs, int64_t b_cs, int64_t m, int64_t n, int64_t k);
// What the product kernel's epilogue applies to the accumulator: out = cast(acc * row_scale[r] * col_scale[c] + bias[c]).
// col_scale == nullptr: the plain product. bias (one value per column) has the output's dtype.
struct F8Epilogue {
    const float* row_scale; int64_t row_scale_stride;
    const float* col_scale; int64_t col_scale_stride;
    const void* bias;
};
int f8_product(int a_kind, int b_kind, const void* a, int64_t a_rs, const void* b, int64_t b_cs, int64_t m, int64_t n, int64_t k, void* out, int out_dtype,
               int64_t out_pitch, const F8Epilogue* epi, cudaStream_t s);
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---- warp / block reductions --------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Block-wide sum broadcast to every thread. `smem` holds 33 floats. blockDim.x % 32 == 0.
__device__ __forceinline__ float block_sum(float v, float* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? smem[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) smem[32] = t;
    }
    __syncthreads();
    return smem[32];
}
__device__ __forceinline__ float block_max(float v, float* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? smem[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) smem[32] = t;
    }
    __syncthreads();
    return smem[32];
}

// NaN-propagating max/min as ATen's amax/amin (and reduce_subgroup.slang:39-53).
__device__ __forceinline__ float nan_max(float a, float b) { return (a != a || a > b) ? a : ((b != b) ? b : (a > b ? a : b)); }
__device__ __forceinline__ float nan_min(float a, float b) { return (a != a || a < b) ? a : ((b != b) ? b : (a < b ? a : b)); }

}  // namespace tvk
