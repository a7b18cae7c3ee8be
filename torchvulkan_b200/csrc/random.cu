// Counter-based random numbers on the device: uniform, normal, Bernoulli fills and dropout.
//
// Replaces the reference's random family (src/api/ops/random.cpp, src/api/ops/dropout.cpp:10-90): a Philox generator
// keyed by the device's (seed, offset) pair, one offset reserved per launch (tvk_rng_reserve, the counterpart of
// VulkanGeneratorImpl::reserve, src/vulkan/generator.cpp:82-168). Philox4x32-10 (Salmon et al., SC'11) is a pure function
// of (key, counter): thread t of a launch draws the 128-bit block at counter (offset + launch-local block index), so a
// launch's numbers depend only on seed, offset and element position - not on the grid - and the same seed replays the
// same stream. Each block gives four 32-bit words = four elements. The streams are this implementation's own: equal
// seeds do not give the reference's (or the CPU generator's) numbers, only the same distributions.
// HBM-bound: one write per element (dropout: one read, one write, one mask byte).
#include "common.cuh"

namespace tvk {

struct Philox {
    uint32_t key[2];
    __device__ __forceinline__ Philox(uint64_t seed) { key[0] = (uint32_t)seed; key[1] = (uint32_t)(seed >> 32); }
    // the 128-bit block number `ctr` (low 64 bits; the high words carry the stream id 0) -> four words
    __device__ __forceinline__ uint4 operator()(uint64_t ctr) const {
        uint32_t c0 = (uint32_t)ctr, c1 = (uint32_t)(ctr >> 32), c2 = 0u, c3 = 0u;
        uint32_t k0 = key[0], k1 = key[1];
#pragma unroll
        for (int r = 0; r < 10; ++r) {
            const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
            const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
            const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
            c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
            k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
        }
        return make_uint4(c0, c1, c2, c3);
    }
};

// a word as a float in (0, 1]: 24 bits, never 0 (so its logarithm is finite)
__device__ __forceinline__ float unit_open0(uint32_t w) { return ((float)(w >> 8) + 1.0f) * (1.0f / 16777216.0f); }
// a word as a float in [0, 1)
__device__ __forceinline__ float unit_open1(uint32_t w) { return (float)(w >> 8) * (1.0f / 16777216.0f); }

template <typename T> __device__ __forceinline__ T rnd_store(float v) { return from_f32<T>(v); }
template <> __device__ __forceinline__ uint8_t rnd_store<uint8_t>(float v) { return v != 0.0f ? 1 : 0; }

// kind 0: uniform in [a, b); 1: normal(mean a, std b) by Box-Muller (two words per pair of values); 2: Bernoulli(p = a)
template <typename T>
__global__ void __launch_bounds__(256) random_fill_kernel(T* __restrict__ out, int64_t n, int kind, float a, float b, uint64_t seed, uint64_t offset,
                                                          const uint64_t* __restrict__ state) {
    if (state) { seed = state[0]; offset += state[1]; }        // a captured launch: the generator state of this replay
    const Philox gen(seed);
    const int64_t blocks = (n + 3) / 4;
    for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < blocks; q += (int64_t)gridDim.x * blockDim.x) {
        const uint4 w = gen(offset + (uint64_t)q);
        float v[4];
        if (kind == 0) {
            const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float u = a + (b - a) * unit_open1(ws[j]);
                v[j] = u >= b ? a : u;                               // the product may round up to b: keep the interval half open
            }
        } else if (kind == 1) {
            // Box-Muller on the hardware logarithm and sine / cosine units: their absolute error (about 2^-21) is far below
            // the 2^-24 granularity of the uniform inputs' effect on a normal sample
            const float r0 = sqrtf(-2.0f * __logf(unit_open0(w.x))), r1 = sqrtf(-2.0f * __logf(unit_open0(w.z)));
            float s0, c0, s1, c1;
            __sincosf(6.283185307179586f * unit_open1(w.y), &s0, &c0);
            __sincosf(6.283185307179586f * unit_open1(w.w), &s1, &c1);
            v[0] = a + b * r0 * c0; v[1] = a + b * r0 * s0; v[2] = a + b * r1 * c1; v[3] = a + b * r1 * s1;
        } else {
            v[0] = unit_open1(w.x) < a ? 1.f : 0.f; v[1] = unit_open1(w.y) < a ? 1.f : 0.f;
            v[2] = unit_open1(w.z) < a ? 1.f : 0.f; v[3] = unit_open1(w.w) < a ? 1.f : 0.f;
        }
        if (4 * q + 3 < n && (((uintptr_t)out) & (4 * sizeof(T) - 1)) == 0) {
            // one store of the four values (the block of four starts at a multiple of 4 * sizeof(T) when the tensor does)
            struct alignas(4 * sizeof(T)) Quad { T v[4]; } quad;
#pragma unroll
            for (int j = 0; j < 4; ++j) quad.v[j] = rnd_store<T>(v[j]);
            *(Quad*)(out + 4 * q) = quad;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (4 * q + j < n) out[4 * q + j] = rnd_store<T>(v[j]);
        }
    }
}

// out = keep ? in * scale : 0, mask = keep, keep ~ Bernoulli(keep_prob)
template <typename T>
__global__ void __launch_bounds__(256) dropout_kernel(T* __restrict__ out, uint8_t* __restrict__ mask, const T* __restrict__ in, int64_t n, float keep_prob,
                                                      float scale, uint64_t seed, uint64_t offset, const uint64_t* __restrict__ state) {
    if (state) { seed = state[0]; offset += state[1]; }
    const Philox gen(seed);
    const int64_t blocks = (n + 3) / 4;
    for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < blocks; q += (int64_t)gridDim.x * blockDim.x) {
        const uint4 w = gen(offset + (uint64_t)q);
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t i = 4 * q + j;
            if (i < n) {
                const bool keep = unit_open1(ws[j]) < keep_prob;
                out[i] = keep ? from_f32<T>(to_f32(in[i]) * scale) : from_f32<T>(0.f);
                mask[i] = keep ? 1 : 0;
            }
        }
    }
}

// The same function of (seed, offset, element index) as dropout_kernel - element i uses word i & 3 of block i >> 2 - with
// eight elements per thread: two Philox blocks, 16-byte packets of 16-bit data (two for fp32), one 8-byte store of mask bytes.
template <typename T>
__global__ void __launch_bounds__(256) dropout_vec8_kernel(T* __restrict__ out, uint8_t* __restrict__ mask, const T* __restrict__ in, int64_t n8, float keep_prob,
                                                           float scale, uint64_t seed, uint64_t offset, const uint64_t* __restrict__ state) {
    if (state) { seed = state[0]; offset += state[1]; }
    const Philox gen(seed);
    constexpr int N = Vec16<T>::N, PK = 8 / N;                     // packets per 8 elements: 1 for 16-bit data, 2 for fp32
    for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < n8; q += (int64_t)gridDim.x * blockDim.x) {
        Vec16<T> v[PK];
#pragma unroll
        for (int k = 0; k < PK; ++k) v[k] = load16_stream(in + 8 * q + k * N);
        const uint4 w0 = gen(offset + (uint64_t)(2 * q)), w1 = gen(offset + (uint64_t)(2 * q + 1));
        const uint32_t ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        uint64_t mbits = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const bool keep = unit_open1(ws[j]) < keep_prob;
            T& e = v[j / N].v[j % N];
            e = keep ? from_f32<T>(to_f32(e) * scale) : from_f32<T>(0.f);
            mbits |= (uint64_t)(keep ? 1 : 0) << (8 * j);
        }
#pragma unroll
        for (int k = 0; k < PK; ++k) store16(out + 8 * q + k * N, v[k]);
        *(uint64_t*)(mask + 8 * q) = mbits;
    }
}

static unsigned random_grid(int64_t n) {
    int64_t b = ((n + 3) / 4 + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (b > cap) b = cap;
    return (unsigned)(b < 1 ? 1 : b);
}

}  // namespace tvk

using namespace tvk;

extern "C" {

int tvk_random_fill(int kind, int dtype, void* out, int64_t n, double a, double b, uint64_t seed, uint64_t offset, const uint64_t* device_state,
                    void* stream) {
    if (n == 0) return TVK_OK;
    TVK_REQUIRE(out && n > 0, "tvk_random_fill: null output or negative size");
    TVK_REQUIRE(kind >= 0 && kind <= 2, "tvk_random_fill: unknown distribution %d", kind);
    TVK_REQUIRE(kind != 0 || a <= b, "tvk_random_fill: uniform needs from <= to");
    TVK_REQUIRE(kind != 1 || b >= 0.0, "tvk_random_fill: normal needs std >= 0");
    TVK_REQUIRE(kind != 2 || (a >= 0.0 && a <= 1.0), "tvk_random_fill: Bernoulli needs 0 <= p <= 1");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == TVK_U8) {
        random_fill_kernel<uint8_t><<<random_grid(n), 256, 0, s>>>((uint8_t*)out, n, kind, (float)a, (float)b, seed, offset, device_state);
    } else {
        TVK_DISPATCH_FLOAT(dtype, T, (random_fill_kernel<T><<<random_grid(n), 256, 0, s>>>((T*)out, n, kind, (float)a, (float)b, seed, offset, device_state)));
    }
    return launch_status("random fill");
}

int tvk_dropout(int dtype, void* out, uint8_t* mask, const void* in, int64_t n, double keep_prob, uint64_t seed, uint64_t offset,
                const uint64_t* device_state, void* stream) {
    if (n == 0) return TVK_OK;
    TVK_REQUIRE(out && mask && in && n > 0, "tvk_dropout: null pointer or negative size");
    TVK_REQUIRE(keep_prob >= 0.0 && keep_prob <= 1.0, "tvk_dropout: keep probability %f is not in [0, 1]", keep_prob);
    const float scale = keep_prob > 0.0 ? (float)(1.0 / keep_prob) : 0.f;
    cudaStream_t s = (cudaStream_t)stream;
    // whole groups of eight elements through the packet kernel when the pointers allow it, the rest (at most seven elements,
    // or everything) through the scalar one: both draw the same numbers for the same element
    int64_t done = 0;
    if (n >= 8 && (((uintptr_t)out | (uintptr_t)in) & 15) == 0 && ((uintptr_t)mask & 7) == 0) {
        const int64_t n8 = n / 8;
        int64_t b = (n8 + 255) / 256;
        const int64_t cap = (int64_t)sm_count() * 16;
        if (b > cap) b = cap;
        TVK_DISPATCH_FLOAT(dtype, T, (dropout_vec8_kernel<T><<<(unsigned)b, 256, 0, s>>>((T*)out, mask, (const T*)in, n8, (float)keep_prob, scale, seed, offset, device_state)));
        done = n8 * 8;
    }
    if (done < n) {
        const size_t es = dtype_size(dtype);
        TVK_DISPATCH_FLOAT(dtype, T, (dropout_kernel<T><<<random_grid(n - done), 256, 0, s>>>((T*)((uint8_t*)out + done * es), mask + done, (const T*)((const uint8_t*)in + done * es),
                                                                                                  n - done, (float)keep_prob, scale, seed, offset + (uint64_t)(done / 4), device_state)));
    }
    return launch_status("dropout");
}

}  // extern "C"
