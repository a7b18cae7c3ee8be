// Row-wise kernels: softmax / log_softmax (fwd + bwd), nll_loss (fwd + bwd), RMSNorm
// (fwd + bwd), embedding (fwd + deterministic dense bwd).
//
// softmax: the reference composes amax, sub, exp, sum, log, sub with an fp32 upcast and a
// downcast around them (src/api/decompositions.cpp:506-571): 6-8 passes. Here each row is
// read once into registers by one warp, reduced with shuffles and written once.
// nll_loss: src/api/ops/nllloss.cpp:79-174, src/shaders/ops/nllloss.slang:20-65.
// RMSNorm: src/api/ops/norm.cpp:169-260, src/shaders/ops/norm.slang:193-317 (256-thread shared
// memory trees, weight gradient striding over all rows per 32-column group); here rows are
// reduced with shuffles and the weight gradient comes from per-CTA register partials.
// embedding: src/api/ops/indexing.cpp:299-345, src/shaders/ops/embedding_backward.slang:36-56
// (sort + binary search + run sum); here each table row collects its hits in index order with
// a block-wide ordered scan, so the sum order is the same without a sort.
#include "common.cuh"

namespace tvk {

// ---- softmax -------------------------------------------------------------------------
// One warp per row, ITEMS values per lane (cols <= 32 * ITEMS).
template <typename TI, typename TO, bool LOG, int ITEMS>
__global__ void __launch_bounds__(128) softmax_fwd_warp_kernel(TO* __restrict__ out, const TI* __restrict__ in, int64_t rows, int64_t cols) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const TI* p = in + row * cols;
    float v[ITEMS];
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
        const int64_t c = lane + 32 * k;
        v[k] = c < cols ? to_f32(p[c]) : -INFINITY;
        m = fmaxf(m, v[k]);
    }
    m = warp_max(m);
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
        const int64_t c = lane + 32 * k;
        const float e = c < cols ? expf(v[k] - m) : 0.f;
        if (!LOG) v[k] = e;
        s += e;
    }
    s = warp_sum(s);
    TO* q = out + row * cols;
    if (LOG) {
        const float ls = logf(s);  // (x - max) - log(sum), the order of log_softmax_vulkan (decompositions.cpp:506-520)
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int64_t c = lane + 32 * k;
            if (c < cols) q[c] = from_f32<TO>((v[k] - m) - ls);
        }
    } else {
        const float inv = 1.0f / s;
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int64_t c = lane + 32 * k;
            if (c < cols) q[c] = from_f32<TO>(v[k] * inv);
        }
    }
}

// One CTA per row for long rows: three passes, the row stays in L1/L2 between them.
template <typename TI, typename TO, bool LOG>
__global__ void __launch_bounds__(256) softmax_fwd_block_kernel(TO* __restrict__ out, const TI* __restrict__ in, int64_t cols) {
    __shared__ float smem[33];
    const TI* p = in + (int64_t)blockIdx.x * cols;
    TO* q = out + (int64_t)blockIdx.x * cols;
    float m = -INFINITY;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, to_f32(p[c]));
    m = block_max(m, smem);
    float s = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += expf(to_f32(p[c]) - m);
    s = block_sum(s, smem);
    if (LOG) {
        const float ls = logf(s);
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) q[c] = from_f32<TO>((to_f32(p[c]) - m) - ls);
    } else {
        const float inv = 1.0f / s;
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) q[c] = from_f32<TO>(expf(to_f32(p[c]) - m) * inv);
    }
}

template <typename T, bool LOG, int ITEMS>
__global__ void __launch_bounds__(128) softmax_bwd_warp_kernel(T* __restrict__ gin, const T* __restrict__ gout, const T* __restrict__ y, int64_t rows, int64_t cols) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const T* g = gout + row * cols;
    const T* o = y + row * cols;
    float gv[ITEMS], yv[ITEMS];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
        const int64_t c = lane + 32 * k;
        gv[k] = c < cols ? to_f32(g[c]) : 0.f;
        yv[k] = c < cols ? to_f32(o[c]) : 0.f;
        s += LOG ? gv[k] : gv[k] * yv[k];
    }
    s = warp_sum(s);
    T* q = gin + row * cols;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
        const int64_t c = lane + 32 * k;
        if (c < cols) q[c] = from_f32<T>(LOG ? gv[k] - expf(yv[k]) * s : yv[k] * (gv[k] - s));
    }
}

template <typename T, bool LOG>
__global__ void __launch_bounds__(256) softmax_bwd_block_kernel(T* __restrict__ gin, const T* __restrict__ gout, const T* __restrict__ y, int64_t cols) {
    __shared__ float smem[33];
    const T* g = gout + (int64_t)blockIdx.x * cols;
    const T* o = y + (int64_t)blockIdx.x * cols;
    T* q = gin + (int64_t)blockIdx.x * cols;
    float s = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += LOG ? to_f32(g[c]) : to_f32(g[c]) * to_f32(o[c]);
    s = block_sum(s, smem);
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float gv = to_f32(g[c]), yv = to_f32(o[c]);
        q[c] = from_f32<T>(LOG ? gv - expf(yv) * s : yv * (gv - s));
    }
}

// Packet variants for rows of whole 16-byte packets: G lanes share a row (a power of two, about one packet per lane, at
// most P), a warp holds 32 / G rows and keeps R consecutive such groups in flight, every access is 128-bit and the
// reductions are shuffles inside the G lanes. Warps walk the row groups with a grid stride.
template <bool OPMAX> __device__ __forceinline__ float lanes_reduce(float v, int G) {
    for (int o = G >> 1; o > 0; o >>= 1) {
        const float u = __shfl_xor_sync(0xffffffffu, v, o);
        v = OPMAX ? fmaxf(v, u) : v + u;
    }
    return v;
}
template <typename TO, int N> __device__ __forceinline__ void store_packet(TO* q, const float (&v)[N]) {
    constexpr int NO = Vec16<TO>::N;
#pragma unroll
    for (int h = 0; h < N / NO; ++h) {
        Vec16<TO> o;
#pragma unroll
        for (int j = 0; j < NO; ++j) o.v[j] = from_f32<TO>(v[h * NO + j]);
        store16_stream(q + h * NO, o);
    }
}
template <typename TI, typename TO, bool LOG, int P, int R>
__global__ void __launch_bounds__(256) softmax_fwd_vec_kernel(TO* __restrict__ out, const TI* __restrict__ in, int64_t rows, int cols, int G) {
    constexpr int N = Vec16<TI>::N;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lg = lane & (G - 1), grp = lane / G, rpw = 32 / G;
    const int npk = cols / N;
    const int64_t groups = (rows + rpw - 1) / rpw, stride = (int64_t)gridDim.x * 8;
    for (int64_t g0 = ((int64_t)blockIdx.x * 8 + warp) * R; g0 < groups; g0 += stride * R) {
        Vec16<TI> xv[R][P];
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int64_t row = (g0 + q) * rpw + grp;
#pragma unroll
            for (int i = 0; i < P; ++i) {
                const int pk = i * G + lg;
                if (row < rows && pk < npk) xv[q][i] = load16_stream(in + row * cols + (int64_t)pk * N);
            }
        }
#pragma unroll
        for (int q = 0; q < R; ++q) {
            if (g0 + q >= groups) continue;       // uniform across the warp
            const int64_t row = (g0 + q) * rpw + grp;
            const bool live = row < rows;
            float m = -INFINITY;
#pragma unroll
            for (int i = 0; i < P; ++i) {
                if (live && i * G + lg < npk) {
#pragma unroll
                    for (int j = 0; j < N; ++j) m = fmaxf(m, to_f32(xv[q][i].v[j]));
                }
            }
            m = lanes_reduce<true>(m, G);
            const float m2 = m * kLog2e;
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < P; ++i) {
                if (live && i * G + lg < npk) {
#pragma unroll
                    for (int j = 0; j < N; ++j) s += exp_shifted<TI>(to_f32(xv[q][i].v[j]), m, m2);
                }
            }
            s = lanes_reduce<false>(s, G);
            const float ls = logf(s), inv = 1.0f / s;
#pragma unroll
            for (int i = 0; i < P; ++i) {
                const int pk = i * G + lg;
                if (live && pk < npk) {
                    float o[N];
#pragma unroll
                    for (int j = 0; j < N; ++j) {
                        const float x = to_f32(xv[q][i].v[j]);
                        o[j] = LOG ? (x - m) - ls : exp_shifted<TI>(x, m, m2) * inv;
                    }
                    store_packet<TO, N>(out + row * cols + (int64_t)pk * N, o);
                }
            }
        }
    }
}
template <typename T, bool LOG, int P, int R>
__global__ void __launch_bounds__(256) softmax_bwd_vec_kernel(T* __restrict__ gin, const T* __restrict__ gout, const T* __restrict__ y, int64_t rows,
                                                             int cols, int G) {
    constexpr int N = Vec16<T>::N;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lg = lane & (G - 1), grp = lane / G, rpw = 32 / G;
    const int npk = cols / N;
    const int64_t groups = (rows + rpw - 1) / rpw, stride = (int64_t)gridDim.x * 8;
    for (int64_t g0 = ((int64_t)blockIdx.x * 8 + warp) * R; g0 < groups; g0 += stride * R) {
        Vec16<T> gv[R][P], yv[R][P];
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int64_t row = (g0 + q) * rpw + grp;
#pragma unroll
            for (int i = 0; i < P; ++i) {
                const int pk = i * G + lg;
                if (row < rows && pk < npk) {
                    gv[q][i] = load16_stream(gout + row * cols + (int64_t)pk * N);
                    yv[q][i] = load16_stream(y + row * cols + (int64_t)pk * N);
                }
            }
        }
#pragma unroll
        for (int q = 0; q < R; ++q) {
            if (g0 + q >= groups) continue;       // uniform across the warp
            const int64_t row = (g0 + q) * rpw + grp;
            const bool live = row < rows;
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < P; ++i) {
                if (live && i * G + lg < npk) {
#pragma unroll
                    for (int j = 0; j < N; ++j) s += LOG ? to_f32(gv[q][i].v[j]) : to_f32(gv[q][i].v[j]) * to_f32(yv[q][i].v[j]);
                }
            }
            s = lanes_reduce<false>(s, G);
#pragma unroll
            for (int i = 0; i < P; ++i) {
                const int pk = i * G + lg;
                if (live && pk < npk) {
                    float o[N];
#pragma unroll
                    for (int j = 0; j < N; ++j) {
                        const float g = to_f32(gv[q][i].v[j]), yy = to_f32(yv[q][i].v[j]);
                        o[j] = LOG ? g - exp_for<T>(yy) * s : yy * (g - s);
                    }
                    store_packet<T, N>(gin + row * cols + (int64_t)pk * N, o);
                }
            }
        }
    }
}
// Lanes per row for the packet kernels: the smallest power of two that leaves at most four packets per lane (measured on
// 128-column fp16 rows: four packets of one row per lane ran at 5.7 TB/s, one packet per lane with four row groups in
// flight at 3.9). Returns 0 when the row does not fit (more than 128 packets).
static int vec_row_lanes(int64_t npk, int* P) {
    if (npk < 1 || npk > 128) return 0;
    int g = 1;
    while (g < 32 && (int64_t)g * 4 < npk) g <<= 1;
    *P = (int)((npk + g - 1) / g);
    return g;
}
static unsigned vec_row_ctas(int64_t rows, int G, int R, int per_sm) {
    const int64_t groups = (rows + (32 / G) - 1) / (32 / G);
    int64_t ctas = (groups + 8 * R - 1) / (8 * R);
    const int64_t cap = (int64_t)sm_count() * per_sm;
    if (ctas > cap) ctas = cap;
    return (unsigned)(ctas < 1 ? 1 : ctas);
}

template <typename TI, typename TO, bool LOG>
static int softmax_fwd_launch(TO* out, const TI* in, int64_t rows, int64_t cols, cudaStream_t s) {
    constexpr int N = Vec16<TI>::N;
    int P = 0;
    const int G = (cols % N == 0 && aligned16(in) && aligned16(out)) ? vec_row_lanes(cols / N, &P) : 0;
    if (G) {
        if (P <= 1) softmax_fwd_vec_kernel<TI, TO, LOG, 1, 4><<<vec_row_ctas(rows, G, 4, 16), 256, 0, s>>>(out, in, rows, (int)cols, G);
        else if (P <= 2) softmax_fwd_vec_kernel<TI, TO, LOG, 2, 2><<<vec_row_ctas(rows, G, 2, 16), 256, 0, s>>>(out, in, rows, (int)cols, G);
        else softmax_fwd_vec_kernel<TI, TO, LOG, 4, 1><<<vec_row_ctas(rows, G, 1, 32), 256, 0, s>>>(out, in, rows, (int)cols, G);
    } else if (cols <= 1024) {
        const unsigned blocks = (unsigned)((rows + 3) / 4);
#define L(I) softmax_fwd_warp_kernel<TI, TO, LOG, I><<<blocks, 128, 0, s>>>(out, in, rows, cols)
        if (cols <= 32) L(1); else if (cols <= 64) L(2); else if (cols <= 128) L(4); else if (cols <= 256) L(8);
        else if (cols <= 512) L(16); else L(32);
#undef L
    } else {
        softmax_fwd_block_kernel<TI, TO, LOG><<<(unsigned)rows, 256, 0, s>>>(out, in, cols);
    }
    return launch_status("softmax forward");
}

template <typename T, bool LOG>
static int softmax_bwd_launch(T* gin, const T* gout, const T* y, int64_t rows, int64_t cols, cudaStream_t s) {
    constexpr int N = Vec16<T>::N;
    int P = 0;
    const int G = (cols % N == 0 && aligned16(gin) && aligned16(gout) && aligned16(y)) ? vec_row_lanes(cols / N, &P) : 0;
    if (G) {
        if (P <= 1) softmax_bwd_vec_kernel<T, LOG, 1, 4><<<vec_row_ctas(rows, G, 4, 8), 256, 0, s>>>(gin, gout, y, rows, (int)cols, G);
        else if (P <= 2) softmax_bwd_vec_kernel<T, LOG, 2, 2><<<vec_row_ctas(rows, G, 2, 8), 256, 0, s>>>(gin, gout, y, rows, (int)cols, G);
        else softmax_bwd_vec_kernel<T, LOG, 4, 1><<<vec_row_ctas(rows, G, 1, 32), 256, 0, s>>>(gin, gout, y, rows, (int)cols, G);
    } else if (cols <= 512) {
        const unsigned blocks = (unsigned)((rows + 3) / 4);
#define L(I) softmax_bwd_warp_kernel<T, LOG, I><<<blocks, 128, 0, s>>>(gin, gout, y, rows, cols)
        if (cols <= 32) L(1); else if (cols <= 64) L(2); else if (cols <= 128) L(4); else if (cols <= 256) L(8); else L(16);
#undef L
    } else {
        softmax_bwd_block_kernel<T, LOG><<<(unsigned)rows, 256, 0, s>>>(gin, gout, y, cols);
    }
    return launch_status("softmax backward");
}

// ---- nll_loss ------------------------------------------------------------------------
template <typename T>
__global__ void nll_fwd_none_kernel(T* __restrict__ out, const T* __restrict__ logp, const int64_t* __restrict__ target,
                                    const T* __restrict__ weight, int64_t n, int64_t c, int64_t ignore_index) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t t = target[i];
    if (t == ignore_index || t < 0 || t >= c) { out[i] = from_f32<T>(0.f); return; }
    const float w = weight ? to_f32(weight[t]) : 1.f;
    out[i] = from_f32<T>(-to_f32(logp[i * c + t]) * w);
}

// Single CTA: sums in a fixed order, so the result is run-to-run identical.
template <typename T>
__global__ void __launch_bounds__(1024) nll_fwd_reduce_kernel(T* __restrict__ out, T* __restrict__ total_weight, const T* __restrict__ logp,
                                                             const int64_t* __restrict__ target, const T* __restrict__ weight, int64_t n,
                                                             int64_t c, int64_t ignore_index, int mean) {
    __shared__ float smem[33];
    float loss = 0.f, wsum = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
        const int64_t t = target[i];
        if (t == ignore_index || t < 0 || t >= c) continue;
        const float w = weight ? to_f32(weight[t]) : 1.f;
        loss -= to_f32(logp[i * c + t]) * w;
        wsum += w;
    }
    loss = block_sum(loss, smem);
    wsum = block_sum(wsum, smem);
    if (threadIdx.x == 0) {
        out[0] = from_f32<T>(mean ? loss / wsum : loss);
        total_weight[0] = from_f32<T>(wsum);
    }
}

template <typename T>
__global__ void nll_bwd_kernel(T* __restrict__ gin, const T* __restrict__ gout, const int64_t* __restrict__ target, const T* __restrict__ weight,
                               const T* __restrict__ total_weight, int64_t n, int64_t c, int reduction, int64_t ignore_index) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n * c) return;
    const int64_t i = idx / c, col = idx - i * c;
    const int64_t t = target[i];
    float v = 0.f;
    if (t != ignore_index && col == t) {
        const float w = weight ? to_f32(weight[t]) : 1.f;
        const float g = to_f32(gout[reduction == 0 ? i : 0]);
        v = -g * w;
        if (reduction == 1) v /= to_f32(total_weight[0]);
    }
    gin[idx] = from_f32<T>(v);
}

// ---- RMSNorm ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(T* __restrict__ y, float* __restrict__ rstd_out, const T* __restrict__ x,
                                                         const T* __restrict__ w, int64_t cols, float eps, int vec) {
    __shared__ float smem[33];
    constexpr int N = Vec16<T>::N;
    const T* p = x + (int64_t)blockIdx.x * cols;
    T* q = y + (int64_t)blockIdx.x * cols;
    float ss = 0.f;
    if (vec) {
        for (int64_t i = threadIdx.x; i < cols / N; i += blockDim.x) {
            Vec16<T> v = load16(p + i * N);
#pragma unroll
            for (int j = 0; j < N; ++j) { const float f = to_f32(v.v[j]); ss += f * f; }
        }
    } else {
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) { const float f = to_f32(p[c]); ss += f * f; }
    }
    ss = block_sum(ss, smem);
    const float rstd = rsqrtf(ss / (float)cols + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[blockIdx.x] = rstd;
    if (vec) {
        for (int64_t i = threadIdx.x; i < cols / N; i += blockDim.x) {
            Vec16<T> v = load16(p + i * N);
            if (w) {
                Vec16<T> wv = load16(w + i * N);
#pragma unroll
                for (int j = 0; j < N; ++j) v.v[j] = from_f32<T>(to_f32(v.v[j]) * rstd * to_f32(wv.v[j]));
            } else {
#pragma unroll
                for (int j = 0; j < N; ++j) v.v[j] = from_f32<T>(to_f32(v.v[j]) * rstd);
            }
            store16(q + i * N, v);
        }
    } else {
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
            q[c] = from_f32<T>(to_f32(p[c]) * rstd * (w ? to_f32(w[c]) : 1.f));
    }
}

// Warp-per-row forward for rows of up to MAXP 16-byte packets per lane: the row stays in registers between the sum of
// squares and the scaling, the reduction is a warp shuffle, and each warp keeps R rows in flight.
template <typename T, int MAXP, int R>
__global__ void __launch_bounds__(256) rmsnorm_fwd_warp_kernel(T* __restrict__ y, float* __restrict__ rstd_out, const T* __restrict__ x,
                                                              const T* __restrict__ w, int64_t rows, int cols, float eps) {
    constexpr int N = Vec16<T>::N;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int npk = cols / N;
    Vec16<T> wv[MAXP];
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
        const int pk = i * 32 + lane;
        if (w && pk < npk) wv[i] = load16(w + (int64_t)pk * N);
    }
    const int64_t stride = (int64_t)gridDim.x * 8;
    for (int64_t row0 = (int64_t)blockIdx.x * 8 + warp; row0 < rows; row0 += stride * R) {
        Vec16<T> xv[R][MAXP];
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int64_t row = row0 + q * stride;
#pragma unroll
            for (int i = 0; i < MAXP; ++i) {
                const int pk = i * 32 + lane;
                if (row < rows && pk < npk) xv[q][i] = load16_stream(x + row * cols + (int64_t)pk * N);
            }
        }
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int64_t row = row0 + q * stride;
            if (row >= rows) continue;               // uniform across the warp
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < MAXP; ++i) {
                if (i * 32 + lane < npk) {
#pragma unroll
                    for (int j = 0; j < N; ++j) { const float f = to_f32(xv[q][i].v[j]); ss += f * f; }
                }
            }
            const float rstd = rsqrtf(warp_sum(ss) / (float)cols + eps);
            if (lane == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
            for (int i = 0; i < MAXP; ++i) {
                const int pk = i * 32 + lane;
                if (pk < npk) {
                    Vec16<T> o;
#pragma unroll
                    for (int j = 0; j < N; ++j) {
                        const float f = to_f32(xv[q][i].v[j]) * rstd;
                        o.v[j] = from_f32<T>(w ? f * to_f32(wv[i].v[j]) : f);
                    }
                    store16_stream(y + row * cols + (int64_t)pk * N, o);
                }
            }
        }
    }
}

constexpr int kRmsBwdMaxCpt = 8;  // columns per thread kept in registers for the weight gradient

// Each CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ...: grad_x per row, and per-thread
// partial sums of grad_y * xhat for the columns the thread owns, written to partial_w[cta, :].
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(T* __restrict__ gx, float* __restrict__ partial_w, const T* __restrict__ gy,
                                                         const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ rstd,
                                                         int64_t rows, int64_t cols) {
    __shared__ float smem[33];
    float wacc[kRmsBwdMaxCpt];
#pragma unroll
    for (int k = 0; k < kRmsBwdMaxCpt; ++k) wacc[k] = 0.f;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xp = x + row * cols;
        const T* gp = gy + row * cols;
        const float rs = rstd[row];
        float dot = 0.f;
        float gw[kRmsBwdMaxCpt], xh[kRmsBwdMaxCpt];
#pragma unroll
        for (int k = 0; k < kRmsBwdMaxCpt; ++k) {
            const int64_t c = threadIdx.x + (int64_t)k * blockDim.x;
            if (c < cols) {
                const float g = to_f32(gp[c]);
                xh[k] = to_f32(xp[c]) * rs;
                gw[k] = g * (w ? to_f32(w[c]) : 1.f);
                dot += gw[k] * xh[k];
                wacc[k] += g * xh[k];
            } else {
                gw[k] = 0.f;
                xh[k] = 0.f;
            }
        }
        dot = block_sum(dot, smem) / (float)cols;
        T* op = gx + row * cols;
#pragma unroll
        for (int k = 0; k < kRmsBwdMaxCpt; ++k) {
            const int64_t c = threadIdx.x + (int64_t)k * blockDim.x;
            if (c < cols) op[c] = from_f32<T>(rs * (gw[k] - xh[k] * dot));
        }
    }
    if (partial_w) {
#pragma unroll
        for (int k = 0; k < kRmsBwdMaxCpt; ++k) {
            const int64_t c = threadIdx.x + (int64_t)k * blockDim.x;
            if (c < cols) partial_w[(int64_t)blockIdx.x * cols + c] = wacc[k];
        }
    }
}

// Warp-per-row variant for rows of up to 8 16-byte packets per lane (2048 fp16 / 1024 fp32 columns, a
// multiple of the packet): the row lives in registers, the only reduction is a warp shuffle, and every
// access is 128-bit. Each lane keeps the weight-gradient sums of the columns it owns; the CTA's eight
// warps fold them through shared memory into one partial row per CTA.
// MAXP = 16-byte packets per lane (cols <= MAXP * 32 packets), R = rows a warp keeps in flight: with one 512-column row
// per warp an SM had 32 KB of loads outstanding, which bounds the kernel by latency, not bandwidth.
template <typename T, int MAXP, int R>
__global__ void __launch_bounds__(256, (MAXP * R <= 4) ? 2 : 1) rmsnorm_bwd_warp_kernel(T* __restrict__ gx, float* __restrict__ partial_w, const T* __restrict__ gy,
                                                              const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ rstd,
                                                              int64_t rows, int cols) {
    constexpr int N = Vec16<T>::N;
    __shared__ float fold[8][32 * N];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int npk = cols / N;
    float wacc[MAXP][N];
    Vec16<T> wv[MAXP];
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
#pragma unroll
        for (int j = 0; j < N; ++j) wacc[i][j] = 0.f;
        const int pk = i * 32 + lane;
        if (w && pk < npk) wv[i] = load16(w + (int64_t)pk * N);
        else {
#pragma unroll
            for (int j = 0; j < N; ++j) wv[i].v[j] = from_f32<T>(1.f);
        }
    }
    const float inv_cols = 1.0f / (float)cols;
    const int64_t stride = (int64_t)gridDim.x * 8;
    for (int64_t row0 = (int64_t)blockIdx.x * 8 + warp; row0 < rows; row0 += stride * R) {
        Vec16<T> gv[R][MAXP], xv[R][MAXP];
        float rs[R], dot[R];
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int64_t row = row0 + q * stride;
            rs[q] = row < rows ? rstd[row] : 0.f;
#pragma unroll
            for (int i = 0; i < MAXP; ++i) {
                const int pk = i * 32 + lane;
                if (row < rows && pk < npk) {
                    gv[q][i] = load16_stream(gy + row * cols + (int64_t)pk * N);
                    xv[q][i] = load16_stream(x + row * cols + (int64_t)pk * N);
                }
            }
        }
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int64_t row = row0 + q * stride;
            dot[q] = 0.f;
#pragma unroll
            for (int i = 0; i < MAXP; ++i) {
                const int pk = i * 32 + lane;
                if (row < rows && pk < npk) {
#pragma unroll
                    for (int j = 0; j < N; ++j) {
                        const float g = to_f32(gv[q][i].v[j]), xh = to_f32(xv[q][i].v[j]) * rs[q];
                        dot[q] += g * to_f32(wv[i].v[j]) * xh;
                        wacc[i][j] += g * xh;
                    }
                }
            }
        }
#pragma unroll
        for (int q = 0; q < R; ++q) dot[q] = warp_sum(dot[q]) * inv_cols;
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int64_t row = row0 + q * stride;
#pragma unroll
            for (int i = 0; i < MAXP; ++i) {
                const int pk = i * 32 + lane;
                if (row < rows && pk < npk) {
                    Vec16<T> o;
#pragma unroll
                    for (int j = 0; j < N; ++j) {
                        const float xh = to_f32(xv[q][i].v[j]) * rs[q];
                        o.v[j] = from_f32<T>(rs[q] * (to_f32(gv[q][i].v[j]) * to_f32(wv[i].v[j]) - xh * dot[q]));
                    }
                    store16_stream(gx + row * cols + (int64_t)pk * N, o);
                }
            }
        }
    }
    if (!partial_w) return;
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
        if (i * 32 * N >= cols) break;          // uniform
        __syncthreads();
#pragma unroll
        for (int j = 0; j < N; ++j) fold[warp][lane * N + j] = wacc[i][j];
        __syncthreads();
        for (int c = threadIdx.x; c < 32 * N; c += 256) {
            const int col = i * 32 * N + c;
            if (col < cols) {
                float s = 0.f;
#pragma unroll
                for (int k = 0; k < 8; ++k) s += fold[k][c];
                partial_w[(int64_t)blockIdx.x * cols + col] = s;
            }
        }
    }
}

// out[c] = sum over parts of partial[part, c]; 32 columns x 32 part-lanes per CTA (a few hundred parts: every thread
// issues all of its loads at once, so the kernel costs about one memory latency).
template <typename T>
__global__ void __launch_bounds__(1024) fold_columns_kernel(T* __restrict__ out, const float* __restrict__ partial, int64_t nparts, int64_t cols) {
    __shared__ float acc[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t c = (int64_t)blockIdx.x * 32 + tx;
    float s = 0.f;
    if (c < cols) {
        int64_t k = ty;
        for (; k + 32 * 7 < nparts; k += 32 * 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = partial[(k + 32 * u) * cols + c];
#pragma unroll
            for (int u = 0; u < 8; ++u) s += v[u];
        }
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = (k + 32 * u < nparts) ? partial[(k + 32 * u) * cols + c] : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u) s += v[u];
    }
    acc[ty][tx] = s;
    __syncthreads();
    if (ty == 0 && c < cols) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 32; ++k) t += acc[k][tx];
        out[c] = from_f32<T>(t);
    }
}

static int rms_bwd_ctas(int64_t rows) {
    int64_t n = (int64_t)sm_count() * 4;
    if (n > rows) n = rows;
    return (int)(n < 1 ? 1 : n);
}

// ---- embedding ---------------------------------------------------------------------------
template <typename T>
__global__ void embedding_fwd_kernel(T* __restrict__ out, const T* __restrict__ table, const int64_t* __restrict__ idx, int64_t num_idx,
                                     int64_t num_rows, int64_t dim, int vec, int* status) {
    constexpr int N = Vec16<T>::N;
    const int64_t i = blockIdx.x;
    const int64_t r = idx[i];
    T* q = out + i * dim;
    const bool ok = r >= 0 && r < num_rows;
    if (!ok && threadIdx.x == 0 && status) {
        if (atomicCAS(status, 0, 2) == 0) { status[1] = 1; status[2] = (int)i; status[3] = (int)r; }
    }
    const T* p = table + (ok ? r : 0) * dim;
    if (vec) {
        for (int64_t k = threadIdx.x; k < dim / N; k += blockDim.x) {
            Vec16<T> v;
            if (ok) v = load16(p + k * N); else v.raw = make_uint4(0, 0, 0, 0);
            store16(q + k * N, v);
        }
    } else {
        for (int64_t c = threadIdx.x; c < dim; c += blockDim.x) q[c] = ok ? p[c] : from_f32<T>(0.f);
    }
}

// Warp-per-index gather for rows of whole 16-byte packets: each warp reads R indices, then copies the R table rows with R
// packets per lane in flight (one CTA per index with a single dependent load chain reached about a quarter of the HBM
// write rate on long index lists). Out-of-range indices write zeros and record (index position, value) in the status word.
template <typename T, int R>
__global__ void __launch_bounds__(256) embedding_fwd_warp_kernel(T* __restrict__ out, const T* __restrict__ table, const int64_t* __restrict__ idx,
                                                                int64_t num_idx, int64_t num_rows, int64_t dim, int* status) {
    constexpr int N = Vec16<T>::N;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t npk = dim / N, stride = (int64_t)gridDim.x * 8;
    for (int64_t i0 = (int64_t)blockIdx.x * 8 + warp; i0 < num_idx; i0 += stride * R) {
        const T* p[R];
        bool ok[R];
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int64_t i = i0 + q * stride;
            const int64_t r = i < num_idx ? idx[i] : 0;
            ok[q] = r >= 0 && r < num_rows;
            if (!ok[q] && lane == 0 && status) {
                if (atomicCAS(status, 0, 2) == 0) { status[1] = 1; status[2] = (int)i; status[3] = (int)r; }
            }
            p[q] = table + (ok[q] ? r : 0) * dim;
        }
        for (int64_t k = lane; k < npk; k += 32) {
            Vec16<T> v[R];
#pragma unroll
            for (int q = 0; q < R; ++q) {
                if (ok[q]) v[q] = load16(p[q] + k * N); else v[q].raw = make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int q = 0; q < R; ++q) {
                const int64_t i = i0 + q * stride;
                if (i < num_idx) store16_stream(out + i * dim + k * N, v[q]);
            }
        }
    }
}

// grid (num_rows, column slabs of 1024). The CTA scans the index list in order, keeps the hits
// of its table row in a shared list (ordered compaction), and adds their gradient rows in that
// order in fp32.
// Indices are taken 2048 at a time, eight consecutive ones per thread (their loads go out together), the hits are placed
// by a block-wide exclusive scan (so the list is in index order), and the gradient rows of eight hits are loaded together
// before they are added one after the other: the order of the fp32 additions, and with it every bit of the result, is
// that of a sequential walk over the indices.
template <typename T>
__global__ void __launch_bounds__(256) embedding_bwd_kernel(T* __restrict__ gtable, const T* __restrict__ grad, const int64_t* __restrict__ idx,
                                                           int64_t num_idx, int64_t dim, int64_t padding_idx) {
    constexpr int PER = 8, CHUNK = 256 * PER;
    __shared__ int hits[CHUNK];
    __shared__ int warp_totals[8];
    const int64_t r = blockIdx.x;
    const int64_t c0 = (int64_t)blockIdx.y * 1024;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (r != padding_idx) {
        for (int64_t base = 0; base < num_idx; base += CHUNK) {
            const int64_t i0 = base + (int64_t)threadIdx.x * PER;
            int64_t v[PER];
#pragma unroll
            for (int j = 0; j < PER; ++j) v[j] = (i0 + j < num_idx) ? idx[i0 + j] : (int64_t)-1 - r;     // never equal to r
            unsigned mask = 0;
#pragma unroll
            for (int j = 0; j < PER; ++j) mask |= (v[j] == r ? 1u : 0u) << j;
            const int mine = __popc(mask);
            int incl = mine;                                         // inclusive scan over the warp
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            if (lane == 31) warp_totals[warp] = incl;
            __syncthreads();
            int offset = incl - mine, cnt = 0;
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                const int t = warp_totals[w];
                if (w < warp) offset += t;
                cnt += t;
            }
#pragma unroll
            for (int j = 0; j < PER; ++j)
                if (mask & (1u << j)) hits[offset++] = threadIdx.x * PER + j;
            __syncthreads();
            int h = 0;
            for (; h + 8 <= cnt; h += 8) {
                float g[8][4];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const T* gp = grad + (base + hits[h + u]) * dim + c0;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int64_t c = threadIdx.x + 256 * k;
                        g[u][k] = (c0 + c < dim) ? to_f32(gp[c]) : 0.f;
                    }
                }
#pragma unroll
                for (int u = 0; u < 8; ++u)
#pragma unroll
                    for (int k = 0; k < 4; ++k) acc[k] += g[u][k];
            }
            for (; h < cnt; ++h) {
                const T* gp = grad + (base + hits[h]) * dim + c0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int64_t c = threadIdx.x + 256 * k;
                    if (c0 + c < dim) acc[k] += to_f32(gp[c]);
                }
            }
            __syncthreads();
        }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int64_t c = c0 + threadIdx.x + 256 * k;
        if (c < dim) gtable[r * dim + c] = from_f32<T>(acc[k]);
    }
}

}  // namespace tvk

using namespace tvk;

extern "C" {

int tvk_softmax_forward(int is_log, int in_dtype, int out_dtype, void* out, const void* in, int64_t rows, int64_t cols, void* stream) {
    TVK_REQUIRE(rows >= 0 && cols >= 0, "tvk_softmax_forward: negative extent");
    if (rows == 0 || cols == 0) return TVK_OK;
    TVK_REQUIRE(out && in, "tvk_softmax_forward: null pointer");
    TVK_REQUIRE(rows <= 0x7fffffffLL, "tvk_softmax_forward: too many rows");
    cudaStream_t s = (cudaStream_t)stream;
    int rc = TVK_OK;
    if (out_dtype == in_dtype) {
        if (is_log) { TVK_DISPATCH_FLOAT(in_dtype, T, rc = (softmax_fwd_launch<T, T, true>((T*)out, (const T*)in, rows, cols, s))); }
        else { TVK_DISPATCH_FLOAT(in_dtype, T, rc = (softmax_fwd_launch<T, T, false>((T*)out, (const T*)in, rows, cols, s))); }
    } else if (out_dtype == TVK_F32) {
        if (is_log) { TVK_DISPATCH_FLOAT(in_dtype, T, rc = (softmax_fwd_launch<T, float, true>((float*)out, (const T*)in, rows, cols, s))); }
        else { TVK_DISPATCH_FLOAT(in_dtype, T, rc = (softmax_fwd_launch<T, float, false>((float*)out, (const T*)in, rows, cols, s))); }
    } else {
        return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: softmax from dtype %d to dtype %d", in_dtype, out_dtype);
    }
    return rc;
}

int tvk_softmax_backward(int is_log, int dtype, void* grad_in, const void* grad_out, const void* out, int64_t rows, int64_t cols,
                         void* stream) {
    TVK_REQUIRE(rows >= 0 && cols >= 0, "tvk_softmax_backward: negative extent");
    if (rows == 0 || cols == 0) return TVK_OK;
    TVK_REQUIRE(grad_in && grad_out && out, "tvk_softmax_backward: null pointer");
    TVK_REQUIRE(rows <= 0x7fffffffLL, "tvk_softmax_backward: too many rows");
    cudaStream_t s = (cudaStream_t)stream;
    int rc = TVK_OK;
    if (is_log) { TVK_DISPATCH_FLOAT(dtype, T, rc = (softmax_bwd_launch<T, true>((T*)grad_in, (const T*)grad_out, (const T*)out, rows, cols, s))); }
    else { TVK_DISPATCH_FLOAT(dtype, T, rc = (softmax_bwd_launch<T, false>((T*)grad_in, (const T*)grad_out, (const T*)out, rows, cols, s))); }
    return rc;
}

int tvk_nll_loss_forward(int dtype, void* out, void* total_weight, const void* logp, const int64_t* target, const void* weight,
                         int64_t n, int64_t c, int reduction, int64_t ignore_index, void* stream) {
    TVK_REQUIRE(n >= 0 && c >= 0, "tvk_nll_loss_forward: negative extent");
    TVK_REQUIRE(reduction >= 0 && reduction <= 2, "tvk_nll_loss_forward: reduction must be 0 (none), 1 (mean) or 2 (sum)");
    TVK_REQUIRE(out && total_weight, "tvk_nll_loss_forward: null output");
    TVK_REQUIRE(n == 0 || (logp && target), "tvk_nll_loss_forward: null input");
    cudaStream_t s = (cudaStream_t)stream;
    if (reduction == 0) {
        if (n == 0) return TVK_OK;
        TVK_DISPATCH_FLOAT(dtype, T, (nll_fwd_none_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>((T*)out, (const T*)logp, target, (const T*)weight, n, c, ignore_index)));
        // total_weight is unused for reduction none; keep it defined.
        int rc = tvk_fill(dtype, total_weight, 0.0, 1, stream);
        if (rc) return rc;
    } else {
        TVK_DISPATCH_FLOAT(dtype, T, (nll_fwd_reduce_kernel<T><<<1, 1024, 0, s>>>((T*)out, (T*)total_weight, (const T*)logp, target, (const T*)weight, n, c, ignore_index, reduction == 1)));
    }
    return launch_status("nll_loss forward");
}

int tvk_nll_loss_backward(int dtype, void* grad_in, const void* grad_out, const int64_t* target, const void* weight,
                          const void* total_weight, int64_t n, int64_t c, int reduction, int64_t ignore_index, void* stream) {
    TVK_REQUIRE(n >= 0 && c >= 0, "tvk_nll_loss_backward: negative extent");
    TVK_REQUIRE(reduction >= 0 && reduction <= 2, "tvk_nll_loss_backward: reduction must be 0 (none), 1 (mean) or 2 (sum)");
    if (n == 0 || c == 0) return TVK_OK;
    TVK_REQUIRE(grad_in && grad_out && target, "tvk_nll_loss_backward: null pointer");
    TVK_REQUIRE(reduction != 1 || total_weight, "tvk_nll_loss_backward: mean reduction needs total_weight");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t total = n * c;
    TVK_DISPATCH_FLOAT(dtype, T, (nll_bwd_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, s>>>((T*)grad_in, (const T*)grad_out, target, (const T*)weight, (const T*)total_weight, n, c, reduction, ignore_index)));
    return launch_status("nll_loss backward");
}

int tvk_rmsnorm_forward(int dtype, void* y, float* rstd, const void* x, const void* weight, int64_t rows, int64_t cols, double eps,
                        void* stream) {
    TVK_REQUIRE(rows >= 0 && cols >= 0, "tvk_rmsnorm_forward: negative extent");
    if (rows == 0 || cols == 0) return TVK_OK;
    TVK_REQUIRE(y && x, "tvk_rmsnorm_forward: null pointer");
    TVK_REQUIRE(rows <= 0x7fffffffLL, "tvk_rmsnorm_forward: too many rows");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t es = dtype_size(dtype);
    const int n = es ? (int)(16 / es) : 1;
    const int vec = aligned16(y) && aligned16(x) && (!weight || aligned16(weight)) && cols % n == 0;
    const int64_t npk = cols / n;
    if (vec && npk <= 4 * 32) {
        int64_t ctas = (rows + 7) / 8;
        const int64_t cap = (int64_t)sm_count() * 8;
        if (ctas > cap) ctas = cap;
        if (npk <= 64) {
            TVK_DISPATCH_FLOAT(dtype, T, (rmsnorm_fwd_warp_kernel<T, 2, 4><<<(unsigned)ctas, 256, 0, s>>>((T*)y, rstd, (const T*)x, (const T*)weight, rows, (int)cols, (float)eps)));
        } else {
            TVK_DISPATCH_FLOAT(dtype, T, (rmsnorm_fwd_warp_kernel<T, 4, 2><<<(unsigned)ctas, 256, 0, s>>>((T*)y, rstd, (const T*)x, (const T*)weight, rows, (int)cols, (float)eps)));
        }
        return launch_status("rmsnorm forward");
    }
    int threads = 32;
    while (threads < 256 && (int64_t)threads * n < cols) threads <<= 1;
    TVK_DISPATCH_FLOAT(dtype, T, (rmsnorm_fwd_kernel<T><<<(unsigned)rows, threads, 0, s>>>((T*)y, rstd, (const T*)x, (const T*)weight, cols, (float)eps, vec)));
    return launch_status("rmsnorm forward");
}

int tvk_rmsnorm_backward_workspace_size(int64_t rows, int64_t cols, uint64_t* bytes) {
    if (!bytes) return set_error(TVK_ERR_INVALID, "tvk_rmsnorm_backward_workspace_size: null output");
    TVK_REQUIRE(rows >= 0 && cols >= 0, "tvk_rmsnorm_backward_workspace_size: negative extent");
    *bytes = (uint64_t)rms_bwd_ctas(rows) * (uint64_t)cols * sizeof(float);
    return TVK_OK;
}

int tvk_rmsnorm_backward(int dtype, void* grad_x, void* grad_w, const void* grad_y, const void* x, const void* weight,
                         const float* rstd, int64_t rows, int64_t cols, void* workspace, uint64_t workspace_bytes, void* stream) {
    TVK_REQUIRE(rows >= 0 && cols >= 0, "tvk_rmsnorm_backward: negative extent");
    if (cols == 0) return TVK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (rows == 0) return grad_w ? tvk_fill(dtype, grad_w, 0.0, cols, stream) : TVK_OK;
    TVK_REQUIRE(grad_x && grad_y && x && rstd, "tvk_rmsnorm_backward: null pointer");
    int threads = 32;
    while (threads < 256 && threads < cols) threads <<= 1;
    if ((int64_t)threads * kRmsBwdMaxCpt < cols)
        return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: rms_norm backward with %lld columns (max %d)",
                         (long long)cols, 256 * kRmsBwdMaxCpt);
    const int ctas = rms_bwd_ctas(rows);
    float* partial = nullptr;
    if (grad_w) {
        const uint64_t need = (uint64_t)ctas * (uint64_t)cols * sizeof(float);
        TVK_REQUIRE(workspace && workspace_bytes >= need, "tvk_rmsnorm_backward: workspace of %llu bytes required, %llu given",
                    (unsigned long long)need, (unsigned long long)workspace_bytes);
        partial = (float*)workspace;
    }
    const int64_t pkt = (int64_t)(16 / dtype_size(dtype));
    const bool warp_rows = cols % pkt == 0 && cols <= 8 * 32 * pkt && aligned16(grad_x) && aligned16(grad_y) && aligned16(x) && (!weight || aligned16(weight));
    int nparts = ctas;
    if (warp_rows) {
        // fewer, fatter CTAs (8 rows in flight each): one partial row per CTA
        int64_t want = ((rows + 7) / 8 < (int64_t)sm_count() * 2) ? (rows + 7) / 8 : (int64_t)sm_count() * 2;
        if (want > ctas) want = ctas;
        nparts = (int)(want < 1 ? 1 : want);
        const int64_t lane_packets = (cols * (int64_t)dtype_size(dtype) / 16 + 31) / 32;      // packets per lane
        if (lane_packets <= 2) {
            TVK_DISPATCH_FLOAT(dtype, T, (rmsnorm_bwd_warp_kernel<T, 2, 2><<<nparts, 256, 0, s>>>((T*)grad_x, partial, (const T*)grad_y, (const T*)x, (const T*)weight, rstd, rows, (int)cols)));
        } else if (lane_packets <= 4) {
            TVK_DISPATCH_FLOAT(dtype, T, (rmsnorm_bwd_warp_kernel<T, 4, 2><<<nparts, 256, 0, s>>>((T*)grad_x, partial, (const T*)grad_y, (const T*)x, (const T*)weight, rstd, rows, (int)cols)));
        } else {
            TVK_DISPATCH_FLOAT(dtype, T, (rmsnorm_bwd_warp_kernel<T, 8, 1><<<nparts, 256, 0, s>>>((T*)grad_x, partial, (const T*)grad_y, (const T*)x, (const T*)weight, rstd, rows, (int)cols)));
        }
    } else {
        TVK_DISPATCH_FLOAT(dtype, T, (rmsnorm_bwd_kernel<T><<<ctas, threads, 0, s>>>((T*)grad_x, partial, (const T*)grad_y, (const T*)x, (const T*)weight, rstd, rows, cols)));
    }
    if (grad_w) {
        TVK_DISPATCH_FLOAT(dtype, T, (fold_columns_kernel<T><<<(unsigned)((cols + 31) / 32), 1024, 0, s>>>((T*)grad_w, partial, nparts, cols)));
    }
    return launch_status("rmsnorm backward");
}

int tvk_embedding_forward(int dtype, void* out, const void* table, const int64_t* idx, int64_t num_idx, int64_t num_rows, int64_t dim,
                          void* stream) {
    TVK_REQUIRE(num_idx >= 0 && num_rows >= 0 && dim >= 0, "tvk_embedding_forward: negative extent");
    if (num_idx == 0 || dim == 0) return TVK_OK;
    TVK_REQUIRE(out && table && idx, "tvk_embedding_forward: null pointer");
    TVK_REQUIRE(num_idx <= 0x7fffffffLL, "tvk_embedding_forward: too many indices");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t es = dtype_size(dtype);
    TVK_REQUIRE(es == 2 || es == 4, "tvk_embedding_forward: dtype %d not supported", dtype);
    const int n = (int)(16 / es);
    const int vec = aligned16(out) && aligned16(table) && dim % n == 0;
    int threads = 32;
    while (threads < 256 && (int64_t)threads * n < dim) threads <<= 1;
    int* status = device_status_word();
    // The copy does not interpret the values: run it on same-width integer types.
    if (vec && num_idx >= 1024) {
        int64_t ctas = (num_idx + 31) / 32;
        const int64_t cap = (int64_t)sm_count() * 8;
        if (ctas > cap) ctas = cap;
        if (es == 2) embedding_fwd_warp_kernel<__half, 4><<<(unsigned)ctas, 256, 0, s>>>((__half*)out, (const __half*)table, idx, num_idx, num_rows, dim, status);
        else embedding_fwd_warp_kernel<float, 4><<<(unsigned)ctas, 256, 0, s>>>((float*)out, (const float*)table, idx, num_idx, num_rows, dim, status);
        return launch_status("embedding forward");
    }
    if (es == 2) embedding_fwd_kernel<__half><<<(unsigned)num_idx, threads, 0, s>>>((__half*)out, (const __half*)table, idx, num_idx, num_rows, dim, vec, status);
    else embedding_fwd_kernel<float><<<(unsigned)num_idx, threads, 0, s>>>((float*)out, (const float*)table, idx, num_idx, num_rows, dim, vec, status);
    return launch_status("embedding forward");
}

int tvk_embedding_backward(int dtype, void* grad_table, const void* grad, const int64_t* idx, int64_t num_idx, int64_t num_rows,
                           int64_t dim, int64_t padding_idx, void* stream) {
    TVK_REQUIRE(num_idx >= 0 && num_rows >= 0 && dim >= 0, "tvk_embedding_backward: negative extent");
    if (num_rows == 0 || dim == 0) return TVK_OK;
    TVK_REQUIRE(grad_table && (num_idx == 0 || (grad && idx)), "tvk_embedding_backward: null pointer");
    TVK_REQUIRE(num_rows <= 0x7fffffffLL && (dim + 1023) / 1024 <= 65535, "tvk_embedding_backward: table too large");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((unsigned)num_rows, (unsigned)((dim + 1023) / 1024));
    TVK_DISPATCH_FLOAT(dtype, T, (embedding_bwd_kernel<T><<<grid, 256, 0, s>>>((T*)grad_table, (const T*)grad, idx, num_idx, dim, padding_idx)));
    return launch_status("embedding backward");
}

}  // extern "C"
