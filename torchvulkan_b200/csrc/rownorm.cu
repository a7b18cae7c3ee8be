// Row-wise kernels next to softmax / RMSNorm: LayerNorm and GroupNorm forward + backward, cross-entropy as ONE pass over
// the logits each way (log_softmax + nll_loss fused), and cumulative scans.
//
// Replaces layer_norm_shader / layer_norm_backward_shader / group_norm (src/api/ops/norm.cpp:264-325 and the rowForward,
// rowBackwardInput, rowBackwardParams entry points of src/shaders/ops/norm.slang:193-317), the log_softmax -> nll_loss
// chain of src/api/decompositions.cpp:506-571 + src/api/ops/nllloss.cpp:79-174 when a caller asks for the fused form, and
// cumscan (src/api/ops/scan.cpp:35-102, src/shaders/ops/scan.slang). Statistics and sums are fp32 whatever the storage
// type (src/shaders/core/dtype.slang:256-283); the variance is two-pass (mean first), as norm.slang:204-226 does.
#include "common.cuh"

namespace tvk {

constexpr int kNormThreads = 256;

__device__ __forceinline__ float block_sum256(float v, float* smem) { return block_sum(v, smem); }
__device__ __forceinline__ bool aligned16_dev(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---- LayerNorm / GroupNorm forward -------------------------------------------------------------------------------
// One CTA per row of `cols` contiguous values. The affine parameters are indexed by (column / aff_div): aff_div = 1 for
// LayerNorm (one weight per column), H*W for GroupNorm rows (one weight per channel of the group, aff_base = first channel
// of the row's group).
template <typename T>
__global__ void __launch_bounds__(kNormThreads) rownorm_fwd_kernel(T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                  const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                                                                  int64_t cols, float eps, int64_t aff_div, int64_t aff_groups, int64_t aff_per_row) {
    __shared__ float smem[33];
    const int64_t row = blockIdx.x;
    const T* p = x + row * cols;
    T* q = y + row * cols;
    const int64_t aff_base = aff_groups > 0 ? (row % aff_groups) * aff_per_row : 0;
    constexpr int N = Vec16<T>::N;
    const bool vec = (cols % N == 0) && aligned16_dev(p) && aligned16_dev(q);
    float s = 0.f;
    if (vec) {
        for (int64_t i = threadIdx.x; i < cols / N; i += blockDim.x) {
            const Vec16<T> v = load16(p + i * N);
#pragma unroll
            for (int j = 0; j < N; ++j) s += to_f32(v.v[j]);
        }
    } else {
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += to_f32(p[c]);
    }
    const float mean = block_sum256(s, smem) / (float)cols;
    float ss = 0.f;
    if (vec) {
        for (int64_t i = threadIdx.x; i < cols / N; i += blockDim.x) {
            const Vec16<T> v = load16(p + i * N);
#pragma unroll
            for (int j = 0; j < N; ++j) { const float d = to_f32(v.v[j]) - mean; ss += d * d; }
        }
    } else {
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) { const float d = to_f32(p[c]) - mean; ss += d * d; }
    }
    const float rstd = rsqrtf(block_sum256(ss, smem) / (float)cols + eps);
    if (threadIdx.x == 0) {
        if (mean_out) mean_out[row] = mean;
        if (rstd_out) rstd_out[row] = rstd;
    }
    if (vec && aff_div == 1 && (!w || aligned16_dev(w)) && (!b || aligned16_dev(b))) {
        for (int64_t i = threadIdx.x; i < cols / N; i += blockDim.x) {
            Vec16<T> v = load16(p + i * N), wv, bv;
            if (w) wv = load16(w + i * N);
            if (b) bv = load16(b + i * N);
#pragma unroll
            for (int j = 0; j < N; ++j) {
                float o = (to_f32(v.v[j]) - mean) * rstd;
                if (w) o *= to_f32(wv.v[j]);
                if (b) o += to_f32(bv.v[j]);
                v.v[j] = from_f32<T>(o);
            }
            store16(q + i * N, v);
        }
    } else {
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
            const int64_t a = aff_base + c / aff_div;
            float o = (to_f32(p[c]) - mean) * rstd;
            if (w) o *= to_f32(w[a]);
            if (b) o += to_f32(b[a]);
            q[c] = from_f32<T>(o);
        }
    }
}

// ---- LayerNorm backward ----------------------------------------------------------------------------------------------
// grad_x = rstd * (g - mean(g) - xhat * mean(g * xhat)) with g = grad_y * w and xhat = (x - mean) * rstd. A CTA walks
// rows blockIdx.x, + gridDim.x, ...; every thread keeps the partial sums of grad_w = sum grad_y * xhat and grad_b = sum
// grad_y for the CPT columns it owns, written once per CTA to partial[cta][2][cols] and folded by ln_fold_kernel.
template <typename T, int CPT>
__global__ void __launch_bounds__(kNormThreads) layernorm_bwd_kernel(T* __restrict__ gx, float* __restrict__ partial, const T* __restrict__ gy,
                                                                    const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ mean,
                                                                    const float* __restrict__ rstd, int64_t rows, int64_t cols) {
    __shared__ float smem[33];
    float wacc[CPT], bacc[CPT];
#pragma unroll
    for (int k = 0; k < CPT; ++k) { wacc[k] = 0.f; bacc[k] = 0.f; }
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xp = x + row * cols;
        const T* gp = gy + row * cols;
        const float mu = mean[row], rs = rstd[row];
        float g[CPT], xh[CPT];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
            const int64_t c = threadIdx.x + (int64_t)k * kNormThreads;
            if (c < cols) {
                const float gyv = to_f32(gp[c]);
                xh[k] = (to_f32(xp[c]) - mu) * rs;
                g[k] = gyv * (w ? to_f32(w[c]) : 1.f);
                s1 += g[k];
                s2 += g[k] * xh[k];
                wacc[k] += gyv * xh[k];
                bacc[k] += gyv;
            } else {
                g[k] = 0.f; xh[k] = 0.f;
            }
        }
        s1 = block_sum256(s1, smem) / (float)cols;
        s2 = block_sum256(s2, smem) / (float)cols;
        if (gx) {
            T* op = gx + row * cols;
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const int64_t c = threadIdx.x + (int64_t)k * kNormThreads;
                if (c < cols) op[c] = from_f32<T>(rs * (g[k] - s1 - xh[k] * s2));
            }
        }
    }
    if (partial) {
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
            const int64_t c = threadIdx.x + (int64_t)k * kNormThreads;
            if (c < cols) {
                partial[((int64_t)blockIdx.x * 2 + 0) * cols + c] = wacc[k];
                partial[((int64_t)blockIdx.x * 2 + 1) * cols + c] = bacc[k];
            }
        }
    }
}

// Warp-per-row LayerNorm for rows of whole 16-byte packets, at most MAXP packets per lane (rows of up to 128 packets; longer rows take the CTA-per-row kernels): the
// row lives in registers, both statistics are warp shuffles, every access is 128-bit, and each warp keeps R rows in
// flight (one 1 KB row per warp leaves an SM with too few bytes outstanding to cover the memory latency).
template <typename T, int MAXP, int R>
__global__ void __launch_bounds__(256, MAXP <= 2 ? 3 : 2) layernorm_fwd_warp_kernel(T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                                                                int64_t rows, int cols, float eps) {
    constexpr int N = Vec16<T>::N;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int npk = cols / N;
    const float inv_cols = 1.0f / (float)cols;
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
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < MAXP; ++i) {
                if (i * 32 + lane < npk) {
#pragma unroll
                    for (int j = 0; j < N; ++j) s += to_f32(xv[q][i].v[j]);
                }
            }
            const float mean = warp_sum(s) * inv_cols;
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < MAXP; ++i) {
                if (i * 32 + lane < npk) {
#pragma unroll
                    for (int j = 0; j < N; ++j) { const float d = to_f32(xv[q][i].v[j]) - mean; ss += d * d; }
                }
            }
            const float rstd = rsqrtf(warp_sum(ss) * inv_cols + eps);
            if (lane == 0) {
                if (mean_out) mean_out[row] = mean;
                if (rstd_out) rstd_out[row] = rstd;
            }
#pragma unroll
            for (int i = 0; i < MAXP; ++i) {
                const int pk = i * 32 + lane;
                if (pk < npk) {
                    // weight and bias come from L1 at each use: holding them in registers costs a resident CTA per SM
                    Vec16<T> o, wv, bv;
                    if (w) wv = load16(w + (int64_t)pk * N);
                    if (b) bv = load16(b + (int64_t)pk * N);
#pragma unroll
                    for (int j = 0; j < N; ++j) {
                        float v = (to_f32(xv[q][i].v[j]) - mean) * rstd;
                        if (w) v *= to_f32(wv.v[j]);
                        if (b) v += to_f32(bv.v[j]);
                        o.v[j] = from_f32<T>(v);
                    }
                    store16_stream(y + row * cols + (int64_t)pk * N, o);
                }
            }
        }
    }
}

// The backward pass in the same shape: each lane also keeps the grad_w / grad_b sums of the columns it owns over all the
// rows its warp walks; the CTA's eight warps fold them through shared memory into partial[cta][2][cols].
template <typename T, int MAXP, int R>
__global__ void __launch_bounds__(256, MAXP <= 2 ? 2 : 1) layernorm_bwd_warp_kernel(T* __restrict__ gx, float* __restrict__ partial, const T* __restrict__ gy,
                                                                const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ mean,
                                                                const float* __restrict__ rstd, int64_t rows, int cols) {
    constexpr int N = Vec16<T>::N;
    __shared__ float fold[8][32 * N];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int npk = cols / N;
    float wacc[MAXP][N], bacc[MAXP][N];
    Vec16<T> wv[MAXP];
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
#pragma unroll
        for (int j = 0; j < N; ++j) { wacc[i][j] = 0.f; bacc[i][j] = 0.f; }
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
        float mu[R], rs[R];
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int64_t row = row0 + q * stride;
            mu[q] = row < rows ? mean[row] : 0.f;
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
            if (row >= rows) continue;               // uniform across the warp
            float s1 = 0.f, s2 = 0.f;
#pragma unroll
            for (int i = 0; i < MAXP; ++i) {
                if (i * 32 + lane < npk) {
#pragma unroll
                    for (int j = 0; j < N; ++j) {
                        const float g0 = to_f32(gv[q][i].v[j]), xh = (to_f32(xv[q][i].v[j]) - mu[q]) * rs[q];
                        const float g = g0 * to_f32(wv[i].v[j]);
                        s1 += g;
                        s2 += g * xh;
                        wacc[i][j] += g0 * xh;
                        bacc[i][j] += g0;
                    }
                }
            }
            s1 = warp_sum(s1) * inv_cols;
            s2 = warp_sum(s2) * inv_cols;
            if (gx) {
#pragma unroll
                for (int i = 0; i < MAXP; ++i) {
                    const int pk = i * 32 + lane;
                    if (pk < npk) {
                        Vec16<T> o;
#pragma unroll
                        for (int j = 0; j < N; ++j) {
                            const float xh = (to_f32(xv[q][i].v[j]) - mu[q]) * rs[q];
                            o.v[j] = from_f32<T>(rs[q] * (to_f32(gv[q][i].v[j]) * to_f32(wv[i].v[j]) - s1 - xh * s2));
                        }
                        store16_stream(gx + row * cols + (int64_t)pk * N, o);
                    }
                }
            }
        }
    }
    if (!partial) return;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
#pragma unroll
        for (int i = 0; i < MAXP; ++i) {
            if (i * 32 * N >= cols) break;          // uniform
            __syncthreads();
#pragma unroll
            for (int j = 0; j < N; ++j) fold[warp][lane * N + j] = which ? bacc[i][j] : wacc[i][j];
            __syncthreads();
            for (int c = threadIdx.x; c < 32 * N; c += 256) {
                const int col = i * 32 * N + c;
                if (col < cols) {
                    float t = 0.f;
#pragma unroll
                    for (int k = 0; k < 8; ++k) t += fold[k][c];
                    partial[((int64_t)blockIdx.x * 2 + which) * cols + col] = t;
                }
            }
        }
    }
}

// out_w[c] = sum over parts of partial[part][0][c], out_b[c] = ... [1][c]: 32 columns x 32 part-lanes per CTA, every thread
// issues its loads together (a few hundred parts cost about one memory latency); blockIdx.y selects weight / bias.
template <typename T>
__global__ void __launch_bounds__(1024) ln_fold_kernel(T* __restrict__ out_w, T* __restrict__ out_b, const float* __restrict__ partial, int64_t nparts,
                                                      int64_t cols) {
    __shared__ float acc[32][33];
    const int which = blockIdx.y;
    T* out = which ? out_b : out_w;
    if (!out) return;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t c = (int64_t)blockIdx.x * 32 + tx;
    float s = 0.f;
    if (c < cols) {
        for (int64_t k = ty; k < nparts; k += 32 * 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = (k + 32 * u < nparts) ? partial[((k + 32 * u) * 2 + which) * cols + c] : 0.f;
#pragma unroll
            for (int u = 0; u < 8; ++u) s += v[u];
        }
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

// ---- GroupNorm backward ------------------------------------------------------------------------------------------------
// Input gradient: one CTA per (sample, group) row of `cols` = (C / G) * HW values, g = grad_y * gamma[channel].
template <typename T>
__global__ void __launch_bounds__(kNormThreads) groupnorm_bwd_input_kernel(T* __restrict__ gx, const T* __restrict__ gy, const T* __restrict__ x,
                                                                          const T* __restrict__ w, const float* __restrict__ mean,
                                                                          const float* __restrict__ rstd, int64_t cols, int64_t hw, int64_t groups,
                                                                          int64_t ch_per_group) {
    __shared__ float smem[33];
    const int64_t row = blockIdx.x;
    const T* xp = x + row * cols;
    const T* gp = gy + row * cols;
    const int64_t ch0 = (row % groups) * ch_per_group;
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float g = to_f32(gp[c]) * (w ? to_f32(w[ch0 + c / hw]) : 1.f);
        s1 += g;
        s2 += g * (to_f32(xp[c]) - mu) * rs;
    }
    s1 = block_sum256(s1, smem) / (float)cols;
    s2 = block_sum256(s2, smem) / (float)cols;
    T* op = gx + row * cols;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float g = to_f32(gp[c]) * (w ? to_f32(w[ch0 + c / hw]) : 1.f);
        op[c] = from_f32<T>(rs * (g - s1 - (to_f32(xp[c]) - mu) * rs * s2));
    }
}
// Parameter gradients: one CTA per channel, summed over the samples and the H*W positions in a fixed order.
template <typename T>
__global__ void __launch_bounds__(kNormThreads) groupnorm_bwd_params_kernel(T* __restrict__ gw, T* __restrict__ gb, const T* __restrict__ gy,
                                                                           const T* __restrict__ x, const float* __restrict__ mean,
                                                                           const float* __restrict__ rstd, int64_t n, int64_t channels, int64_t hw,
                                                                           int64_t groups) {
    __shared__ float smem[33];
    const int64_t ch = blockIdx.x;
    const int64_t g = ch / (channels / groups);
    float sw = 0.f, sb = 0.f;
    const int64_t total = n * hw;
    for (int64_t i = threadIdx.x; i < total; i += blockDim.x) {
        const int64_t smp = i / hw, pos = i - smp * hw;
        const int64_t off = (smp * channels + ch) * hw + pos;
        const float gyv = to_f32(gy[off]);
        sw += gyv * (to_f32(x[off]) - mean[smp * groups + g]) * rstd[smp * groups + g];
        sb += gyv;
    }
    sw = block_sum256(sw, smem);
    sb = block_sum256(sb, smem);
    if (threadIdx.x == 0) {
        if (gw) gw[ch] = from_f32<T>(sw);
        if (gb) gb[ch] = from_f32<T>(sb);
    }
}

// ---- cross-entropy ---------------------------------------------------------------------------------------------------
// G lanes per row (a power of two up to 32, chosen so that a row of c logits is about one 16-byte packet per lane), 32 / G
// rows per warp: row maximum, log-sum-exp (fp32, natural log), then the row's loss (lse - x[t]) * w[t]. Targets equal to
// ignore_index or outside [0, c) contribute nothing (src/shaders/ops/nllloss.slang:20-39). CTAs walk the row groups with a
// grid stride, so the number of partial sums does not grow with n.
// reduction 0: loss_rows[i] is the output; otherwise per-CTA partial sums of loss and weight go to part[cta][2].
template <int OPMAX> __device__ __forceinline__ float group_reduce(float v, int G) {
    for (int o = G >> 1; o > 0; o >>= 1) {
        const float u = __shfl_xor_sync(0xffffffffu, v, o);
        v = OPMAX ? fmaxf(v, u) : v + u;
    }
    return v;
}
template <typename T>
__global__ void __launch_bounds__(256) xent_fwd_kernel(T* __restrict__ loss_rows, float* __restrict__ lse_out, float* __restrict__ part,
                                                      const T* __restrict__ logits, const int64_t* __restrict__ target, const T* __restrict__ weight,
                                                      int64_t n, int64_t c, int64_t ignore_index, int G, int vec) {
    constexpr int N = Vec16<T>::N;
    __shared__ float sl[8], swt[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lg = lane & (G - 1), grp = lane / G, rpw = 32 / G;
    float loss_acc = 0.f, wt_acc = 0.f;
    const int64_t groups = (n + rpw - 1) / rpw;
    for (int64_t wg = (int64_t)blockIdx.x * 8 + warp; wg < groups; wg += (int64_t)gridDim.x * 8) {
        const int64_t row = wg * rpw + grp;
        const bool live_row = row < n;
        const T* p = logits + (live_row ? row : 0) * c;
        float m = -INFINITY;
        if (vec) {
            for (int64_t pk = lg; pk < c / N; pk += G) {
                const Vec16<T> v = load16(p + pk * N);
#pragma unroll
                for (int j = 0; j < N; ++j) m = fmaxf(m, to_f32(v.v[j]));
            }
        } else {
            for (int64_t j = lg; j < c; j += G) m = fmaxf(m, to_f32(p[j]));
        }
        m = group_reduce<1>(m, G);
        float s = 0.f;
        if (vec) {
            for (int64_t pk = lg; pk < c / N; pk += G) {
                const Vec16<T> v = load16(p + pk * N);
#pragma unroll
                for (int j = 0; j < N; ++j) s += expf(to_f32(v.v[j]) - m);
            }
        } else {
            for (int64_t j = lg; j < c; j += G) s += expf(to_f32(p[j]) - m);
        }
        s = group_reduce<0>(s, G);
        const float lse = m + logf(s);
        if (live_row && lg == 0) {
            const int64_t t = target[row];
            float loss = 0.f;
            if (lse_out) lse_out[row] = lse;
            if (t != ignore_index && t >= 0 && t < c) {
                const float wt = weight ? to_f32(weight[t]) : 1.f;
                loss = (lse - to_f32(p[t])) * wt;
                wt_acc += wt;
            }
            loss_acc += loss;
            if (loss_rows) loss_rows[row] = from_f32<T>(loss);
        }
    }
    if (part) {
        loss_acc = warp_sum(loss_acc);
        wt_acc = warp_sum(wt_acc);
        if (lane == 0) { sl[warp] = loss_acc; swt[warp] = wt_acc; }
        __syncthreads();
        if (threadIdx.x == 0) {
            float a = 0.f, b = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) { a += sl[k]; b += swt[k]; }
            part[(int64_t)blockIdx.x * 2] = a;
            part[(int64_t)blockIdx.x * 2 + 1] = b;
        }
    }
}
// Packet variants of the two kernels above for rows of up to P packets per lane: the row is read once into registers, and
// each warp keeps R row groups in flight (with a single 16-byte load per lane outstanding the kernels are bound by memory
// latency at about a fifth of the HBM rate).
template <typename T, int P, int R>
__global__ void __launch_bounds__(256) xent_fwd_vec_kernel(T* __restrict__ loss_rows, float* __restrict__ lse_out, float* __restrict__ part,
                                                          const T* __restrict__ logits, const int64_t* __restrict__ target,
                                                          const T* __restrict__ weight, int64_t n, int c, int64_t ignore_index, int G) {
    constexpr int N = Vec16<T>::N;
    __shared__ float sl[8], swt[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lg = lane & (G - 1), grp = lane / G, rpw = 32 / G;
    const int npk = c / N;
    float loss_acc = 0.f, wt_acc = 0.f;
    const int64_t groups = (n + rpw - 1) / rpw, stride = (int64_t)gridDim.x * 8;
    for (int64_t g0 = ((int64_t)blockIdx.x * 8 + warp) * R; g0 < groups; g0 += stride * R) {
        Vec16<T> xv[R][P];
        int64_t tg[R];
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int64_t row = (g0 + q) * rpw + grp;
            tg[q] = (row < n && lg == 0) ? target[row] : -1;
#pragma unroll
            for (int i = 0; i < P; ++i) {
                const int pk = i * G + lg;
                if (row < n && pk < npk) xv[q][i] = load16_stream(logits + row * c + (int64_t)pk * N);
            }
        }
#pragma unroll
        for (int q = 0; q < R; ++q) {
            if (g0 + q >= groups) continue;       // uniform across the warp
            const int64_t row = (g0 + q) * rpw + grp;
            const bool live_row = row < n;
            float m = -INFINITY;
#pragma unroll
            for (int i = 0; i < P; ++i) {
                if (live_row && i * G + lg < npk) {
#pragma unroll
                    for (int j = 0; j < N; ++j) m = fmaxf(m, to_f32(xv[q][i].v[j]));
                }
            }
            m = group_reduce<1>(m, G);
            const float m2 = m * kLog2e;
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < P; ++i) {
                if (live_row && i * G + lg < npk) {
#pragma unroll
                    for (int j = 0; j < N; ++j) sum += exp_shifted<T>(to_f32(xv[q][i].v[j]), m, m2);
                }
            }
            sum = group_reduce<0>(sum, G);
            const float lse = m + logf(sum);
            if (live_row && lg == 0) {
                const int64_t t = tg[q];
                float loss = 0.f;
                if (lse_out) lse_out[row] = lse;
                if (t != ignore_index && t >= 0 && t < c) {
                    const float wt = weight ? to_f32(weight[t]) : 1.f;
                    loss = (lse - to_f32(logits[row * c + t])) * wt;     // the row was just read: an L1 / L2 hit
                    wt_acc += wt;
                }
                loss_acc += loss;
                if (loss_rows) loss_rows[row] = from_f32<T>(loss);
            }
        }
    }
    if (part) {
        loss_acc = warp_sum(loss_acc);
        wt_acc = warp_sum(wt_acc);
        if (lane == 0) { sl[warp] = loss_acc; swt[warp] = wt_acc; }
        __syncthreads();
        if (threadIdx.x == 0) {
            float a = 0.f, b = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) { a += sl[k]; b += swt[k]; }
            part[(int64_t)blockIdx.x * 2] = a;
            part[(int64_t)blockIdx.x * 2 + 1] = b;
        }
    }
}
template <typename T, int P, int R>
__global__ void __launch_bounds__(256) xent_bwd_vec_kernel(T* __restrict__ gl, const T* __restrict__ gout, const T* __restrict__ logits,
                                                          const float* __restrict__ lse, const int64_t* __restrict__ target,
                                                          const T* __restrict__ weight, const T* __restrict__ total_weight, int64_t n, int c,
                                                          int reduction, int64_t ignore_index, int G) {
    constexpr int N = Vec16<T>::N;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lg = lane & (G - 1), grp = lane / G, rpw = 32 / G;
    const int npk = c / N;
    const int64_t groups = (n + rpw - 1) / rpw, stride = (int64_t)gridDim.x * 8;
    const float inv_total = reduction == 1 ? 1.0f / to_f32(total_weight[0]) : 1.0f;
    const float g_all = reduction == 0 ? 0.f : to_f32(gout[0]);
    for (int64_t g0 = ((int64_t)blockIdx.x * 8 + warp) * R; g0 < groups; g0 += stride * R) {
        Vec16<T> xv[R][P];
        int64_t tg[R];
        float ls[R], gr[R];
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int64_t row = (g0 + q) * rpw + grp;
            const bool in = row < n;
            tg[q] = in ? target[row] : -1;
            ls[q] = in ? lse[row] : 0.f;
            gr[q] = (in && reduction == 0) ? to_f32(gout[row]) : g_all;
#pragma unroll
            for (int i = 0; i < P; ++i) {
                const int pk = i * G + lg;
                if (in && pk < npk) xv[q][i] = load16_stream(logits + row * c + (int64_t)pk * N);
            }
        }
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int64_t row = (g0 + q) * rpw + grp;
            if (row >= n) continue;
            const int64_t t = tg[q];
            const bool live = t != ignore_index && t >= 0 && t < c;
            const float scale = live ? gr[q] * (weight ? to_f32(weight[t]) : 1.f) * inv_total : 0.f;
            const int tt = live ? (int)t : -1;
            const float l2 = ls[q] * kLog2e;
#pragma unroll
            for (int i = 0; i < P; ++i) {
                const int pk = i * G + lg;
                if (pk < npk) {
                    Vec16<T> o;
                    if (live) {
                        const int tp = tt - pk * N;      // position of the target inside this packet, if it is there
#pragma unroll
                        for (int j = 0; j < N; ++j) {
                            const float sm = exp_shifted<T>(to_f32(xv[q][i].v[j]), ls[q], l2);
                            o.v[j] = from_f32<T>((sm - (j == tp ? 1.f : 0.f)) * scale);
                        }
                    } else {
                        o.raw = make_uint4(0, 0, 0, 0);
                    }
                    store16_stream(gl + row * c + (int64_t)pk * N, o);
                }
            }
        }
    }
}

// loss = sum(part loss) [/ sum(part weight) for the mean]; total_weight also returned (nll_loss_forward's second output).
template <typename T>
__global__ void __launch_bounds__(256) xent_finalize_kernel(T* __restrict__ loss, T* __restrict__ total_weight, const float* __restrict__ part,
                                                           int64_t nparts, int mean) {
    __shared__ float smem[33];
    float a = 0.f, b = 0.f;
    for (int64_t k = threadIdx.x; k < nparts; k += blockDim.x) { a += part[k * 2]; b += part[k * 2 + 1]; }
    a = block_sum(a, smem);
    b = block_sum(b, smem);
    if (threadIdx.x == 0) {
        if (loss) loss[0] = from_f32<T>(mean ? a / b : a);
        if (total_weight) total_weight[0] = from_f32<T>(b);
    }
}
// grad_logits[i, j] = (softmax(x_i)[j] - [j == t_i]) * w[t_i] * g (/ total_weight for the mean); zero rows for ignored targets.
template <typename T>
__global__ void __launch_bounds__(256) xent_bwd_kernel(T* __restrict__ gl, const T* __restrict__ gout, const T* __restrict__ logits,
                                                      const float* __restrict__ lse, const int64_t* __restrict__ target,
                                                      const T* __restrict__ weight, const T* __restrict__ total_weight, int64_t n, int64_t c,
                                                      int reduction, int64_t ignore_index, int G, int vec) {
    constexpr int N = Vec16<T>::N;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lg = lane & (G - 1), grp = lane / G, rpw = 32 / G;
    const int64_t groups = (n + rpw - 1) / rpw;
    const float inv_total = reduction == 1 ? 1.0f / to_f32(total_weight[0]) : 1.0f;
    for (int64_t wg = (int64_t)blockIdx.x * 8 + warp; wg < groups; wg += (int64_t)gridDim.x * 8) {
        const int64_t row = wg * rpw + grp;
        if (row >= n) continue;
        const int64_t t = target[row];
        const bool live = t != ignore_index && t >= 0 && t < c;
        float scale = 0.f;
        if (live) scale = to_f32(gout[reduction == 0 ? row : 0]) * (weight ? to_f32(weight[t]) : 1.f) * inv_total;
        const float l = lse[row];
        const T* p = logits + row * c;
        T* o = gl + row * c;
        if (vec) {
            for (int64_t pk = lg; pk < c / N; pk += G) {
                Vec16<T> v = load16_stream(p + pk * N);
#pragma unroll
                for (int j = 0; j < N; ++j) {
                    const float sm = expf(to_f32(v.v[j]) - l);
                    v.v[j] = from_f32<T>(live ? (sm - ((pk * N + j) == t ? 1.f : 0.f)) * scale : 0.f);
                }
                store16_stream(o + pk * N, v);
            }
        } else {
            for (int64_t j = lg; j < c; j += G) {
                const float sm = expf(to_f32(p[j]) - l);
                o[j] = from_f32<T>(live ? (sm - (j == t ? 1.f : 0.f)) * scale : 0.f);
            }
        }
    }
}

// ---- scans ---------------------------------------------------------------------------------------------------------------
template <int OP> __device__ __forceinline__ float scan_identity() { return OP == TVK_SCAN_PROD ? 1.f : (OP == TVK_SCAN_LOGADDEXP ? -INFINITY : 0.f); }
template <int OP> __device__ __forceinline__ float scan_combine(float a, float b) {
    if constexpr (OP == TVK_SCAN_PROD) return a * b;
    else if constexpr (OP == TVK_SCAN_LOGADDEXP) {
        if (a != a || b != b) return a + b;
        const float m = fmaxf(a, b);
        if (m == -INFINITY) return -INFINITY;
        return m + log1pf(expf(-fabsf(a - b)));
    } else return a + b;
}
// inner == 1: one CTA per line, 256 threads x 8 consecutive elements per sweep, the running prefix carried across sweeps.
template <typename T, int OP>
__global__ void __launch_bounds__(256) scan_line_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t n) {
    __shared__ float warp_tot[8];
    __shared__ float carry_s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* p = in + (int64_t)blockIdx.x * n;
    T* q = out + (int64_t)blockIdx.x * n;
    float carry = scan_identity<OP>();
    for (int64_t base = 0; base < n; base += 256 * 8) {
        const int64_t i0 = base + (int64_t)threadIdx.x * 8;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (i0 + j < n) ? to_f32(p[i0 + j]) : scan_identity<OP>();
#pragma unroll
        for (int j = 1; j < 8; ++j) v[j] = scan_combine<OP>(v[j - 1], v[j]);
        // exclusive scan of the per-thread totals: within the warp, then across the eight warps
        float tot = v[7], incl = tot;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl = scan_combine<OP>(up, incl);
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        float before = carry;
        for (int w8 = 0; w8 < warp; ++w8) before = scan_combine<OP>(before, warp_tot[w8]);
        const float excl = __shfl_up_sync(0xffffffffu, incl, 1);
        if (lane > 0) before = scan_combine<OP>(before, excl);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (i0 + j < n) q[i0 + j] = from_f32<T>(scan_combine<OP>(before, v[j]));
        if (threadIdx.x == 255) carry_s = scan_combine<OP>(before, tot);
        __syncthreads();
        carry = carry_s;
        __syncthreads();
    }
}
// inner > 1: one thread per (outer, inner) column walking the scanned axis; neighbouring threads read neighbouring addresses.
template <typename T, int OP>
__global__ void __launch_bounds__(256) scan_strided_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t outer, int64_t n, int64_t inner) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= outer * inner) return;
    const int64_t o = idx / inner, i = idx - o * inner;
    const T* p = in + o * n * inner + i;
    T* q = out + o * n * inner + i;
    float acc = scan_identity<OP>();
    for (int64_t k = 0; k < n; ++k) {
        acc = scan_combine<OP>(acc, to_f32(p[k * inner]));
        q[k * inner] = from_f32<T>(acc);
    }
}
__global__ void __launch_bounds__(256) scan_i64_kernel(int64_t* __restrict__ out, const int64_t* __restrict__ in, int64_t outer, int64_t n, int64_t inner,
                                                      int prod) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= outer * inner) return;
    const int64_t o = idx / inner, i = idx - o * inner;
    const int64_t* p = in + o * n * inner + i;
    int64_t* q = out + o * n * inner + i;
    int64_t acc = prod ? 1 : 0;
    for (int64_t k = 0; k < n; ++k) {
        acc = prod ? acc * p[k * inner] : acc + p[k * inner];
        q[k * inner] = acc;
    }
}

static int xent_max_ctas() { return sm_count() * 8; }
// lanes per row (the smallest power of two that leaves at most four packets, or elements, per lane) and whether rows are
// walked in 16-byte packets
static void xent_shape(int dtype, const void* logits, int64_t c, int* G, int* vec) {
    const int N = (int)(16 / dtype_size(dtype));
    *vec = (c % N == 0) && aligned16(logits);
    const int64_t units = *vec ? c / N : c;
    int g = 1;
    while (g < 32 && (int64_t)g * 4 < units) g <<= 1;
    *G = g;
}
static int64_t xent_ctas(int64_t n, int G, int per_sm) {
    const int64_t groups = (n + (32 / G) - 1) / (32 / G);
    int64_t ctas = (groups + 7) / 8;
    if (ctas > (int64_t)sm_count() * per_sm) ctas = (int64_t)sm_count() * per_sm;
    return ctas < 1 ? 1 : ctas;
}

static int ln_bwd_ctas(int64_t rows) {
    int64_t c = (int64_t)sm_count() * 2;
    if (c > (rows + 7) / 8) c = (rows + 7) / 8;
    return (int)(c < 1 ? 1 : c);
}

}  // namespace tvk

using namespace tvk;

extern "C" {

int tvk_layernorm_forward(int dtype, void* y, float* mean, float* rstd, const void* x, const void* weight, const void* bias, int64_t rows,
                          int64_t cols, double eps, void* stream) {
    TVK_REQUIRE(rows >= 0 && cols >= 0, "tvk_layernorm_forward: negative extent");
    if (rows == 0 || cols == 0) return TVK_OK;
    TVK_REQUIRE(y && x, "tvk_layernorm_forward: null pointer");
    TVK_REQUIRE(rows <= 0x7fffffffLL, "tvk_layernorm_forward: too many rows");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t es = (int64_t)dtype_size(dtype);
    const int64_t npk = es ? cols * es / 16 : 0;
    const bool packets = es && (cols * es) % 16 == 0 && aligned16(x) && aligned16(y) && (!weight || aligned16(weight)) && (!bias || aligned16(bias));
    if (packets && npk <= 4 * 32) {
        // warp-per-row kernels: enough CTAs to fill the GPU a few times over, each warp walking rows with a grid stride
        int64_t ctas = (rows + 7) / 8;
        const int64_t cap = (int64_t)sm_count() * 8;
        if (ctas > cap) ctas = cap;
#define TVK_LN_FWD(MAXP_, R_)                                                                                                                       \
    TVK_DISPATCH_FLOAT(dtype, T, (layernorm_fwd_warp_kernel<T, MAXP_, R_><<<(unsigned)ctas, 256, 0, s>>>((T*)y, mean, rstd, (const T*)x, (const T*)weight, \
                                                                                                         (const T*)bias, rows, (int)cols, (float)eps)))
        if (npk <= 64) { TVK_LN_FWD(2, 4); }
        else { TVK_LN_FWD(4, 2); }
#undef TVK_LN_FWD
        return launch_status("layer norm forward");
    }
    TVK_DISPATCH_FLOAT(dtype, T, (rownorm_fwd_kernel<T><<<(unsigned)rows, kNormThreads, 0, s>>>((T*)y, mean, rstd, (const T*)x, (const T*)weight, (const T*)bias,
                                                                                                cols, (float)eps, 1, 0, 0)));
    return launch_status("layer norm forward");
}

int tvk_layernorm_backward_workspace_size(int64_t rows, int64_t cols, uint64_t* bytes) {
    if (!bytes) return set_error(TVK_ERR_INVALID, "tvk_layernorm_backward_workspace_size: null output");
    TVK_REQUIRE(rows >= 0 && cols >= 0, "tvk_layernorm_backward_workspace_size: negative extent");
    *bytes = (uint64_t)ln_bwd_ctas(rows) * 2 * (uint64_t)cols * sizeof(float);
    return TVK_OK;
}

int tvk_layernorm_backward(int dtype, void* grad_x, void* grad_w, void* grad_b, const void* grad_y, const void* x, const void* weight,
                           const float* mean, const float* rstd, int64_t rows, int64_t cols, void* workspace, uint64_t workspace_bytes,
                           void* stream) {
    TVK_REQUIRE(rows >= 0 && cols >= 0, "tvk_layernorm_backward: negative extent");
    if (cols == 0) return TVK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const bool params = grad_w || grad_b;
    if (rows == 0) {
        if (grad_w) TVK_CUDA_CHECK(cudaMemsetAsync(grad_w, 0, cols * dtype_size(dtype), s));
        if (grad_b) TVK_CUDA_CHECK(cudaMemsetAsync(grad_b, 0, cols * dtype_size(dtype), s));
        return TVK_OK;
    }
    TVK_REQUIRE(grad_y && x && mean && rstd, "tvk_layernorm_backward: null pointer");
    if (cols > 32 * (int64_t)kNormThreads)
        return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: layer_norm backward over %lld normalized elements (limit %d)", (long long)cols,
                         32 * kNormThreads);
    const int ctas = ln_bwd_ctas(rows);
    float* partial = nullptr;
    if (params) {
        const uint64_t need = (uint64_t)ctas * 2 * (uint64_t)cols * sizeof(float);
        TVK_REQUIRE(workspace && workspace_bytes >= need, "tvk_layernorm_backward: workspace of %llu bytes required, %llu given", (unsigned long long)need,
                    (unsigned long long)workspace_bytes);
        partial = (float*)workspace;
    }
    const int64_t es = (int64_t)dtype_size(dtype);
    const int64_t npk = cols * es / 16;
    const bool packets = (cols * es) % 16 == 0 && aligned16(x) && aligned16(grad_y) && (!grad_x || aligned16(grad_x)) && (!weight || aligned16(weight));
    if (packets && npk <= 4 * 32) {
#define TVK_LN_BWDW(MAXP_, R_)                                                                                                                       \
    TVK_DISPATCH_FLOAT(dtype, T, (layernorm_bwd_warp_kernel<T, MAXP_, R_><<<ctas, 256, 0, s>>>((T*)grad_x, partial, (const T*)grad_y, (const T*)x,   \
                                                                                               (const T*)weight, mean, rstd, rows, (int)cols)))
        if (npk <= 64) { TVK_LN_BWDW(2, 2); }
        else { TVK_LN_BWDW(4, 1); }
#undef TVK_LN_BWDW
        if (params) {
            const dim3 grid((unsigned)((cols + 31) / 32), 2);
            TVK_DISPATCH_FLOAT(dtype, T, (ln_fold_kernel<T><<<grid, 1024, 0, s>>>((T*)grad_w, (T*)grad_b, partial, ctas, cols)));
        }
        return launch_status("layer norm backward");
    }
    const int cpt = (int)((cols + kNormThreads - 1) / kNormThreads);
#define TVK_LN_BWD(CPT_)                                                                                                                             \
    TVK_DISPATCH_FLOAT(dtype, T, (layernorm_bwd_kernel<T, CPT_><<<ctas, kNormThreads, 0, s>>>((T*)grad_x, partial, (const T*)grad_y, (const T*)x,   \
                                                                                               (const T*)weight, mean, rstd, rows, cols)))
    if (cpt <= 2) { TVK_LN_BWD(2); }
    else if (cpt <= 4) { TVK_LN_BWD(4); }
    else if (cpt <= 8) { TVK_LN_BWD(8); }
    else if (cpt <= 16) { TVK_LN_BWD(16); }
    else { TVK_LN_BWD(32); }
#undef TVK_LN_BWD
    if (params) {
        const dim3 grid((unsigned)((cols + 31) / 32), 2);
        TVK_DISPATCH_FLOAT(dtype, T, (ln_fold_kernel<T><<<grid, 1024, 0, s>>>((T*)grad_w, (T*)grad_b, partial, ctas, cols)));
    }
    return launch_status("layer norm backward");
}

int tvk_groupnorm_forward(int dtype, void* y, float* mean, float* rstd, const void* x, const void* weight, const void* bias, int64_t n,
                          int64_t channels, int64_t hw, int64_t groups, double eps, void* stream) {
    TVK_REQUIRE(n >= 0 && channels >= 0 && hw >= 0 && groups > 0, "tvk_groupnorm_forward: bad extent");
    TVK_REQUIRE(channels % groups == 0, "tvk_groupnorm_forward: %lld channels do not divide into %lld groups", (long long)channels, (long long)groups);
    if (n == 0 || channels == 0 || hw == 0) return TVK_OK;
    TVK_REQUIRE(y && x, "tvk_groupnorm_forward: null pointer");
    const int64_t rows = n * groups, cpg = channels / groups;
    TVK_REQUIRE(rows <= 0x7fffffffLL, "tvk_groupnorm_forward: too many rows");
    cudaStream_t s = (cudaStream_t)stream;
    TVK_DISPATCH_FLOAT(dtype, T, (rownorm_fwd_kernel<T><<<(unsigned)rows, kNormThreads, 0, s>>>((T*)y, mean, rstd, (const T*)x, (const T*)weight, (const T*)bias,
                                                                                                cpg * hw, (float)eps, hw, groups, cpg)));
    return launch_status("group norm forward");
}

int tvk_groupnorm_backward(int dtype, void* grad_x, void* grad_w, void* grad_b, const void* grad_y, const void* x, const void* weight,
                           const float* mean, const float* rstd, int64_t n, int64_t channels, int64_t hw, int64_t groups, void* stream) {
    TVK_REQUIRE(n >= 0 && channels >= 0 && hw >= 0 && groups > 0 && channels % groups == 0, "tvk_groupnorm_backward: bad extent");
    cudaStream_t s = (cudaStream_t)stream;
    if (n == 0 || hw == 0 || channels == 0) {
        if (grad_w && channels) TVK_CUDA_CHECK(cudaMemsetAsync(grad_w, 0, channels * dtype_size(dtype), s));
        if (grad_b && channels) TVK_CUDA_CHECK(cudaMemsetAsync(grad_b, 0, channels * dtype_size(dtype), s));
        return TVK_OK;
    }
    TVK_REQUIRE(grad_y && x && mean && rstd, "tvk_groupnorm_backward: null pointer");
    const int64_t rows = n * groups, cpg = channels / groups;
    TVK_REQUIRE(rows <= 0x7fffffffLL && channels <= 0x7fffffffLL, "tvk_groupnorm_backward: too many rows");
    if (grad_x) {
        TVK_DISPATCH_FLOAT(dtype, T, (groupnorm_bwd_input_kernel<T><<<(unsigned)rows, kNormThreads, 0, s>>>((T*)grad_x, (const T*)grad_y, (const T*)x,
                                                                                                            (const T*)weight, mean, rstd, cpg * hw, hw, groups, cpg)));
    }
    if (grad_w || grad_b) {
        TVK_DISPATCH_FLOAT(dtype, T, (groupnorm_bwd_params_kernel<T><<<(unsigned)channels, kNormThreads, 0, s>>>((T*)grad_w, (T*)grad_b, (const T*)grad_y,
                                                                                                                 (const T*)x, mean, rstd, n, channels, hw, groups)));
    }
    return launch_status("group norm backward");
}

int tvk_cross_entropy_workspace_size(int64_t n, uint64_t* bytes) {
    if (!bytes) return set_error(TVK_ERR_INVALID, "tvk_cross_entropy_workspace_size: null output");
    TVK_REQUIRE(n >= 0, "tvk_cross_entropy_workspace_size: negative extent");
    *bytes = (uint64_t)xent_max_ctas() * 2 * sizeof(float);
    return TVK_OK;
}

int tvk_cross_entropy_forward(int dtype, void* loss, void* total_weight, float* lse, const void* logits, const int64_t* target, const void* weight,
                              int64_t n, int64_t c, int reduction, int64_t ignore_index, void* workspace, uint64_t workspace_bytes, void* stream) {
    TVK_REQUIRE(n >= 0 && c >= 0, "tvk_cross_entropy_forward: negative extent");
    TVK_REQUIRE(reduction >= 0 && reduction <= 2, "tvk_cross_entropy_forward: unknown reduction %d", reduction);
    TVK_REQUIRE(loss, "tvk_cross_entropy_forward: null output");
    cudaStream_t s = (cudaStream_t)stream;
    if (n > 0) TVK_REQUIRE(logits && target && c > 0, "tvk_cross_entropy_forward: null pointer or no classes");
    int G = 1, vec = 0;
    xent_shape(dtype, logits, c > 0 ? c : 1, &G, &vec);
    const int64_t ctas = xent_ctas(n, G, 8);      // the partial sums are sized for eight CTAs per SM
    float* part = nullptr;
    if (reduction != 0) {
        const uint64_t need = (uint64_t)ctas * 2 * sizeof(float);
        TVK_REQUIRE(n == 0 || (workspace && workspace_bytes >= need), "tvk_cross_entropy_forward: workspace of %llu bytes required, %llu given",
                    (unsigned long long)need, (unsigned long long)workspace_bytes);
        part = (float*)workspace;
    }
    const int64_t npk = vec ? c / (int64_t)(16 / dtype_size(dtype)) : 0;
    const int P = vec ? (int)((npk + G - 1) / G) : 0;
    if (n > 0 && vec && P <= 4 && c <= 0x7fffffffLL) {
#define TVK_XENT_FWD(P_, R_)                                                                                                                          \
    TVK_DISPATCH_FLOAT(dtype, T, (xent_fwd_vec_kernel<T, P_, R_><<<(unsigned)ctas, 256, 0, s>>>(reduction == 0 ? (T*)loss : nullptr, lse, part, (const T*)logits, \
                                                                                                target, (const T*)weight, n, (int)c, ignore_index, G)))
        if (P <= 1) { TVK_XENT_FWD(1, 4); } else if (P <= 2) { TVK_XENT_FWD(2, 2); } else { TVK_XENT_FWD(4, 1); }
#undef TVK_XENT_FWD
    } else if (n > 0) {
        TVK_DISPATCH_FLOAT(dtype, T, (xent_fwd_kernel<T><<<(unsigned)ctas, 256, 0, s>>>(reduction == 0 ? (T*)loss : nullptr, lse, part, (const T*)logits, target,
                                                                                        (const T*)weight, n, c, ignore_index, G, vec)));
    }
    if (reduction != 0) {
        TVK_DISPATCH_FLOAT(dtype, T, (xent_finalize_kernel<T><<<1, 256, 0, s>>>((T*)loss, (T*)total_weight, part, n > 0 ? ctas : 0, reduction == 1)));
    }
    return launch_status("cross entropy forward");
}

int tvk_cross_entropy_backward(int dtype, void* grad_logits, const void* grad_out, const void* logits, const float* lse, const int64_t* target,
                               const void* weight, const void* total_weight, int64_t n, int64_t c, int reduction, int64_t ignore_index,
                               void* stream) {
    TVK_REQUIRE(n >= 0 && c >= 0, "tvk_cross_entropy_backward: negative extent");
    TVK_REQUIRE(reduction >= 0 && reduction <= 2, "tvk_cross_entropy_backward: unknown reduction %d", reduction);
    if (n == 0 || c == 0) return TVK_OK;
    TVK_REQUIRE(grad_logits && grad_out && logits && lse && target, "tvk_cross_entropy_backward: null pointer");
    TVK_REQUIRE(reduction != 1 || total_weight, "tvk_cross_entropy_backward: the mean needs total_weight");
    int G = 1, vec = 0;
    xent_shape(dtype, logits, c, &G, &vec);
    if (vec && !aligned16(grad_logits)) vec = 0;
    const int64_t ctas = xent_ctas(n, G, 32);
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t npk = vec ? c / (int64_t)(16 / dtype_size(dtype)) : 0;
    const int P = vec ? (int)((npk + G - 1) / G) : 0;
    if (vec && P <= 4 && c <= 0x7fffffffLL) {
#define TVK_XENT_BWD(P_, R_)                                                                                                                          \
    TVK_DISPATCH_FLOAT(dtype, T, (xent_bwd_vec_kernel<T, P_, R_><<<(unsigned)ctas, 256, 0, s>>>((T*)grad_logits, (const T*)grad_out, (const T*)logits, lse, target, \
                                                                                                (const T*)weight, (const T*)total_weight, n, (int)c, reduction,     \
                                                                                                ignore_index, G)))
        if (P <= 1) { TVK_XENT_BWD(1, 4); } else if (P <= 2) { TVK_XENT_BWD(2, 2); } else { TVK_XENT_BWD(4, 1); }
#undef TVK_XENT_BWD
        return launch_status("cross entropy backward");
    }
    TVK_DISPATCH_FLOAT(dtype, T, (xent_bwd_kernel<T><<<(unsigned)ctas, 256, 0, s>>>((T*)grad_logits, (const T*)grad_out, (const T*)logits, lse, target,
                                                                                    (const T*)weight, (const T*)total_weight, n, c, reduction, ignore_index, G, vec)));
    return launch_status("cross entropy backward");
}

int tvk_scan(int op, int dtype, void* out, const void* in, int64_t outer, int64_t n, int64_t inner, void* stream) {
    TVK_REQUIRE(op >= TVK_SCAN_SUM && op <= TVK_SCAN_LOGADDEXP, "tvk_scan: unknown op %d", op);
    TVK_REQUIRE(outer >= 0 && n >= 0 && inner >= 0, "tvk_scan: negative extent");
    if (outer == 0 || n == 0 || inner == 0) return TVK_OK;
    TVK_REQUIRE(out && in, "tvk_scan: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t cols = outer * inner;
    if (dtype == TVK_I64) {
        TVK_REQUIRE(op != TVK_SCAN_LOGADDEXP, "tvk_scan: logcumsumexp of an integer tensor");
        TVK_REQUIRE((cols + 255) / 256 <= 0x7fffffffLL, "tvk_scan: too many lines");
        scan_i64_kernel<<<(unsigned)((cols + 255) / 256), 256, 0, s>>>((int64_t*)out, (const int64_t*)in, outer, n, inner, op == TVK_SCAN_PROD);
        return launch_status("scan");
    }
#define TVK_SCAN_LAUNCH(OP_)                                                                                                                          \
    if (inner == 1 && (n >= 512 || outer < 1024)) {                                                                                                   \
        TVK_REQUIRE(outer <= 0x7fffffffLL, "tvk_scan: too many lines");                                                                               \
        TVK_DISPATCH_FLOAT(dtype, T, (scan_line_kernel<T, OP_><<<(unsigned)outer, 256, 0, s>>>((T*)out, (const T*)in, n)));                           \
    } else {                                                                                                                                          \
        TVK_REQUIRE((cols + 255) / 256 <= 0x7fffffffLL, "tvk_scan: too many lines");                                                                  \
        TVK_DISPATCH_FLOAT(dtype, T, (scan_strided_kernel<T, OP_><<<(unsigned)((cols + 255) / 256), 256, 0, s>>>((T*)out, (const T*)in, outer, n, inner))); \
    }
    if (op == TVK_SCAN_SUM) { TVK_SCAN_LAUNCH(TVK_SCAN_SUM) }
    else if (op == TVK_SCAN_PROD) { TVK_SCAN_LAUNCH(TVK_SCAN_PROD) }
    else { TVK_SCAN_LAUNCH(TVK_SCAN_LOGADDEXP) }
#undef TVK_SCAN_LAUNCH
    return launch_status("scan");
}

}  // extern "C"
