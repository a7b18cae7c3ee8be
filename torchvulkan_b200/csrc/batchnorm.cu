// Training-mode batch normalisation over an [n, c, hw] (NCHW) view, forward and backward.
//
// Replaces batch_norm_shader / batch_norm_backward_shader (src/api/ops/norm.cpp:327-428) and
// batchForward / batchBackward (src/shaders/ops/norm.slang:72-191). The reference launches one
// 256-thread group per channel (grid = c <= 256 groups) that strides over n*hw with a div/mod per
// element; here every channel is split over enough CTAs to fill the GPU, each CTA walks whole
// contiguous hw-rows of its channel with 16-byte packets, and the per-channel statistics are
// folded from per-CTA partials. Statistics are fp32 (norm.slang uses T.Accum); variance is taken
// about a shift (the channel's first element) so one pass gives the stability of the reference's
// two passes; running_var is updated with the unbiased variance (norm.slang:99-113).
// Traffic: forward 2 reads + 1 write of x, backward 2 reads of (dy, x) + 1 write.
#include "common.cuh"

namespace tvk {

constexpr int kBnThreads = 256;
constexpr int kBnMaxSplits = 64;

static int bn_splits(int64_t n, int64_t c, int64_t hw) {
    // CTAs per channel: fill the GPU about four times, at least one image per CTA.
    int64_t want = ((int64_t)sm_count() * 4 + c - 1) / c;
    if (want > n) want = n;
    if (want > kBnMaxSplits) want = kBnMaxSplits;
    if (want < 1) want = 1;
    (void)hw;
    return (int)want;
}

// Iterates the elements of channel `ch` in images [n0, n1): calls f(offset, count_is_vector).
template <typename T, typename FVec, typename FScalar>
__device__ __forceinline__ void for_channel(const T* base, int64_t ch, int64_t c, int64_t hw, int64_t n0, int64_t n1, bool vec, FVec fv, FScalar fs) {
    constexpr int N = Vec16<T>::N;
    if (vec) {
        const int64_t ppr = hw / N;  // packets per row
        const int64_t total = (n1 - n0) * ppr;
        for (int64_t i = threadIdx.x; i < total; i += blockDim.x) {
            const int64_t img = n0 + i / ppr, pk = i - (i / ppr) * ppr;
            fv((img * c + ch) * hw + pk * N);
        }
    } else {
        const int64_t total = (n1 - n0) * hw;
        for (int64_t i = threadIdx.x; i < total; i += blockDim.x) {
            const int64_t img = n0 + i / hw, e = i - (i / hw) * hw;
            fs((img * c + ch) * hw + e);
        }
    }
    (void)base;
}

// partial[(ch * splits + split) * 2 + {0,1}] = sum(x - shift), sum((x - shift)^2)
template <typename T>
__global__ void __launch_bounds__(kBnThreads) bn_stats_kernel(float* __restrict__ partial, const T* __restrict__ x, int64_t n, int64_t c, int64_t hw,
                                                             int splits, int vec) {
    __shared__ float smem[33];
    constexpr int N = Vec16<T>::N;
    const int64_t ch = blockIdx.x;
    const int split = blockIdx.y;
    const int64_t per = (n + splits - 1) / splits;
    const int64_t n0 = split * per, n1 = (n0 + per) < n ? (n0 + per) : n;
    const float shift = to_f32(x[ch * hw]);
    float s1 = 0.f, s2 = 0.f;
    if (n0 < n1) {
        for_channel<T>(
            x, ch, c, hw, n0, n1, vec != 0,
            [&](int64_t off) {
                Vec16<T> v = load16(x + off);
#pragma unroll
                for (int j = 0; j < N; ++j) { const float d = to_f32(v.v[j]) - shift; s1 += d; s2 += d * d; }
            },
            [&](int64_t off) { const float d = to_f32(x[off]) - shift; s1 += d; s2 += d * d; });
    }
    s1 = block_sum(s1, smem);
    s2 = block_sum(s2, smem);
    if (threadIdx.x == 0) {
        partial[(ch * splits + split) * 2 + 0] = s1;
        partial[(ch * splits + split) * 2 + 1] = s2;
    }
}

__device__ __forceinline__ void store_stat(void* p, int dtype, int64_t i, float v) {
    if (dtype == TVK_F32) ((float*)p)[i] = v;
    else if (dtype == TVK_F16) ((__half*)p)[i] = __float2half_rn(v);
    else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ float load_stat(const void* p, int dtype, int64_t i) {
    if (dtype == TVK_F32) return ((const float*)p)[i];
    if (dtype == TVK_F16) return __half2float(((const __half*)p)[i]);
    return __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

template <typename T>
__global__ void __launch_bounds__(kBnThreads) bn_apply_kernel(T* __restrict__ y, float* __restrict__ save_mean, float* __restrict__ save_invstd,
                                                             const float* __restrict__ partial, const T* __restrict__ x, const T* __restrict__ weight,
                                                             const T* __restrict__ bias, int stat_dtype, void* running_mean, void* running_var,
                                                             int64_t n, int64_t c, int64_t hw, int splits, float momentum, float eps, int vec) {
    constexpr int N = Vec16<T>::N;
    const int64_t ch = blockIdx.x;
    const int split = blockIdx.y;
    // Every CTA of the channel folds the same partials in the same order.
    const float shift = to_f32(x[ch * hw]);
    double s1 = 0.0, s2 = 0.0;
    for (int k = 0; k < splits; ++k) {
        s1 += (double)partial[(ch * splits + k) * 2 + 0];
        s2 += (double)partial[(ch * splits + k) * 2 + 1];
    }
    const double cnt = (double)n * (double)hw;
    const double dmean = s1 / cnt;
    double var = s2 / cnt - dmean * dmean;
    if (var < 0.0) var = 0.0;
    const float mean = (float)((double)shift + dmean);
    const float invstd = rsqrtf((float)var + eps);
    if (split == 0 && threadIdx.x == 0) {
        save_mean[ch] = mean;
        save_invstd[ch] = invstd;
        if (running_mean) store_stat(running_mean, stat_dtype, ch, (1.f - momentum) * load_stat(running_mean, stat_dtype, ch) + momentum * mean);
        if (running_var) {
            const float unbiased = cnt > 1.0 ? (float)(var * cnt / (cnt - 1.0)) : (float)var;
            store_stat(running_var, stat_dtype, ch, (1.f - momentum) * load_stat(running_var, stat_dtype, ch) + momentum * unbiased);
        }
    }
    const float w = weight ? to_f32(weight[ch]) : 1.f;
    const float b = bias ? to_f32(bias[ch]) : 0.f;
    const float scale = w * invstd;
    const float offset = b - mean * scale;
    const int64_t per = (n + splits - 1) / splits;
    const int64_t n0 = split * per, n1 = (n0 + per) < n ? (n0 + per) : n;
    if (n0 >= n1) return;
    for_channel<T>(
        x, ch, c, hw, n0, n1, vec != 0,
        [&](int64_t off) {
            Vec16<T> v = load16(x + off);
#pragma unroll
            for (int j = 0; j < N; ++j) v.v[j] = from_f32<T>(to_f32(v.v[j]) * scale + offset);
            store16(y + off, v);
        },
        [&](int64_t off) { y[off] = from_f32<T>(to_f32(x[off]) * scale + offset); });
}

// partial[(ch * splits + split) * 2 + {0,1}] = sum(dy), sum(dy * (x - mean))
template <typename T>
__global__ void __launch_bounds__(kBnThreads) bn_bwd_stats_kernel(float* __restrict__ partial, const T* __restrict__ dy, const T* __restrict__ x,
                                                                 const float* __restrict__ save_mean, int64_t n, int64_t c, int64_t hw, int splits, int vec) {
    __shared__ float smem[33];
    constexpr int N = Vec16<T>::N;
    const int64_t ch = blockIdx.x;
    const int split = blockIdx.y;
    const int64_t per = (n + splits - 1) / splits;
    const int64_t n0 = split * per, n1 = (n0 + per) < n ? (n0 + per) : n;
    const float mean = save_mean[ch];
    float s1 = 0.f, s2 = 0.f;
    if (n0 < n1) {
        for_channel<T>(
            x, ch, c, hw, n0, n1, vec != 0,
            [&](int64_t off) {
                Vec16<T> vx = load16(x + off), vg = load16(dy + off);
#pragma unroll
                for (int j = 0; j < N; ++j) { const float g = to_f32(vg.v[j]); s1 += g; s2 += g * (to_f32(vx.v[j]) - mean); }
            },
            [&](int64_t off) { const float g = to_f32(dy[off]); s1 += g; s2 += g * (to_f32(x[off]) - mean); });
    }
    s1 = block_sum(s1, smem);
    s2 = block_sum(s2, smem);
    if (threadIdx.x == 0) {
        partial[(ch * splits + split) * 2 + 0] = s1;
        partial[(ch * splits + split) * 2 + 1] = s2;
    }
}

template <typename T>
__global__ void __launch_bounds__(kBnThreads) bn_bwd_apply_kernel(T* __restrict__ dx, T* __restrict__ dw, T* __restrict__ db, const float* __restrict__ partial,
                                                                 const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ weight,
                                                                 const float* __restrict__ save_mean, const float* __restrict__ save_invstd, int64_t n,
                                                                 int64_t c, int64_t hw, int splits, int vec) {
    constexpr int N = Vec16<T>::N;
    const int64_t ch = blockIdx.x;
    const int split = blockIdx.y;
    double s1 = 0.0, s2 = 0.0;
    for (int k = 0; k < splits; ++k) {
        s1 += (double)partial[(ch * splits + k) * 2 + 0];
        s2 += (double)partial[(ch * splits + k) * 2 + 1];
    }
    const float mean = save_mean[ch], invstd = save_invstd[ch];
    const float sum_dy = (float)s1, sum_dy_xmu = (float)s2;
    if (split == 0 && threadIdx.x == 0) {
        if (dw) dw[ch] = from_f32<T>(sum_dy_xmu * invstd);
        if (db) db[ch] = from_f32<T>(sum_dy);
    }
    if (!dx) return;
    const float cnt = (float)((double)n * (double)hw);
    const float w = weight ? to_f32(weight[ch]) : 1.f;
    const float k1 = sum_dy / cnt;
    const float k2 = sum_dy_xmu * invstd * invstd / cnt;
    const float scale = w * invstd;
    const int64_t per = (n + splits - 1) / splits;
    const int64_t n0 = split * per, n1 = (n0 + per) < n ? (n0 + per) : n;
    if (n0 >= n1) return;
    for_channel<T>(
        x, ch, c, hw, n0, n1, vec != 0,
        [&](int64_t off) {
            Vec16<T> vx = load16(x + off), vg = load16(dy + off);
#pragma unroll
            for (int j = 0; j < N; ++j) vg.v[j] = from_f32<T>((to_f32(vg.v[j]) - k1 - (to_f32(vx.v[j]) - mean) * k2) * scale);
            store16(dx + off, vg);
        },
        [&](int64_t off) { dx[off] = from_f32<T>((to_f32(dy[off]) - k1 - (to_f32(x[off]) - mean) * k2) * scale); });
}

// ---- channels-last: x is [rows = n*hw, c] with the channel contiguous ---------------------------------
// A thread owns one 16-byte packet of channels and walks rows; its per-channel sums stay in registers
// and the row lanes of a CTA fold through shared memory. Three launches per direction: column
// statistics -> per-channel constants -> elementwise apply.
constexpr int kClMaxSplits = 1024;
// Upper bound of the row splits for c channels, whatever the dtype and row count (sizes the workspace).
static int cl_splits_cap(int64_t c) {
    int64_t tiles = (c / 8 + kBnThreads - 1) / kBnThreads;
    if (tiles < 1) tiles = 1;
    const int64_t want = ((int64_t)sm_count() * 4 + tiles - 1) / tiles;
    return (int)(want > kClMaxSplits ? kClMaxSplits : want);
}

struct ClGeom {
    int ppr;        // packets per row
    int tpr;        // threads per row inside a CTA (= packets covered per CTA column tile)
    int lanes;      // row lanes per CTA
    int col_tiles;  // CTAs along the channel axis
    int splits;     // CTAs along the row axis
};
static ClGeom cl_geom(int64_t rows, int64_t c, int packet) {
    ClGeom g;
    g.ppr = (int)(c / packet);
    g.tpr = g.ppr < kBnThreads ? g.ppr : kBnThreads;
    g.lanes = kBnThreads / g.tpr;
    g.col_tiles = (g.ppr + g.tpr - 1) / g.tpr;
    // four CTAs of 256 threads per SM: with two, an SM had 32-64 KB of loads outstanding and the kernels ran at about half
    // of the HBM rate
    int64_t want = ((int64_t)sm_count() * 4 + g.col_tiles - 1) / g.col_tiles;
    const int64_t max_by_rows = (rows + g.lanes - 1) / g.lanes;
    if (want > max_by_rows) want = max_by_rows;
    if (want > kClMaxSplits) want = kClMaxSplits;
    g.splits = (int)(want < 1 ? 1 : want);
    return g;
}

// partial[(split * c + ch) * 2 + {0,1}]. MODE 0: sum(x - shift), sum((x - shift)^2), shift = x[0, ch].
// MODE 1: sum(dy), sum(dy * (x - mean[ch])).
template <typename T, int MODE>
__global__ void __launch_bounds__(kBnThreads) bn_cl_stats_kernel(float* __restrict__ partial, const T* __restrict__ x, const T* __restrict__ dy,
                                                                const float* __restrict__ mean, int64_t rows, int64_t c, ClGeom g) {
    constexpr int N = Vec16<T>::N;
    __shared__ float fold[kBnThreads][2 * N + 1];
    const int tcol = threadIdx.x % g.tpr, lane = threadIdx.x / g.tpr;
    const int pk = blockIdx.x * g.tpr + tcol;
    const bool active = lane < g.lanes && pk < g.ppr;
    float s1[N], s2[N], ref[N];
#pragma unroll
    for (int j = 0; j < N; ++j) { s1[j] = 0.f; s2[j] = 0.f; ref[j] = 0.f; }
    if (active) {
        if (MODE == 0) {
            const Vec16<T> v0 = load16(x + (int64_t)pk * N);
#pragma unroll
            for (int j = 0; j < N; ++j) ref[j] = to_f32(v0.v[j]);
        } else {
#pragma unroll
            for (int j = 0; j < N; ++j) ref[j] = mean[(int64_t)pk * N + j];
        }
        const int64_t per = (rows + g.splits - 1) / g.splits;
        const int64_t r0 = (int64_t)blockIdx.y * per, r1 = (r0 + per) < rows ? (r0 + per) : rows;
        constexpr int U = MODE == 0 ? 8 : 4;   // rows in flight per thread (16 bytes each, twice that with dy)
        auto accumulate = [&](const Vec16<T>& vx, const Vec16<T>& vg) {
            if (MODE == 0) {
#pragma unroll
                for (int j = 0; j < N; ++j) { const float d = to_f32(vx.v[j]) - ref[j]; s1[j] += d; s2[j] += d * d; }
            } else {
#pragma unroll
                for (int j = 0; j < N; ++j) { const float gg = to_f32(vg.v[j]); s1[j] += gg; s2[j] += gg * (to_f32(vx.v[j]) - ref[j]); }
            }
        };
        int64_t r = r0 + lane;
        for (; r + (int64_t)(U - 1) * g.lanes < r1; r += (int64_t)U * g.lanes) {
            Vec16<T> vx[U], vg[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t off = (r + (int64_t)u * g.lanes) * c + (int64_t)pk * N;
                vx[u] = load16_stream(x + off);
                if (MODE == 1) vg[u] = load16_stream(dy + off);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) accumulate(vx[u], vg[u]);
        }
        for (; r < r1; r += g.lanes) {
            const int64_t off = r * c + (int64_t)pk * N;
            Vec16<T> vx = load16_stream(x + off), vg;
            if (MODE == 1) vg = load16_stream(dy + off);
            accumulate(vx, vg);
        }
    }
#pragma unroll
    for (int j = 0; j < N; ++j) { fold[threadIdx.x][2 * j] = s1[j]; fold[threadIdx.x][2 * j + 1] = s2[j]; }
    __syncthreads();
    // every thread folds some (channel, statistic) outputs of the CTA over the row lanes
    const int outputs = g.tpr * 2 * N;
    for (int o = threadIdx.x; o < outputs; o += kBnThreads) {
        const int tc = o / (2 * N), k = o - tc * (2 * N);
        const int pko = blockIdx.x * g.tpr + tc;
        if (pko >= g.ppr) continue;
        float a = 0.f;
        for (int l = 0; l < g.lanes; ++l) a += fold[l * g.tpr + tc][k];
        const int64_t ch = (int64_t)pko * N + (k >> 1);
        partial[((int64_t)blockIdx.y * c + ch) * 2 + (k & 1)] = a;
    }
}

// Sum over the row splits of one channel's two statistics, by one warp. The loads of eight splits per lane are issued
// together (a dependent load-add chain costs a memory latency per step, and this kernel is nothing but that chain).
__device__ __forceinline__ void cl_fold_partials(const float* __restrict__ partial, int64_t ch, int64_t c, int splits, int ln, double& s1, double& s2) {
    constexpr int U = 8;
    int k = ln;
    for (; k + 32 * (U - 1) < splits; k += 32 * U) {
        float2 pr[U];
#pragma unroll
        for (int u = 0; u < U; ++u) pr[u] = *(const float2*)(partial + ((int64_t)(k + 32 * u) * c + ch) * 2);
#pragma unroll
        for (int u = 0; u < U; ++u) { s1 += (double)pr[u].x; s2 += (double)pr[u].y; }
    }
    float2 tail[U];
#pragma unroll
    for (int u = 0; u < U; ++u) tail[u] = (k + 32 * u < splits) ? *(const float2*)(partial + ((int64_t)(k + 32 * u) * c + ch) * 2) : make_float2(0.f, 0.f);
#pragma unroll
    for (int u = 0; u < U; ++u) { s1 += (double)tail[u].x; s2 += (double)tail[u].y; }
    s1 = warp_sum_f64(s1);
    s2 = warp_sum_f64(s2);
}

// Forward constants per channel: save_mean, save_invstd, running stats; coef[ch] = {scale, offset}.
template <typename T>
__global__ void bn_cl_fwd_finalize_kernel(float* __restrict__ coef, float* __restrict__ save_mean, float* __restrict__ save_invstd,
                                          const float* __restrict__ partial, const T* __restrict__ x, const T* __restrict__ weight,
                                          const T* __restrict__ bias, int stat_dtype, void* running_mean, void* running_var, int64_t rows, int64_t c,
                                          int splits, float momentum, float eps) {
    // one warp per channel: the lanes share the partials of the row splits
    const int64_t ch = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int ln = threadIdx.x & 31;
    if (ch >= c) return;
    double s1 = 0.0, s2 = 0.0;
    cl_fold_partials(partial, ch, c, splits, ln, s1, s2);
    if (ln != 0) return;
    const double cnt = (double)rows;
    const double dmean = s1 / cnt;
    double var = s2 / cnt - dmean * dmean;
    if (var < 0.0) var = 0.0;
    const float mean = (float)((double)to_f32(x[ch]) + dmean);
    const float invstd = rsqrtf((float)var + eps);
    save_mean[ch] = mean;
    save_invstd[ch] = invstd;
    if (running_mean) store_stat(running_mean, stat_dtype, ch, (1.f - momentum) * load_stat(running_mean, stat_dtype, ch) + momentum * mean);
    if (running_var) {
        const float unbiased = cnt > 1.0 ? (float)(var * cnt / (cnt - 1.0)) : (float)var;
        store_stat(running_var, stat_dtype, ch, (1.f - momentum) * load_stat(running_var, stat_dtype, ch) + momentum * unbiased);
    }
    const float scale = (weight ? to_f32(weight[ch]) : 1.f) * invstd;
    coef[2 * ch] = scale;
    coef[2 * ch + 1] = (bias ? to_f32(bias[ch]) : 0.f) - mean * scale;
}

// Backward constants: dw, db and coef[ch] = {scale, k1, k2, mean} with dx = (dy - k1 - (x - mean) * k2) * scale.
template <typename T>
__global__ void bn_cl_bwd_finalize_kernel(float* __restrict__ coef, T* __restrict__ dw, T* __restrict__ db, const float* __restrict__ partial,
                                          const T* __restrict__ weight, const float* __restrict__ save_mean, const float* __restrict__ save_invstd,
                                          int64_t rows, int64_t c, int splits) {
    const int64_t ch = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int ln = threadIdx.x & 31;
    if (ch >= c) return;
    double s1 = 0.0, s2 = 0.0;
    cl_fold_partials(partial, ch, c, splits, ln, s1, s2);
    if (ln != 0) return;
    const float mean = save_mean[ch], invstd = save_invstd[ch];
    const float sum_dy = (float)s1, sum_dy_xmu = (float)s2;
    if (dw) dw[ch] = from_f32<T>(sum_dy_xmu * invstd);
    if (db) db[ch] = from_f32<T>(sum_dy);
    const float cnt = (float)rows;
    coef[4 * ch + 0] = (weight ? to_f32(weight[ch]) : 1.f) * invstd;
    coef[4 * ch + 1] = sum_dy / cnt;
    coef[4 * ch + 2] = sum_dy_xmu * invstd * invstd / cnt;
    coef[4 * ch + 3] = mean;
}

// MODE 0: y = x * scale + offset. MODE 1: dx = (dy - k1 - (x - mean) * k2) * scale. Same thread layout as the
// statistics kernel: a thread keeps the constants of its 16-byte packet of channels in registers and walks rows.
template <typename T, int MODE>
__global__ void __launch_bounds__(kBnThreads) bn_cl_apply_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ dy,
                                                                const float* __restrict__ coef, int64_t rows, int64_t c, ClGeom g) {
    constexpr int N = Vec16<T>::N;
    constexpr int U = 4;
    const int tcol = threadIdx.x % g.tpr, lane = threadIdx.x / g.tpr;
    const int pk = blockIdx.x * g.tpr + tcol;
    if (lane >= g.lanes || pk >= g.ppr) return;
    float k0[N], k1[N], k2[N], k3[N];
#pragma unroll
    for (int j = 0; j < N; ++j) {
        const int64_t ch = (int64_t)pk * N + j;
        if (MODE == 0) {
            const float2 k = *(const float2*)(coef + 2 * ch);
            k0[j] = k.x; k1[j] = k.y; k2[j] = 0.f; k3[j] = 0.f;
        } else {
            const float4 k = *(const float4*)(coef + 4 * ch);
            k0[j] = k.x; k1[j] = k.y; k2[j] = k.z; k3[j] = k.w;
        }
    }
    auto apply = [&](Vec16<T>& vx, const Vec16<T>& vg) {
#pragma unroll
        for (int j = 0; j < N; ++j) {
            if (MODE == 0) vx.v[j] = from_f32<T>(to_f32(vx.v[j]) * k0[j] + k1[j]);
            else vx.v[j] = from_f32<T>((to_f32(vg.v[j]) - k1[j] - (to_f32(vx.v[j]) - k3[j]) * k2[j]) * k0[j]);
        }
    };
    const int64_t per = (rows + g.splits - 1) / g.splits;
    const int64_t r0 = (int64_t)blockIdx.y * per, r1 = (r0 + per) < rows ? (r0 + per) : rows;
    int64_t r = r0 + lane;
    for (; r + (int64_t)(U - 1) * g.lanes < r1; r += (int64_t)U * g.lanes) {
        Vec16<T> vx[U], vg[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t off = (r + (int64_t)u * g.lanes) * c + (int64_t)pk * N;
            vx[u] = load16_stream(x + off);
            if (MODE == 1) vg[u] = load16_stream(dy + off);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            apply(vx[u], vg[u]);
            store16_stream(out + (r + (int64_t)u * g.lanes) * c + (int64_t)pk * N, vx[u]);
        }
    }
    for (; r < r1; r += g.lanes) {
        const int64_t off = r * c + (int64_t)pk * N;
        Vec16<T> vx = load16_stream(x + off), vg;
        if (MODE == 1) vg = load16_stream(dy + off);
        apply(vx, vg);
        store16_stream(out + off, vx);
    }
}

// Evaluation mode: every element is scaled and shifted by its channel's constants (four small cached loads).
template <typename T>
__global__ void __launch_bounds__(256) bn_inference_kernel(T* __restrict__ y, const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                                                          int stat_dtype, const void* __restrict__ mean, const void* __restrict__ var, int64_t total,
                                                          int64_t c, int64_t hw, int channels_last, float eps) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t ch = channels_last ? i % c : (i / hw) % c;
        const float scale = rsqrtf(load_stat(var, stat_dtype, ch) + eps) * (w ? to_f32(w[ch]) : 1.f);
        const float shift = (b ? to_f32(b[ch]) : 0.f) - load_stat(mean, stat_dtype, ch) * scale;
        y[i] = from_f32<T>(to_f32(x[i]) * scale + shift);
    }
}

static uint64_t cl_workspace_bytes(int64_t c) { return ((uint64_t)c * cl_splits_cap(c) * 2 + (uint64_t)c * 4) * sizeof(float); }

}  // namespace tvk

using namespace tvk;

extern "C" {

int tvk_batchnorm_cl_workspace_size(int64_t rows, int64_t c, uint64_t* bytes) {
    if (!bytes) return set_error(TVK_ERR_INVALID, "tvk_batchnorm_cl_workspace_size: null output");
    TVK_REQUIRE(rows >= 0 && c >= 0, "tvk_batchnorm_cl_workspace_size: negative extent");
    *bytes = cl_workspace_bytes(c);
    return TVK_OK;
}

int tvk_batchnorm_inference(int dtype, void* y, const void* x, const void* weight, const void* bias, int stat_dtype, const void* running_mean,
                            const void* running_var, int64_t n, int64_t c, int64_t hw, int channels_last, double eps, void* stream) {
    TVK_REQUIRE(dtype == TVK_F32 || dtype == TVK_F16 || dtype == TVK_BF16, "torchvulkan [NOT IMPLEMENTED]: batch_norm for dtype %d", dtype);
    TVK_REQUIRE(n >= 0 && c >= 0 && hw >= 0, "tvk_batchnorm_inference: negative extent");
    const int64_t total = n * c * hw;
    if (total == 0) return TVK_OK;
    TVK_REQUIRE(y && x && running_mean && running_var, "tvk_batchnorm_inference: null pointer (evaluation mode needs the running statistics)");
    TVK_REQUIRE(is_float_dtype(stat_dtype), "tvk_batchnorm_inference: bad running-stat dtype %d", stat_dtype);
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)sm_count() * 16) blocks = (int64_t)sm_count() * 16;
    TVK_DISPATCH_FLOAT(dtype, T, (bn_inference_kernel<T><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((T*)y, (const T*)x, (const T*)weight, (const T*)bias, stat_dtype,
                                                                                                        running_mean, running_var, total, c, hw, channels_last, (float)eps)));
    return launch_status("batch_norm inference");
}

static int cl_check(int dtype, int64_t rows, int64_t c, const void* a, const void* b, const void* o, const char* who) {
    const size_t es = dtype_size(dtype);
    TVK_REQUIRE(dtype == TVK_F32 || dtype == TVK_F16 || dtype == TVK_BF16, "torchvulkan [NOT IMPLEMENTED]: %s for dtype %d", who, dtype);
    TVK_REQUIRE(rows > 0 && c > 0 && c <= 0x7fffffffLL, "%s: expected more than 0 values per channel", who);
    if (c % (int64_t)(16 / es) != 0 || !aligned16(a) || (b && !aligned16(b)) || (o && !aligned16(o)))
        return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: %s needs 16-byte aligned tensors and a channel count that is a multiple of %d", who,
                         (int)(16 / es));
    return TVK_OK;
}

int tvk_batchnorm_forward_cl(int dtype, void* y, float* save_mean, float* save_invstd, const void* x, const void* weight, const void* bias,
                             int stat_dtype, void* running_mean, void* running_var, int64_t rows, int64_t c, double momentum, double eps,
                             void* workspace, uint64_t workspace_bytes, void* stream) {
    if (c == 0) return TVK_OK;
    TVK_REQUIRE(y && x && save_mean && save_invstd, "tvk_batchnorm_forward_cl: null pointer");
    int rc = cl_check(dtype, rows, c, x, nullptr, y, "channels-last batch_norm");
    if (rc) return rc;
    TVK_REQUIRE(!(running_mean || running_var) || is_float_dtype(stat_dtype), "tvk_batchnorm_forward_cl: bad running-stat dtype %d", stat_dtype);
    TVK_REQUIRE(workspace && workspace_bytes >= cl_workspace_bytes(c), "tvk_batchnorm_forward_cl: workspace of %llu bytes required, %llu given",
                (unsigned long long)cl_workspace_bytes(c), (unsigned long long)workspace_bytes);
    cudaStream_t s = (cudaStream_t)stream;
    const int packet = (int)(16 / dtype_size(dtype));
    const ClGeom g = cl_geom(rows, c, packet);
    float* partial = (float*)workspace;
    float* coef = partial + (size_t)c * cl_splits_cap(c) * 2;
    dim3 grid((unsigned)g.col_tiles, (unsigned)g.splits);
    TVK_DISPATCH_FLOAT(dtype, T, (bn_cl_stats_kernel<T, 0><<<grid, kBnThreads, 0, s>>>(partial, (const T*)x, nullptr, nullptr, rows, c, g)));
    TVK_DISPATCH_FLOAT(dtype, T, (bn_cl_fwd_finalize_kernel<T><<<(unsigned)((c + 7) / 8), 256, 0, s>>>(coef, save_mean, save_invstd, partial, (const T*)x, (const T*)weight, (const T*)bias, stat_dtype, running_mean, running_var, rows, c, g.splits, (float)momentum, (float)eps)));
    TVK_DISPATCH_FLOAT(dtype, T, (bn_cl_apply_kernel<T, 0><<<grid, kBnThreads, 0, s>>>((T*)y, (const T*)x, nullptr, coef, rows, c, g)));
    return launch_status("channels-last batch_norm forward");
}

int tvk_batchnorm_backward_cl(int dtype, void* grad_x, void* grad_w, void* grad_b, const void* grad_y, const void* x, const void* weight,
                              const float* save_mean, const float* save_invstd, int64_t rows, int64_t c, void* workspace, uint64_t workspace_bytes,
                              void* stream) {
    if (c == 0 || rows == 0) return TVK_OK;
    TVK_REQUIRE(grad_y && x && save_mean && save_invstd, "tvk_batchnorm_backward_cl: null pointer");
    int rc = cl_check(dtype, rows, c, x, grad_y, grad_x, "channels-last batch_norm backward");
    if (rc) return rc;
    TVK_REQUIRE(workspace && workspace_bytes >= cl_workspace_bytes(c), "tvk_batchnorm_backward_cl: workspace of %llu bytes required, %llu given",
                (unsigned long long)cl_workspace_bytes(c), (unsigned long long)workspace_bytes);
    cudaStream_t s = (cudaStream_t)stream;
    const int packet = (int)(16 / dtype_size(dtype));
    const ClGeom g = cl_geom(rows, c, packet);
    float* partial = (float*)workspace;
    float* coef = partial + (size_t)c * cl_splits_cap(c) * 2;
    dim3 grid((unsigned)g.col_tiles, (unsigned)g.splits);
    TVK_DISPATCH_FLOAT(dtype, T, (bn_cl_stats_kernel<T, 1><<<grid, kBnThreads, 0, s>>>(partial, (const T*)x, (const T*)grad_y, save_mean, rows, c, g)));
    TVK_DISPATCH_FLOAT(dtype, T, (bn_cl_bwd_finalize_kernel<T><<<(unsigned)((c + 7) / 8), 256, 0, s>>>(coef, (T*)grad_w, (T*)grad_b, partial, (const T*)weight, save_mean, save_invstd, rows, c, g.splits)));
    if (grad_x) {
        TVK_DISPATCH_FLOAT(dtype, T, (bn_cl_apply_kernel<T, 1><<<grid, kBnThreads, 0, s>>>((T*)grad_x, (const T*)x, (const T*)grad_y, coef, rows, c, g)));
    }
    return launch_status("channels-last batch_norm backward");
}

int tvk_batchnorm_workspace_size(int64_t n, int64_t c, int64_t hw, uint64_t* bytes) {
    if (!bytes) return set_error(TVK_ERR_INVALID, "tvk_batchnorm_workspace_size: null output");
    TVK_REQUIRE(n >= 0 && c >= 0 && hw >= 0, "tvk_batchnorm_workspace_size: negative extent");
    *bytes = (uint64_t)c * kBnMaxSplits * 2 * sizeof(float);
    return TVK_OK;
}

int tvk_batchnorm_forward(int dtype, void* y, float* save_mean, float* save_invstd, const void* x, const void* weight, const void* bias,
                          int stat_dtype, void* running_mean, void* running_var, int64_t n, int64_t c, int64_t hw, double momentum,
                          double eps, void* workspace, uint64_t workspace_bytes, void* stream) {
    TVK_REQUIRE(n >= 0 && c >= 0 && hw >= 0, "tvk_batchnorm_forward: negative extent");
    if (c == 0) return TVK_OK;
    TVK_REQUIRE(n * hw > 0, "tvk_batchnorm_forward: expected more than 0 values per channel");
    TVK_REQUIRE(y && x && save_mean && save_invstd, "tvk_batchnorm_forward: null pointer");
    TVK_REQUIRE(c <= 0x7fffffffLL, "tvk_batchnorm_forward: too many channels");
    TVK_REQUIRE(!(running_mean || running_var) || is_float_dtype(stat_dtype), "tvk_batchnorm_forward: bad running-stat dtype %d", stat_dtype);
    uint64_t need = 0;
    tvk_batchnorm_workspace_size(n, c, hw, &need);
    TVK_REQUIRE(workspace && workspace_bytes >= need, "tvk_batchnorm_forward: workspace of %llu bytes required, %llu given",
                (unsigned long long)need, (unsigned long long)workspace_bytes);
    cudaStream_t s = (cudaStream_t)stream;
    const int splits = bn_splits(n, c, hw);
    const size_t es = dtype_size(dtype);
    const int N = es ? (int)(16 / es) : 1;
    const int vec = aligned16(x) && aligned16(y) && hw % N == 0;
    float* partial = (float*)workspace;
    dim3 grid((unsigned)c, (unsigned)splits);
    TVK_DISPATCH_FLOAT(dtype, T, (bn_stats_kernel<T><<<grid, kBnThreads, 0, s>>>(partial, (const T*)x, n, c, hw, splits, vec)));
    TVK_DISPATCH_FLOAT(dtype, T, (bn_apply_kernel<T><<<grid, kBnThreads, 0, s>>>((T*)y, save_mean, save_invstd, partial, (const T*)x, (const T*)weight, (const T*)bias, stat_dtype, running_mean, running_var, n, c, hw, splits, (float)momentum, (float)eps, vec)));
    return launch_status("batch_norm forward");
}

int tvk_batchnorm_backward(int dtype, void* grad_x, void* grad_w, void* grad_b, const void* grad_y, const void* x, const void* weight,
                           const float* save_mean, const float* save_invstd, int64_t n, int64_t c, int64_t hw, void* workspace,
                           uint64_t workspace_bytes, void* stream) {
    TVK_REQUIRE(n >= 0 && c >= 0 && hw >= 0, "tvk_batchnorm_backward: negative extent");
    if (c == 0 || n * hw == 0) return TVK_OK;
    TVK_REQUIRE(grad_y && x && save_mean && save_invstd, "tvk_batchnorm_backward: null pointer");
    uint64_t need = 0;
    tvk_batchnorm_workspace_size(n, c, hw, &need);
    TVK_REQUIRE(workspace && workspace_bytes >= need, "tvk_batchnorm_backward: workspace of %llu bytes required, %llu given",
                (unsigned long long)need, (unsigned long long)workspace_bytes);
    cudaStream_t s = (cudaStream_t)stream;
    const int splits = bn_splits(n, c, hw);
    const size_t es = dtype_size(dtype);
    const int N = es ? (int)(16 / es) : 1;
    const int vec = aligned16(x) && aligned16(grad_y) && (!grad_x || aligned16(grad_x)) && hw % N == 0;
    float* partial = (float*)workspace;
    dim3 grid((unsigned)c, (unsigned)splits);
    TVK_DISPATCH_FLOAT(dtype, T, (bn_bwd_stats_kernel<T><<<grid, kBnThreads, 0, s>>>(partial, (const T*)grad_y, (const T*)x, save_mean, n, c, hw, splits, vec)));
    TVK_DISPATCH_FLOAT(dtype, T, (bn_bwd_apply_kernel<T><<<grid, kBnThreads, 0, s>>>((T*)grad_x, (T*)grad_w, (T*)grad_b, partial, (const T*)grad_y, (const T*)x, (const T*)weight, save_mean, save_invstd, n, c, hw, splits, vec)));
    return launch_status("batch_norm backward");
}

}  // extern "C"
