// Dense contraction: C[b] = act(alpha * A[b] @ B[b] + beta * bias[b]).
//
// Replaces dispatch_matmul_coop_shader / dispatch_matmul_simd_shader
// (src/api/ops/matmul.cpp:250-329, 373-582) and the matmul_coop / matmul_simd shaders
// (src/shaders/ops/matmul_coop.slang:158-223, 364-415; src/shaders/helpers/gemm_simd.slang:101-281).
//
// Tensor-core path (sm_100a): a persistent, warp-specialised kernel.
//   warp 0      TMA producer: cp.async.bulk.tensor tiles of A and B into a ring of
//               128-byte-swizzled shared-memory stages, completion on mbarriers
//   warp 1      MMA issuer: one lane issues tcgen05.mma (M=128, N=BN, K=32 bytes per step)
//               with the fp32 accumulator in tensor memory (two accumulators, so the epilogue
//               of tile i overlaps the main loop of tile i+1); tcgen05.commit frees stages
//   warps 2-5   epilogue: tcgen05.ld the accumulator, alpha/beta*bias/ReLU/GELU, convert, store
// Row- and column-major operands are both consumed in place (K-major or MN-major shared
// memory descriptors), as the reference does with its *_TRANSPOSED specialisations
// (matmul_coop.slang:62-114). fp32 runs as 3xTF32: operands are split into tf32 hi/lo parts
// in a workspace and the main loop makes three passes (hi*hi + lo*hi + hi*lo) into the same
// fp32 accumulator. Every mbarrier wait is bounded; a wait that runs out raises the device
// status word and the CTA leaves through the normal teardown (TMEM is freed).
//
// CUDA-core path: a 64x64x16 register-tiled kernel with arbitrary strides and optional
// split-K, for operands TMA cannot address (row pitch not a multiple of 16 bytes) and for
// shapes with a very small M or N.
#include "common.cuh"
#include "gemm_tc.cuh"

#include <cuda.h>

#include <mutex>

namespace tvk {

// =====================================================================================
// CUDA-core kernel
// =====================================================================================
namespace simt {

constexpr int TM = 64, TN = 64, TK = 16;

struct Params {
    int64_t m, n, k;
    int64_t a_rs, a_cs, a_bs, b_rs, b_cs, b_bs;
    int64_t c_rs, c_bs;
    int64_t bias_rs, bias_cs, bias_bs;
    float alpha, beta;
    int act;
    int splits;          // > 1: fp32 partials [batch][split][m][n] go to `partial`
    int64_t k_chunk;     // k range per split (multiple of TK)
    // split-K epilogue only: the activation-gradient operand of tvk_gemm_desc (C's shape and type, row pitch aux_rs)
    const void* aux;
    int64_t aux_rs;
    int aux_op;
    void* c2;            // second output (C's strides): C gets the value before the activation, c2 the activated one
};


__device__ __forceinline__ float apply_act(float v, int act) { return tc::act_apply(v, act); }

template <typename T>
__global__ void __launch_bounds__(256) gemm_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C, const T* __restrict__ bias,
                                                  float* __restrict__ partial, Params p, int64_t batch0) {
    __shared__ float As[TK][TM + 4];
    __shared__ float Bs[TK][TN + 4];
    const int64_t bz = batch0 + blockIdx.z / p.splits;
    const int split = blockIdx.z % p.splits;
    const int64_t m0 = (int64_t)blockIdx.y * TM, n0 = (int64_t)blockIdx.x * TN;
    const T* Ab = A + bz * p.a_bs;
    const T* Bb = B + bz * p.b_bs;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4x4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    const int64_t k_begin = (int64_t)split * p.k_chunk;
    int64_t k_end = k_begin + p.k_chunk;
    if (k_end > p.k) k_end = p.k;
    // Loader mapping: pick the thread->element order that walks the contiguous direction of
    // each operand so the loads coalesce for both row- and column-major inputs.
    const bool a_k_fast = p.a_cs == 1;
    const bool b_n_fast = p.b_cs == 1;
    for (int64_t k0 = k_begin; k0 < k_end; k0 += TK) {
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int e = threadIdx.x + it * 256;  // 0..1023
            int mi, ki;
            if (a_k_fast) { ki = e & 15; mi = e >> 4; } else { mi = e & 63; ki = e >> 6; }
            const int64_t gm = m0 + mi, gk = k0 + ki;
            As[ki][mi] = (gm < p.m && gk < k_end) ? to_f32(Ab[gm * p.a_rs + gk * p.a_cs]) : 0.f;
            int ni, kj;
            if (b_n_fast) { ni = e & 63; kj = e >> 6; } else { kj = e & 15; ni = e >> 4; }
            const int64_t gn = n0 + ni, gk2 = k0 + kj;
            Bs[kj][ni] = (gn < p.n && gk2 < k_end) ? to_f32(Bb[gk2 * p.b_rs + gn * p.b_cs]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t gm = m0 + ty * 4 + i;
        if (gm >= p.m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t gn = n0 + tx * 4 + j;
            if (gn >= p.n) continue;
            if (p.splits > 1) {
                partial[(((bz - batch0) * p.splits + split) * p.m + gm) * p.n + gn] = acc[i][j];
            } else {
                float v = p.alpha * acc[i][j];
                if (bias) v += p.beta * to_f32(bias[bz * p.bias_bs + gm * p.bias_rs + gn * p.bias_cs]);
                C[bz * p.c_bs + gm * p.c_rs + gn] = from_f32<T>(apply_act(v, p.act));
            }
        }
    }
}

template <typename T>
__global__ void splitk_epilogue_kernel(const float* __restrict__ partial, T* __restrict__ C, const T* __restrict__ bias, Params p, int64_t batch0,
                                       int64_t nbatch) {
    const int64_t total = nbatch * p.m * p.n;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = idx / (p.m * p.n), r = idx - b * p.m * p.n;
        const int64_t gm = r / p.n, gn = r - gm * p.n;
        float s = 0.f;
        for (int sp = 0; sp < p.splits; ++sp) s += partial[((b * p.splits + sp) * p.m + gm) * p.n + gn];
        const int64_t bz = batch0 + b;
        float v = p.alpha * s;
        if (bias) v += p.beta * to_f32(bias[bz * p.bias_bs + gm * p.bias_rs + gn * p.bias_cs]);
        C[bz * p.c_bs + gm * p.c_rs + gn] = from_f32<T>(apply_act(v, p.act));
    }
}

// The same for one batch and n a multiple of four: a thread owns four neighbouring outputs, reads the partials as
// float4 (all splits' loads independent of each other) and divides once per four outputs.
template <typename T>
__global__ void __launch_bounds__(256) splitk_epilogue_vec_kernel(const float* __restrict__ partial, T* __restrict__ C, const T* __restrict__ bias, Params p) {
    const int64_t n4 = p.n >> 2, total = p.m * n4, plane = p.m * p.n;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t gm = idx / n4, gn = (idx - gm * n4) << 2;
        const float* src = partial + gm * p.n + gn;
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        int sp = 0;
        for (; sp + 4 <= p.splits; sp += 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = *(const float4*)(src + (int64_t)(sp + u) * plane);
#pragma unroll
            for (int u = 0; u < 4; ++u) { s.x += v[u].x; s.y += v[u].y; s.z += v[u].z; s.w += v[u].w; }
        }
        for (; sp < p.splits; ++sp) {
            const float4 v = *(const float4*)(src + (int64_t)sp * plane);
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        float o[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float v = p.alpha * o[e];
            if (bias) v += p.beta * to_f32(bias[gm * p.bias_rs + (gn + e) * p.bias_cs]);
            if (p.aux_op) v = tc::aux_apply(v, to_f32(((const T*)p.aux)[gm * p.aux_rs + gn + e]), p.aux_op);
            if (p.c2) {
                C[gm * p.c_rs + gn + e] = from_f32<T>(v);
                ((T*)p.c2)[gm * p.c_rs + gn + e] = from_f32<T>(apply_act(v, p.act));
            } else {
                C[gm * p.c_rs + gn + e] = from_f32<T>(apply_act(v, p.act));
            }
        }
    }
}

// ---- skinny shapes (a classifier head and its weight gradient: n or m of about ten) --------------------
// Neither fits a 64x64 (let alone 128xBN) tile; both are bandwidth problems over one large operand.

// n <= 16, A rows and B columns both contiguous along k (C = A @ W^T with W [n, k]): a 256-thread CTA owns two output
// rows, its threads split k in 16-byte packets (each W packet is used for both rows), and the 2 x n dot products
// are folded through warp shuffles and shared memory. W stays in L1/L2.
constexpr int kSkinnyNRows = 2;
template <typename T>
__global__ void __launch_bounds__(256) skinny_n_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C, const T* __restrict__ bias,
                                                      Params p) {
    constexpr int N = Vec16<T>::N;
    constexpr int R = kSkinnyNRows;
    __shared__ float fold[8][R * 16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row0 = (int64_t)blockIdx.x * R;
    const int64_t bz = blockIdx.y;
    const T* b = B + bz * p.b_bs;
    const T* a[R];
#pragma unroll
    for (int r = 0; r < R; ++r) a[r] = A + bz * p.a_bs + (row0 + r < p.m ? row0 + r : row0) * p.a_rs;
    float acc[R][16];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[r][j] = 0.f;
    const int64_t packets = p.k / N;
    const int iters = (int)((packets + 255) / 256);
    // independent iterations, unrolled so that the loads of several of them are in flight together
#pragma unroll 4
    for (int it = 0; it < iters; ++it) {
        const int64_t q = (int64_t)it * 256 + threadIdx.x;
        if (q >= packets) break;
        float fa[R][N];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const Vec16<T> va = load16_stream(a[r] + q * N);
#pragma unroll
            for (int e = 0; e < N; ++e) fa[r][e] = to_f32(va.v[e]);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if (j < p.n) {
                const Vec16<T> vb = load16(b + j * p.b_cs + q * N);
#pragma unroll
                for (int e = 0; e < N; ++e) {
                    const float fb = to_f32(vb.v[e]);
#pragma unroll
                    for (int r = 0; r < R; ++r) acc[r][j] = fmaf(fa[r][e], fb, acc[r][j]);
                }
            }
        }
    }
    for (int64_t kk = packets * N + threadIdx.x; kk < p.k; kk += 256) {      // k not a multiple of the packet
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (j < p.n) {
                const float fb = to_f32(b[j * p.b_cs + kk]);
#pragma unroll
                for (int r = 0; r < R; ++r) acc[r][j] = fmaf(to_f32(a[r][kk]), fb, acc[r][j]);
            }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float t = warp_sum(acc[r][j]);
            if (lane == 0) fold[warp][r * 16 + j] = t;
        }
    __syncthreads();
    if (threadIdx.x < R * 16) {
        const int r = threadIdx.x >> 4, j = threadIdx.x & 15;
        const int64_t row = row0 + r;
        if (row < p.m && j < p.n) {
            float t = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) t += fold[w][threadIdx.x];
            float v = p.alpha * t;
            if (bias) v += p.beta * to_f32(bias[bz * p.bias_bs + row * p.bias_rs + j * p.bias_cs]);
            C[bz * p.c_bs + row * p.c_rs + j] = from_f32<T>(apply_act(v, p.act));
        }
    }
}

// m <= 16, B rows contiguous along n: a thread owns one 16-byte packet of columns and all m rows of it; the k range
// is cut into slices over blockIdx.y and each slice writes an fp32 partial [slice][m][n] (splitk_epilogue_kernel sums).
constexpr int kSkinnyMSlice = 32;
template <typename T>
__global__ void __launch_bounds__(128) skinny_m_kernel(const T* __restrict__ A, const T* __restrict__ B, float* __restrict__ partial, Params p) {
    constexpr int N = Vec16<T>::N;
    __shared__ float as[kSkinnyMSlice][16];
    const int64_t col = ((int64_t)blockIdx.x * 128 + threadIdx.x) * N;
    const int64_t k0 = (int64_t)blockIdx.y * kSkinnyMSlice;
    const int64_t kn = (p.k - k0) < kSkinnyMSlice ? (p.k - k0) : kSkinnyMSlice;
    for (int e = threadIdx.x; e < kSkinnyMSlice * 16; e += 128) {
        const int kk = e >> 4, mi = e & 15;
        as[kk][mi] = (kk < kn && mi < p.m) ? to_f32(A[mi * p.a_rs + (k0 + kk) * p.a_cs]) : 0.f;
    }
    __syncthreads();
    if (col >= p.n) return;
    float acc[16][N];
#pragma unroll
    for (int i = 0; i < 16; ++i)
#pragma unroll
        for (int e = 0; e < N; ++e) acc[i][e] = 0.f;
    const bool full = col + N <= p.n;
    for (int kk = 0; kk < kn; ++kk) {
        float fb[N];
        if (full) {
            const Vec16<T> vb = load16_stream(B + (k0 + kk) * p.b_rs + col);
#pragma unroll
            for (int e = 0; e < N; ++e) fb[e] = to_f32(vb.v[e]);
        } else {
#pragma unroll
            for (int e = 0; e < N; ++e) fb[e] = (col + e < p.n) ? to_f32(B[(k0 + kk) * p.b_rs + col + e]) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float fa = as[kk][i];
#pragma unroll
            for (int e = 0; e < N; ++e) acc[i][e] = fmaf(fa, fb[e], acc[i][e]);
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        if (i < p.m) {
            float* dst = partial + ((int64_t)blockIdx.y * p.m + i) * p.n + col;
#pragma unroll
            for (int e = 0; e < N; ++e)
                if (col + e < p.n) dst[e] = acc[i][e];
        }
    }
}

// dst[r][c] = src(r, c) for c < cols, 0 for cols <= c < pitch: a small operand whose rows TMA cannot address (row pitch
// not a multiple of 16 bytes, or the wrong index contiguous) is copied once into a K-major buffer that it can.
template <typename T>
__global__ void repack_kernel(T* __restrict__ dst, const T* __restrict__ src, int64_t rows, int64_t cols, int64_t pitch, int64_t src_rs, int64_t src_cs) {
    const int64_t total = rows * pitch;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / pitch, c = i - r * pitch;
        dst[i] = c < cols ? src[r * src_rs + c * src_cs] : from_f32<T>(0.f);
    }
}

static int plan_splits(int64_t batch, int64_t m, int64_t n, int64_t k, int64_t* k_chunk) {
    const int64_t tiles = batch * ((m + TM - 1) / TM) * ((n + TN - 1) / TN);
    const int64_t sms = sm_count();
    int64_t splits = 1;
    if (tiles < sms && k >= 512) {
        splits = (2 * sms + tiles - 1) / tiles;
        const int64_t max_splits = k / 128;
        if (splits > max_splits) splits = max_splits;
        if (splits > 64) splits = 64;
        if (splits < 1) splits = 1;
    }
    int64_t chunk = (k + splits - 1) / splits;
    chunk = (chunk + TK - 1) / TK * TK;
    if (chunk < TK) chunk = TK;
    splits = (k + chunk - 1) / chunk;
    if (splits < 1) splits = 1;
    *k_chunk = chunk;
    return (int)splits;
}

// k <= 16, B rows contiguous along n (the input gradient of a classifier head: dY [m, 10] @ W [10, n]; a rank-k update):
// there is no contraction to speak of, the product is bound by writing C (and reading aux). A thread owns one 16-byte
// packet of columns for kSmallKRows rows: it walks the k rows of B once (each packet of B is used for all its rows), the
// m x k factors of A sit in shared memory and are read as broadcasts. alpha, bias, the activation and the
// activation-gradient operand (aux) are applied in registers: C = act((alpha * A @ B + beta * bias) * act'(aux)).
constexpr int kSmallKRows = 4, kSmallKMax = 16;
template <typename T>
__global__ void __launch_bounds__(256) small_k_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C, const T* __restrict__ bias, Params p) {
    constexpr int N = Vec16<T>::N;
    constexpr int R = kSmallKRows;
    __shared__ float As[R][kSmallKMax];
    const int64_t row0 = (int64_t)blockIdx.y * R;
    const int64_t col = ((int64_t)blockIdx.x * 256 + threadIdx.x) * N;
    const bool live = col < p.n;
    // every load this thread needs is issued before anything waits on one: the k packets of B, then the aux packets
    Vec16<T> vb[kSmallKMax], aux[R];
#pragma unroll
    for (int kk = 0; kk < kSmallKMax; ++kk)
        if (live && kk < p.k) vb[kk] = load16(B + kk * p.b_rs + col);
    if (p.aux_op && live) {
#pragma unroll
        for (int r = 0; r < R; ++r)
            if (row0 + r < p.m) aux[r] = load16_stream((const T*)p.aux + (row0 + r) * p.aux_rs + col);
    }
    if (threadIdx.x < R * kSmallKMax) {
        const int r = threadIdx.x / kSmallKMax, kk = threadIdx.x % kSmallKMax;
        As[r][kk] = (row0 + r < p.m && kk < p.k) ? to_f32(A[(row0 + r) * p.a_rs + kk * p.a_cs]) : 0.f;
    }
    __syncthreads();
    if (!live) return;
    float acc[R][N];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int e = 0; e < N; ++e) acc[r][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < kSmallKMax; ++kk) {
        if (kk < p.k) {
#pragma unroll
            for (int e = 0; e < N; ++e) {
                const float fb = to_f32(vb[kk].v[e]);
#pragma unroll
                for (int r = 0; r < R; ++r) acc[r][e] = fmaf(As[r][kk], fb, acc[r][e]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int64_t row = row0 + r;
        if (row < p.m) {
            Vec16<T> out;
#pragma unroll
            for (int e = 0; e < N; ++e) {
                float v = p.alpha * acc[r][e];
                if (bias) v += p.beta * to_f32(bias[row * p.bias_rs + (col + e) * p.bias_cs]);
                if (p.aux_op) v = tc::aux_apply(v, to_f32(aux[r].v[e]), p.aux_op);
                out.v[e] = from_f32<T>(apply_act(v, p.act));
            }
            store16(C + row * p.c_rs + col, out);
        }
    }
}

}  // namespace simt

// =====================================================================================
// tcgen05 kernel
// =====================================================================================
namespace tc {



// 3xTF32 operand split: hi = round-to-nearest tf32 of x, lo = x - hi (exact in fp32). The copies
// are always written K-major ([rows][k], pitch ld) whatever the source layout: element (r, k) of
// the source is at r * src_rs + k * src_ks. A source whose rows are the contiguous direction is
// transposed through shared memory so both sides stay coalesced. The tf32 MMA then only ever
// sees K-major operands (an MN-major tf32 tile would need the 32-byte-base swizzle variant).
// grid (k tiles, row tiles, batch), block (32, 8).
__global__ void __launch_bounds__(256) split_tf32_kernel(float* __restrict__ hi, float* __restrict__ lo, const float* __restrict__ src,
                                                        int64_t rows, int64_t k, int64_t src_rs, int64_t src_ks, int64_t src_bs,
                                                        int64_t ld) {
    __shared__ float tile[32][33];
    const int64_t b = blockIdx.z;
    src += b * src_bs;
    hi += b * rows * ld;
    lo += b * rows * ld;
    const int64_t k0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
    const bool transpose = src_ks != 1;
    if (transpose) {
        for (int j = threadIdx.y; j < 32; j += 8) {
            const int64_t kk = k0 + j, r = r0 + threadIdx.x;
            tile[j][threadIdx.x] = (kk < k && r < rows) ? src[r * src_rs + kk * src_ks] : 0.f;
        }
        __syncthreads();
    }
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int64_t r = r0 + j, kk = k0 + threadIdx.x;
        if (r >= rows || kk >= k) continue;
        const float x = transpose ? tile[threadIdx.x][j] : src[r * src_rs + kk];
        uint32_t h;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
        const float hf = __uint_as_float(h);
        hi[r * ld + kk] = hf;
        lo[r * ld + kk] = x - hf;
    }
}

// ---- host side ---------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
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

struct Operand {
    const void* ptr;
    int64_t rows, cols;     // logical: A is m x k, B is k x n
    int64_t rs, cs, bs;
    bool mn_major;          // the M (for A) / N (for B) index is the contiguous one
};

// A operand view for TMA: `inner` contiguous extent, `outer` extent with pitch, batch.
static int encode_operand(CUtensorMap* map, int dtype, const void* ptr, int64_t inner, int64_t outer, int64_t pitch_elems,
                          int64_t batch, int64_t batch_stride_elems, int box_inner, int box_outer) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return set_error(TVK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    // A training step issues the same few contractions over and over: keep the encoded
    // descriptors in a small per-thread direct-mapped cache keyed by everything that defines them.
    struct Key {
        const void* ptr;
        int64_t inner, outer, pitch, batch, bstride;
        int box_inner, box_outer, dtype;
        bool operator==(const Key& o) const {
            return ptr == o.ptr && inner == o.inner && outer == o.outer && pitch == o.pitch && batch == o.batch && bstride == o.bstride &&
                   box_inner == o.box_inner && box_outer == o.box_outer && dtype == o.dtype;
        }
    };
    struct Entry {
        Key key;
        CUtensorMap map;
        bool valid;
    };
    constexpr int kCacheSize = 128;
    thread_local Entry cache[kCacheSize] = {};
    const Key key = {ptr, inner, outer, pitch_elems, batch, batch_stride_elems, box_inner, box_outer, dtype};
    uint64_t h = (uint64_t)(uintptr_t)ptr * 0x9E3779B97F4A7C15ull;
    h ^= (uint64_t)inner * 0xC2B2AE3D27D4EB4Full + (uint64_t)outer * 0x165667B19E3779F9ull + (uint64_t)box_outer * 31 + (uint64_t)box_inner;
    Entry& slot = cache[(h >> 32) % kCacheSize];
    if (slot.valid && slot.key == key) {
        *map = slot.map;
        return TVK_OK;
    }
    const int es = (int)dtype_size(dtype);
    CUtensorMapDataType dt = dtype == TVK_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                             : dtype == TVK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                             : dtype == TVK_U8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8          // float8 operands travel as bytes
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)(batch > 0 ? batch : 1)};
    cuuint64_t bstride = (cuuint64_t)batch_stride_elems * es;
    if (batch <= 1 || bstride == 0) {
        dims[2] = 1;
        bstride = (cuuint64_t)outer * (cuuint64_t)pitch_elems * es;
    }
    cuuint64_t strides[2] = {(cuuint64_t)pitch_elems * es, bstride};
    cuuint32_t box[3] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, dt, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return set_error(TVK_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d (inner %lld outer %lld pitch %lld batch %lld)", (int)r,
                         (long long)inner, (long long)outer, (long long)pitch_elems, (long long)batch);
    slot.key = key;
    slot.map = *map;
    slot.valid = true;
    return TVK_OK;
}

// Can TMA address this operand in place?
static bool tma_ok(const void* ptr, int64_t rows, int64_t cols, int64_t rs, int64_t cs, int64_t bs, int64_t batch, int es) {
    if (((uintptr_t)ptr & 15) != 0) return false;
    const int64_t q = 16 / es;
    int64_t pitch;
    if (cs == 1 && rs % q == 0 && rs >= cols) pitch = rs;
    else if (rs == 1 && cs % q == 0 && cs >= rows) pitch = cs;
    else return false;
    if (pitch * es >= (int64_t)1 << 40) return false;
    if (batch > 1 && bs != 0 && (bs % q != 0 || bs < 0)) return false;
    if (rs < 0 || cs < 0) return false;
    return true;
}

// min_bn: an MN-major B tile is made of whole 128-byte rows of N, so BN cannot be narrower
// than one such row (64 two-byte or 32 four-byte elements).
static int pick_bn(int64_t batch, int64_t m, int64_t n, int min_bn, int max_bn, int mt = 1) {
    const int64_t sms = sm_count();
    const int64_t tiles_m = (m + mt * BM - 1) / (mt * BM);
    // Tuning override (the counterpart of pinning an entry in the reference's autotune cache).
    static const int forced = [] {
        const char* e = getenv("TORCHVULKAN_GEMM_BN");
        const int v = e ? atoi(e) : 0;
        return (v == 32 || v == 64 || v == 128 || v == 256) ? v : 0;
    }();
    if (forced >= min_bn && forced <= max_bn) return forced;
    const int cand[4] = {256, 128, 64, 32};
    const double eff[4] = {1.0, 0.92, 0.75, 0.5};
    int best = 128;
    double best_score = -1;
    for (int i = 0; i < 4; ++i) {
        const int bn = cand[i];
        if (bn < min_bn || bn > max_bn) continue;
        if (bn > min_bn && bn > 32 && n <= bn / 2) continue;  // would be mostly padding
        const int64_t tiles = batch * tiles_m * ((n + bn - 1) / bn);
        const int64_t waves = (tiles + sms - 1) / sms;
        const double util = (double)tiles / (double)(waves * sms);
        const double pad = (double)n / (double)(((n + bn - 1) / bn) * bn);
        const double score = util * eff[i] * pad;
        if (score > best_score) { best_score = score; best = bn; }
    }
    return best;
}

// Block shape for the half types by a small cost model, fitted to measurements on this GPU: a CTA has about 190 KB of
// operand stages in flight and a loaded fill latency of about 2.3 us, i.e. it can pull ~85 GB/s, so a k-block (64 values
// of K) costs max(fill of its (128*MT + BN) operand rows, its MMAs); blocks run in waves over the SMs; the epilogue of a
// block is exposed only when there is a single accumulator set. (4096^3: 1 x 256 blocks 155 us, 2 x 256 blocks 104 us;
// 256 x 8192 x 8192: 1 x 128 blocks 50 us, 2 x 256 blocks 90 us - both as the model orders them.)
static void pick_block(int64_t batch, int64_t m, int64_t n, int64_t k, int min_bn, int max_bn, int min_mt, int max_mt, int* mt_out, int* bn_out) {
    const double sms = (double)sm_count();
    const double kblocks = (double)((k + 63) / 64);
    double best = 1e300;
    *mt_out = min_mt;
    *bn_out = min_bn > 128 ? min_bn : 128;
    for (int mt = min_mt; mt <= max_mt; ++mt) {
        for (int bn = 256; bn >= 32; bn >>= 1) {
            if (bn < min_bn || bn > max_bn) continue;
            if (bn > min_bn && bn > 32 && n <= bn / 2) continue;   // would be mostly padding
            const double tiles = (double)batch * (double)((m + mt * BM - 1) / (mt * BM)) * (double)((n + bn - 1) / bn);
            const double waves = ceil(tiles / sms);
            const double fill_us = (double)(BM * mt + bn) * 128.0 / 85.0e3;
            const double mma_us = 0.38 * mt * (bn > 128 ? bn : 128) / 256.0;
            const double epi_us = 1.2 * mt * bn / 256.0;
            const bool one_acc_set = 2 * mt * bn > 512;
            const double main_us = kblocks * (fill_us > mma_us ? fill_us : mma_us);
            const double block_us = one_acc_set ? main_us + epi_us : (main_us > epi_us ? main_us : epi_us);
            const double t = waves * block_us + (one_acc_set ? 0.0 : epi_us);
            if (t < best * 0.98) { best = t; *mt_out = mt; *bn_out = bn; }
        }
    }
}

}  // namespace tc

// =====================================================================================
// dispatch
// =====================================================================================
// Tuning overrides set through tvk_debug_gemm_tuning (0 / -1 = the library's own choice). They stand where the
// reference pins an entry of its autotune cache (src/vulkan/autotuner.cpp:123-178): a sweep sets them, measures, and
// the winners become the rules of pick_block / tc_splitk_plan below.
struct GemmTuning {
    int bn = 0, mt = 0, splits = 0, group_m = 0, debug = 0;
};
static GemmTuning g_tune;
static thread_local int t_block_bn = 0, t_block_mt = 0;      // block shape for the launch that run_tc_splitk issues (0 = the cost model's)

static bool fused_epilogue(const tvk_gemm_desc* d) { return d->c2 != nullptr || d->aux_op != TVK_AUX_NONE; }

static int validate(const tvk_gemm_desc* d) {
    if (!d) return set_error(TVK_ERR_INVALID, "tvk_gemm: null descriptor");
    TVK_REQUIRE(d->dtype == TVK_F32 || d->dtype == TVK_F16 || d->dtype == TVK_BF16,
                "torchvulkan [NOT IMPLEMENTED]: matmul of dtype %d", d->dtype);
    TVK_REQUIRE(d->batch >= 0 && d->m >= 0 && d->n >= 0 && d->k >= 0, "tvk_gemm: negative extent");
    TVK_REQUIRE(d->activation >= TVK_ACT_NONE && d->activation <= TVK_ACT_GELU, "tvk_gemm: unknown activation %d", d->activation);
    if (d->batch == 0 || d->m == 0 || d->n == 0) return TVK_OK;
    TVK_REQUIRE(d->c, "tvk_gemm: null output");
    TVK_REQUIRE(d->k == 0 || (d->a && d->b), "tvk_gemm: null operand");
    TVK_REQUIRE(d->c_rs >= d->n, "tvk_gemm: output row pitch %lld smaller than n %lld", (long long)d->c_rs, (long long)d->n);
    TVK_REQUIRE(d->n_peer_c >= 0 && d->n_peer_c <= 7, "tvk_gemm: n_peer_c %d outside [0, 7]", d->n_peer_c);
    for (int q = 0; q < d->n_peer_c; ++q) TVK_REQUIRE(d->peer_c[q], "tvk_gemm: peer_c[%d] is null", q);
    TVK_REQUIRE(d->aux_op >= TVK_AUX_NONE && d->aux_op <= TVK_AUX_RELU_BACKWARD, "tvk_gemm: unknown aux_op %d", d->aux_op);
    TVK_REQUIRE(d->aux_op == TVK_AUX_NONE || d->aux, "tvk_gemm: aux_op %d without an aux operand", d->aux_op);
    if (fused_epilogue(d)) {
        if (d->dtype == TVK_F32 || d->c_f32 || d->n_peer_c > 0)
            return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: fused epilogue (c2 / aux) with fp32 data or peer copies");
        TVK_REQUIRE(d->aux_op == TVK_AUX_NONE || d->aux_rs >= d->n, "tvk_gemm: aux row pitch %lld smaller than n %lld", (long long)d->aux_rs, (long long)d->n);
    }
    return TVK_OK;
}

static bool tc_eligible(const tvk_gemm_desc* d) {
    if (d->k == 0) return false;
    const int es = (int)dtype_size(d->dtype);
    if (d->dtype == TVK_F32) {
        // fp32 operands are re-laid out by the hi/lo split, so any non-negative strides work
        if (d->a_rs < 0 || d->a_cs < 0 || d->a_bs < 0 || d->b_rs < 0 || d->b_cs < 0 || d->b_bs < 0) return false;
    } else {
        if (!tc::tma_ok(d->a, d->m, d->k, d->a_rs, d->a_cs, d->a_bs, d->batch, es)) return false;
        if (!tc::tma_ok(d->b, d->k, d->n, d->b_rs, d->b_cs, d->b_bs, d->batch, es)) return false;
    }
    if (d->m > (int64_t)0x7fffffff || d->n > (int64_t)0x7fffffff || d->k > (int64_t)0x7fffffff) return false;
    return true;
}

static uint64_t align256(uint64_t v) { return (v + 255) / 256 * 256; }

// A skinny product over one large operand (a classifier head: m x 10 x k, its input gradient m x n x 10 and its weight
// gradient 10 x n x k) is a streaming problem that the TMA pipeline handles better than CUDA-core loops even though most
// of the 128-row MMA is padding, provided the launch has enough blocks: k long enough to split, or n wide enough.
static bool skinny_tc_worthwhile(const tvk_gemm_desc* d) {
    if (d->batch != 1 || d->dtype == TVK_F32) return false;
    if ((double)d->m * (double)d->n * (double)d->k < 2.0e6) return false;
    if (d->n < 32) return d->m >= 128 && d->k >= 2048 && d->k % 64 == 0;      // split-K fills the GPU
    if (d->m < 32) return d->n >= 2048;                                        // 64-wide tiles along n do
    return true;
}

// Operands TMA cannot address in place but that are small enough to copy: which of them to repack so that the launch can
// take the tensor-core path, and the workspace that takes. Both false: no repacking (not needed, or not worth it).
struct Repack {
    bool a = false, b = false;
    int64_t kp = 0;                 // padded k (row pitch of the copies)
    uint64_t a_bytes = 0, b_bytes = 0;
};
static Repack plan_repack(const tvk_gemm_desc* d) {
    Repack r;
    if (d->dtype == TVK_F32 || d->batch != 1 || d->k == 0 || d->force_path == 2 || d->c_f32 || d->n_peer_c > 0) return r;
    if (d->m > (int64_t)0x7fffffff || d->n > (int64_t)0x7fffffff || d->k > (int64_t)0x7fffffff) return r;
    if (!skinny_tc_worthwhile(d) || (d->m >= 32 && d->n >= 32 && d->k >= 32)) return r;      // only the skinny cases
    const int es = (int)dtype_size(d->dtype);
    const bool a_ok = tc::tma_ok(d->a, d->m, d->k, d->a_rs, d->a_cs, 0, 1, es), b_ok = tc::tma_ok(d->b, d->k, d->n, d->b_rs, d->b_cs, 0, 1, es);
    if (a_ok && b_ok) return r;
    const int64_t limit = 1 << 20;      // elements: the copy must stay negligible next to the large operand
    if ((!a_ok && d->m * d->k > limit) || (!b_ok && d->n * d->k > limit)) return r;
    if (d->a_rs < 0 || d->a_cs < 0 || d->b_rs < 0 || d->b_cs < 0) return r;
    r.kp = (d->k + 7) / 8 * 8;
    r.a = !a_ok; r.b = !b_ok;
    r.a_bytes = r.a ? align256((uint64_t)d->m * r.kp * es) : 0;
    r.b_bytes = r.b ? align256((uint64_t)d->n * r.kp * es) : 0;
    return r;
}

static bool small_k_ok(const tvk_gemm_desc* d);

static int choose_path(const tvk_gemm_desc* d) {
    if (small_k_ok(d)) return 2;                                          // output-bound: a CUDA-core kernel that also takes aux
    if (d->c_f32 && d->dtype != TVK_F32) return tc_eligible(d) ? 1 : 0;   // mixed output exists on the tensor-core path only
    if (d->n_peer_c > 0) return tc_eligible(d) ? 1 : 0;                   // so do the pushed peer copies
    if (fused_epilogue(d)) {                                              // the fused epilogues exist on the tensor-core path only
        if (d->dtype == TVK_F32) return 0;
        if (tc_eligible(d)) return 1;
        const Repack r = plan_repack(d);
        return (r.a || r.b) ? 1 : 0;
    }
    if (d->force_path == 2) return 2;
    const bool ok = tc_eligible(d);
    if (d->force_path == 1) return ok ? 1 : 0;
    if (!ok) {
        const Repack r = plan_repack(d);
        return (r.a || r.b) ? 1 : 2;
    }
    if ((double)d->m * (double)d->n * (double)d->k * (double)d->batch < 2.0e6) return 2;
    // Very skinny outputs leave the 128-row MMA mostly idle: only where the launch still fills the GPU
    if ((d->m < 32 || d->n < 32) && !skinny_tc_worthwhile(d)) return 2;
    return 1;
}

// the small-k kernel: k of at most 16, one batch, B and C (and aux) rows contiguous and addressable in 16-byte packets
static bool small_k_ok(const tvk_gemm_desc* d) {
    const int64_t es = (int64_t)dtype_size(d->dtype), N = 16 / es;
    if (d->k < 1 || d->k > simt::kSmallKMax || d->batch != 1 || d->n < 512 || d->n % N != 0 || d->m < 1) return false;
    if (d->c2 || d->c_f32 || d->n_peer_c > 0 || d->force_path == 1) return false;
    if (d->b_cs != 1 || !aligned16(d->b) || (d->b_rs * es) % 16 != 0 || !aligned16(d->c) || (d->c_rs * es) % 16 != 0) return false;
    if (d->aux_op != TVK_AUX_NONE && (!d->aux || !aligned16(d->aux) || (d->aux_rs * es) % 16 != 0)) return false;
    return (d->m + simt::kSmallKRows - 1) / simt::kSmallKRows <= 65535;
}
static int run_small_k(const tvk_gemm_desc* d, cudaStream_t s) {
    simt::Params p = {};
    p.m = d->m; p.n = d->n; p.k = d->k;
    p.a_rs = d->a_rs; p.a_cs = d->a_cs; p.b_rs = d->b_rs; p.b_cs = d->b_cs;
    p.c_rs = d->c_rs;
    p.bias_rs = d->bias_rs; p.bias_cs = d->bias_cs;
    p.alpha = d->alpha; p.beta = d->beta; p.act = d->activation;
    p.aux = d->aux_op ? d->aux : nullptr; p.aux_rs = d->aux_rs; p.aux_op = d->aux_op;
    const int64_t N = 16 / (int64_t)dtype_size(d->dtype);
    dim3 grid((unsigned)((d->n / N + 255) / 256), (unsigned)((d->m + simt::kSmallKRows - 1) / simt::kSmallKRows));
    TVK_DISPATCH_FLOAT(d->dtype, T, (simt::small_k_kernel<T><<<grid, 256, 0, s>>>((const T*)d->a, (const T*)d->b, (T*)d->c, (const T*)d->bias, p)));
    return launch_status("small-k gemm");
}

static bool skinny_n_ok(const tvk_gemm_desc* d) {
    const int64_t es = (int64_t)dtype_size(d->dtype);
    return d->n >= 1 && d->n <= 16 && d->k >= 64 && d->a_cs == 1 && d->b_rs == 1 && d->batch <= 65535 && aligned16(d->a) && aligned16(d->b) &&
           (d->a_rs * es) % 16 == 0 && (d->b_cs * es) % 16 == 0 && (d->a_bs * es) % 16 == 0 && (d->b_bs * es) % 16 == 0;
}
static bool skinny_m_ok(const tvk_gemm_desc* d) {
    const int64_t es = (int64_t)dtype_size(d->dtype);
    return d->m >= 1 && d->m <= 16 && d->n >= 512 && d->batch == 1 && d->b_cs == 1 && aligned16(d->b) && (d->b_rs * es) % 16 == 0 &&
           (d->k + simt::kSkinnyMSlice - 1) / simt::kSkinnyMSlice <= 65535;
}
static uint64_t skinny_m_workspace(const tvk_gemm_desc* d) {
    return (uint64_t)((d->k + simt::kSkinnyMSlice - 1) / simt::kSkinnyMSlice) * d->m * d->n * sizeof(float);
}

static int run_simt(const tvk_gemm_desc* d, void* ws, uint64_t ws_bytes, cudaStream_t s) {
    simt::Params p = {};
    p.m = d->m; p.n = d->n; p.k = d->k;
    p.a_rs = d->a_rs; p.a_cs = d->a_cs; p.a_bs = d->a_bs;
    p.b_rs = d->b_rs; p.b_cs = d->b_cs; p.b_bs = d->b_bs;
    p.c_rs = d->c_rs; p.c_bs = d->c_bs;
    p.bias_rs = d->bias_rs; p.bias_cs = d->bias_cs; p.bias_bs = d->bias_bs;
    p.alpha = d->alpha; p.beta = d->beta; p.act = d->activation;
    if (fused_epilogue(d)) return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: fused epilogue (c2 / aux) on the CUDA-core path");
    if (skinny_n_ok(d)) {
        dim3 grid((unsigned)((d->m + simt::kSkinnyNRows - 1) / simt::kSkinnyNRows), (unsigned)d->batch);
        TVK_DISPATCH_FLOAT(d->dtype, T, (simt::skinny_n_kernel<T><<<grid, 256, 0, s>>>((const T*)d->a, (const T*)d->b, (T*)d->c, (const T*)d->bias, p)));
        return launch_status("skinny-n gemm");
    }
    if (skinny_m_ok(d)) {
        const uint64_t need = skinny_m_workspace(d);
        TVK_REQUIRE(ws && ws_bytes >= need, "tvk_gemm: workspace of %llu bytes required, %llu given", (unsigned long long)need, (unsigned long long)ws_bytes);
        const int N = (int)(16 / dtype_size(d->dtype));
        p.splits = (int)((d->k + simt::kSkinnyMSlice - 1) / simt::kSkinnyMSlice);
        dim3 grid((unsigned)((d->n + 128 * N - 1) / (128 * N)), (unsigned)p.splits);
        TVK_DISPATCH_FLOAT(d->dtype, T, (simt::skinny_m_kernel<T><<<grid, 128, 0, s>>>((const T*)d->a, (const T*)d->b, (float*)ws, p)));
        const int64_t total = d->m * d->n;
        int64_t blocks = (total + 255) / 256;
        if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
        TVK_DISPATCH_FLOAT(d->dtype, T, (simt::splitk_epilogue_kernel<T><<<(unsigned)blocks, 256, 0, s>>>((const float*)ws, (T*)d->c, (const T*)d->bias, p, 0, 1)));
        return launch_status("skinny-m gemm");
    }
    p.splits = simt::plan_splits(d->batch, d->m, d->n, d->k, &p.k_chunk);
    const int64_t gx = (d->n + simt::TN - 1) / simt::TN, gy = (d->m + simt::TM - 1) / simt::TM;
    if (gy > 65535) return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: CUDA-core matmul with m = %lld", (long long)d->m);
    const int64_t max_batch_per_launch = 65535 / p.splits;
    float* partial = (float*)ws;
    if (p.splits > 1) {
        const uint64_t per_batch = (uint64_t)p.splits * d->m * d->n * sizeof(float);
        TVK_REQUIRE(ws && ws_bytes >= per_batch, "tvk_gemm: workspace of %llu bytes required, %llu given", (unsigned long long)per_batch,
                    (unsigned long long)ws_bytes);
    }
    for (int64_t b0 = 0; b0 < d->batch;) {
        int64_t nb = d->batch - b0;
        if (nb > max_batch_per_launch) nb = max_batch_per_launch;
        if (p.splits > 1) {
            // Workspace holds the partials of as many batches as fit.
            const uint64_t per_batch = (uint64_t)p.splits * d->m * d->n * sizeof(float);
            const int64_t fit = (int64_t)(ws_bytes / per_batch);
            if (nb > fit) nb = fit;
        }
        dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)(nb * p.splits));
        TVK_DISPATCH_FLOAT(d->dtype, T, (simt::gemm_kernel<T><<<grid, 256, 0, s>>>((const T*)d->a, (const T*)d->b, (T*)d->c, (const T*)d->bias, partial, p, b0)));
        if (p.splits > 1) {
            const int64_t total = nb * d->m * d->n;
            int64_t blocks = (total + 255) / 256;
            if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
            TVK_DISPATCH_FLOAT(d->dtype, T, (simt::splitk_epilogue_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(partial, (T*)d->c, (const T*)d->bias, p, b0, nb)));
        }
        b0 += nb;
    }
    return launch_status("CUDA-core gemm");
}

// Tiles per CTA block fixed from outside the cost model: 1 for fp32 (its chunked epilogue handles one tile) and for
// outputs one tile tall, else the tuning override TORCHVULKAN_GEMM_MT, else 0 = undecided.
static int pick_mt(const tvk_gemm_desc* d) {
    if (d->dtype == TVK_F32 || d->m <= tc::BM) return 1;
    if (g_tune.mt == 1 || g_tune.mt == 2) return g_tune.mt;
    if (t_block_mt) return t_block_mt;
    const char* e = getenv("TORCHVULKAN_GEMM_MT");   // read per call so that a test can switch it
    const int v = e ? atoi(e) : 0;
    return (v == 1 || v == 2) ? v : 0;   // 0: let the cost model decide
}

static int run_tc(const tvk_gemm_desc* d, void* ws, uint64_t ws_bytes, cudaStream_t s) {
    const int es = (int)dtype_size(d->dtype);
    int mt = pick_mt(d);   // 0 = not fixed yet
    const bool f32 = d->dtype == TVK_F32;
    tc::Params p = {};
    p.m = d->m; p.n = d->n; p.batch = d->batch;
    const int bk = 128 / es;
    p.num_kb = (int)((d->k + bk - 1) / bk);
    p.passes = f32 ? 3 : 1;

    // Operand views. K-major: the contraction index is contiguous.
    const void* a_ptr[2] = {d->a, d->a};
    const void* b_ptr[2] = {d->b, d->b};
    int64_t a_rs = d->a_rs, a_cs = d->a_cs, a_bs = d->a_bs;
    int64_t b_rs = d->b_rs, b_cs = d->b_cs, b_bs = d->b_bs;
    // An operand that can be read either way (a vector) is taken K-major.
    bool a_mn = !(a_cs == 1 && a_rs % (16 / es) == 0 && a_rs >= d->k);
    bool b_mn = !(b_rs == 1 && b_cs % (16 / es) == 0 && b_cs >= d->k);

    if (f32) {
        // hi/lo copies, always K-major: A as [m][k], B as [n][k], pitch rounded to 16 bytes.
        const int64_t ld = (d->k + 3) / 4 * 4;
        const bool a_b = d->batch > 1 && a_bs != 0, b_b = d->batch > 1 && b_bs != 0;
        const int64_t a_nb = a_b ? d->batch : 1, b_nb = b_b ? d->batch : 1;
        const uint64_t a_bytes = align256((uint64_t)a_nb * d->m * ld * 4), b_bytes = align256((uint64_t)b_nb * d->n * ld * 4);
        const uint64_t need = 2 * a_bytes + 2 * b_bytes;
        TVK_REQUIRE(ws && ws_bytes >= need, "tvk_gemm: workspace of %llu bytes required, %llu given", (unsigned long long)need,
                    (unsigned long long)ws_bytes);
        TVK_REQUIRE(((uintptr_t)ws & 255) == 0, "tvk_gemm: workspace must be 256-byte aligned");
        TVK_REQUIRE(a_nb <= 65535 && b_nb <= 65535 && (d->m + 31) / 32 <= 65535 && (d->n + 31) / 32 <= 65535,
                    "torchvulkan [NOT IMPLEMENTED]: fp32 matmul of this extent on the tensor-core path");
        float* a_hi = (float*)ws;
        float* a_lo = (float*)((uint8_t*)ws + a_bytes);
        float* b_hi = (float*)((uint8_t*)ws + 2 * a_bytes);
        float* b_lo = (float*)((uint8_t*)ws + 2 * a_bytes + b_bytes);
        const dim3 block(32, 8);
        const dim3 ga((unsigned)((d->k + 31) / 32), (unsigned)((d->m + 31) / 32), (unsigned)a_nb);
        const dim3 gb((unsigned)((d->k + 31) / 32), (unsigned)((d->n + 31) / 32), (unsigned)b_nb);
        tc::split_tf32_kernel<<<ga, block, 0, s>>>(a_hi, a_lo, (const float*)d->a, d->m, d->k, a_rs, a_cs, a_bs, ld);
        tc::split_tf32_kernel<<<gb, block, 0, s>>>(b_hi, b_lo, (const float*)d->b, d->n, d->k, b_cs, b_rs, b_bs, ld);
        a_ptr[0] = a_hi; a_ptr[1] = a_lo;
        b_ptr[0] = b_hi; b_ptr[1] = b_lo;
        a_rs = ld; a_cs = 1;
        b_rs = 1; b_cs = ld;
        a_bs = a_b ? d->m * ld : 0;
        b_bs = b_b ? d->n * ld : 0;
        a_mn = b_mn = false;
    }
    int bn;
    if (f32) {
        bn = tc::pick_bn(d->batch, d->m, d->n, 32, 64, 1);
    } else {
        const char* e = getenv("TORCHVULKAN_GEMM_BN");
        const int v = g_tune.bn ? g_tune.bn : (t_block_bn ? t_block_bn : (e ? atoi(e) : 0));
        const int forced_bn = (v == 32 || v == 64 || v == 128 || v == 256) ? v : 0;
        const int min_bn = b_mn ? 128 / es : 32;
        const int lo = forced_bn >= min_bn ? forced_bn : min_bn, hi = forced_bn >= min_bn ? forced_bn : 256;
        tc::pick_block(d->batch, d->m, d->n, d->k, lo, hi, mt == 0 ? 1 : mt, mt == 0 ? 2 : mt, &mt, &bn);
    }
    p.chunk_kb = 2;  // 64 values of K per chain
    p.tiles_m = (int)((d->m + mt * tc::BM - 1) / (mt * tc::BM));
    p.tiles_n = (int)((d->n + bn - 1) / bn);
    p.total_tiles = (int64_t)d->batch * p.tiles_m * p.tiles_n;
    if (p.total_tiles >= ((int64_t)1 << 31)) return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: matmul with %lld output tiles", (long long)p.total_tiles);
    p.c = d->c; p.c_rs = d->c_rs; p.c_bs = d->c_bs;
    p.bias = d->bias; p.bias_rs = d->bias_rs; p.bias_cs = d->bias_cs; p.bias_bs = d->bias_bs;
    p.alpha = d->alpha; p.beta = d->beta; p.act = d->activation; p.out_dtype = d->c_f32 ? TVK_F32 : d->dtype;
    p.status = device_status_word();
    p.n_peers = d->n_peer_c;
    for (int q = 0; q < d->n_peer_c; ++q) p.peer_c[q] = d->peer_c[q];
    p.c2 = d->c2;
    p.aux = d->aux_op ? d->aux : nullptr; p.aux_rs = d->aux_rs; p.aux_bs = d->aux_bs; p.aux_op = d->aux_op;
    {
        const int64_t es_out = p.out_dtype == TVK_F32 ? 4 : 2;
        bool aligned = ((uintptr_t)d->c & 15) == 0 && (d->c_rs * es_out) % 16 == 0 && (d->c_bs * es_out) % 16 == 0;
        for (int q = 0; q < d->n_peer_c; ++q) aligned = aligned && ((uintptr_t)d->peer_c[q] & 15) == 0;
        // Staging pays for itself over NVLink (whole 128-byte lines per store instead of 32 scattered 16-byte writes);
        // for the local copy alone the direct 16-byte-per-row stores measure about 10 % faster (L2 merges them).
        static const bool always = getenv("TORCHVULKAN_GEMM_STAGE_ALWAYS") != nullptr;
        p.stage_ok = (aligned && (d->n_peer_c > 0 || always)) ? 1 : 0;
    }
    p.group_m = g_tune.group_m > 0 ? g_tune.group_m : 8;
    p.debug = g_tune.debug;
    p.a_mn = a_mn; p.b_mn = b_mn;
    p.a_batched = d->batch > 1 && a_bs != 0;
    p.b_batched = d->batch > 1 && b_bs != 0;

    const uint32_t fmt = d->dtype == TVK_F16 ? 0u : (d->dtype == TVK_BF16 ? 1u : 2u);
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) | ((uint32_t)(bn >> 3) << 17) |
              ((uint32_t)(tc::BM >> 4) << 24);

    CUtensorMap maps[6] = {};
    const int ch = 128 / es;
    for (int i = 0; i < 2; ++i) {
        int rc;
        if (!a_mn) rc = tc::encode_operand(&maps[i], d->dtype, a_ptr[i], d->k, d->m, a_rs, d->batch, a_bs, bk, mt * tc::BM);
        else rc = tc::encode_operand(&maps[i], d->dtype, a_ptr[i], d->m, d->k, a_cs, d->batch, a_bs, ch, bk);
        if (rc) return rc;
        if (!b_mn) rc = tc::encode_operand(&maps[2 + i], d->dtype, b_ptr[i], d->k, d->n, b_cs, d->batch, b_bs, bk, bn);
        else rc = tc::encode_operand(&maps[2 + i], d->dtype, b_ptr[i], d->n, d->k, b_rs, d->batch, b_bs, ch, bk);
        if (rc) return rc;
    }
    {
        // C through TMA stores: 32-row x 128-byte boxes. Needs what a tensor map needs (16-byte aligned base and pitches)
        // and tiles made of whole boxes; the copies pushed to peers and the fp32 chunked epilogue keep their own stores.
        const int64_t es_out = p.out_dtype == TVK_F32 ? 4 : 2;
        const int gcols = (int)(128 / es_out);
        static const bool off = getenv("TORCHVULKAN_GEMM_NO_TMA_STORE") != nullptr;
        const bool aligned = ((uintptr_t)d->c & 15) == 0 && (d->c_rs * es_out) % 16 == 0 && (d->batch <= 1 || (d->c_bs * es_out) % 16 == 0) &&
                             d->c_rs * es_out < ((int64_t)1 << 40);
        p.tma_store = (!off && !f32 && d->n_peer_c == 0 && aligned && bn % gcols == 0) ? 1 : 0;
        if (p.tma_store && p.c2 && ((uintptr_t)p.c2 & 15) != 0) p.tma_store = 0;
        if (p.tma_store) {
            int rc = tc::encode_operand(&maps[4], p.out_dtype, d->c, d->n, d->m, d->c_rs, d->batch, d->batch > 1 ? d->c_bs : 0, gcols, 32);
            if (rc) return rc;
            if (p.c2) rc = tc::encode_operand(&maps[5], p.out_dtype, p.c2, d->n, d->m, d->c_rs, d->batch, d->batch > 1 ? d->c_bs : 0, gcols, 32);
            if (rc) return rc;
        }
    }
    const bool fused = p.c2 != nullptr || p.aux_op != TVK_AUX_NONE;
    if (f32) return tc::launch_tf32(bn, 1, maps, p, s);
    if (p.out_dtype == TVK_F32) return tc::launch_half_f32out(bn, mt, maps, p, s);
    if (d->dtype == TVK_F16) return fused ? tc::launch_f16_fused(bn, mt, maps, p, s) : tc::launch_f16(bn, mt, maps, p, s);
    if (d->dtype == TVK_BF16) return fused ? tc::launch_bf16_fused(bn, mt, maps, p, s) : tc::launch_bf16(bn, mt, maps, p, s);
    return set_error(TVK_ERR_INVALID, "tvk_gemm: internal tile selection error");
}

// ---- float8 product (used by scaled_mm.cu) ---------------------------------------------------------------
// acc[m][acc_pitch] (fp32) = A @ B for float8 operands read in place: A rows and B columns contiguous along k (both
// "K-major": the layout torch._scaled_mm asks for), 16-byte aligned with pitches that are multiples of 16. kinds: 0 = e4m3,
// 1 = e5m2 per operand. tcgen05.mma kind::f8f6f4, 128 values of K per stage.
bool f8_product_ok(const void* a, int64_t a_rs, int64_t a_cs, const void* b, int64_t b_rs, int64_t b_cs, int64_t m, int64_t n, int64_t k) {
    static const bool off = getenv("TORCHVULKAN_SCALED_MM_WIDEN") != nullptr;       // keep the widening path (tests compare the two)
    if (off || m <= 0 || n <= 0 || k <= 0) return false;
    if (!tc::tma_ok(a, m, k, a_rs, a_cs, 0, 1, 1) || a_cs != 1) return false;
    if (!tc::tma_ok(b, k, n, b_rs, b_cs, 0, 1, 1) || b_rs != 1) return false;
    return m <= 0x7fffffffLL && n <= 0x7fffffffLL && k <= 0x7fffffffLL;
}

int f8_product(int a_kind, int b_kind, const void* a, int64_t a_rs, const void* b, int64_t b_cs, int64_t m, int64_t n, int64_t k, void* out, int out_dtype,
               int64_t out_pitch, const F8Epilogue* epi, cudaStream_t s) {
    if (out_dtype != TVK_F32 && out_dtype != TVK_F16 && out_dtype != TVK_BF16) return set_error(TVK_ERR_INVALID, "float8 product: output dtype %d", out_dtype);
    tc::Params p = {};
    p.m = m; p.n = n; p.batch = 1;
    const int bk = 128;
    p.num_kb = (int)((k + bk - 1) / bk);
    p.passes = 1;
    p.chunk_kb = 2;
    int mt = m <= tc::BM ? 1 : 0, bn = 128;
    // the cost model counts k-blocks of 128 bytes: a float8 k-block holds 128 values, a 16-bit one 64
    tc::pick_block(1, m, n, k / 2 > 0 ? k / 2 : 1, 32, 256, mt == 0 ? 1 : mt, mt == 0 ? 2 : mt, &mt, &bn);
    p.tiles_m = (int)((m + mt * tc::BM - 1) / (mt * tc::BM));
    p.tiles_n = (int)((n + bn - 1) / bn);
    p.total_tiles = (int64_t)p.tiles_m * p.tiles_n;
    if (p.total_tiles >= ((int64_t)1 << 31)) return set_error(TVK_ERR_UNSUPPORTED, "torchvulkan [NOT IMPLEMENTED]: matmul with %lld output tiles", (long long)p.total_tiles);
    p.c = out; p.c_rs = out_pitch; p.c_bs = 0;
    p.alpha = 1.f; p.beta = 0.f; p.act = TVK_ACT_NONE; p.out_dtype = out_dtype;
    if (epi) {
        p.row_scale = epi->row_scale; p.row_scale_stride = (int)epi->row_scale_stride;
        p.col_scale = epi->col_scale; p.col_scale_stride = (int)epi->col_scale_stride;
        if (epi->bias) { p.bias = epi->bias; p.bias_rs = 0; p.bias_cs = 1; p.bias_bs = 0; p.beta = 1.f; }
    }
    p.status = device_status_word();
    p.group_m = 8;
    p.idesc = (1u << 4) | ((uint32_t)a_kind << 7) | ((uint32_t)b_kind << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(tc::BM >> 4) << 24);
    CUtensorMap maps[6] = {};
    int rc = tc::encode_operand(&maps[0], TVK_U8, a, k, m, a_rs, 1, 0, bk, mt * tc::BM);
    if (rc) return rc;
    maps[1] = maps[0];
    rc = tc::encode_operand(&maps[2], TVK_U8, b, k, n, b_cs, 1, 0, bk, bn);
    if (rc) return rc;
    maps[3] = maps[2];
    const int64_t es_out = out_dtype == TVK_F32 ? 4 : 2;
    const int gcols = (int)(128 / es_out);
    const bool aligned = ((uintptr_t)out & 15) == 0 && (out_pitch * es_out) % 16 == 0 && out_pitch * es_out < ((int64_t)1 << 40);
    p.tma_store = (aligned && bn % gcols == 0) ? 1 : 0;
    if (p.tma_store) {
        rc = tc::encode_operand(&maps[4], out_dtype, out, n, m, out_pitch, 1, 0, gcols, 32);
        if (rc) return rc;
    }
    if (out_dtype == TVK_F16) return tc::launch_f8_f16out(bn, mt, maps, p, s);
    if (out_dtype == TVK_BF16) return tc::launch_f8_bf16out(bn, mt, maps, p, s);
    return tc::launch_f8_f32out(bn, mt, maps, p, s);
}

// ---- split-K on the tensor-core path ------------------------------------------------------------------
// A weight-gradient GEMM (m, n in the hundreds, k in the thousands) has too few output tiles to occupy the
// GPU. Its K range is cut into `splits` equal slices that run as the BATCHES of one ordinary launch (slice s of A
// and B is the same matrix shifted by s*kc along K, i.e. a batch stride), each writing an fp32 partial, and the
// partials are summed with the epilogue by simt::splitk_epilogue_kernel.
// One or two 128-row tiles against a large weight matrix (the forward and input-gradient products of a wide layer at a
// small batch): every CTA streams its own columns of B over the whole of K, and what bounds the kernel is the rate at
// which one SM pulls bytes through L2 (about 90 GB/s), not DRAM. 256-column tiles over a slice of K cut the bytes per CTA
// (256x8192x8192: 128x128 tiles over all of K = 4 MB per CTA, 48.7 us; 128x256 tiles over half of K = 3 MB, 43.8 us
// including the pass that sums the two fp32 partials). Returns the number of K slices, 0 when the shape is not of this kind.
static int weight_streaming_splits(const tvk_gemm_desc* d) {
    if (d->m > 2 * tc::BM || d->n < 2048 || d->k < 4096 || d->n % 4 != 0) return 0;
    const int64_t base = ((d->m + tc::BM - 1) / tc::BM) * ((d->n + 255) / 256);
    const int64_t want = (int64_t)sm_count() / base;
    const int64_t nkb = d->k / 64;
    int best = 0;
    for (int sp = 2; sp <= 8 && sp <= want; sp *= 2)
        if (nkb % sp == 0 && d->k / sp >= 1024) best = sp;
    return best;
}

// The CTA-pair kernel (gemm_tc_2sm.cu) takes the K slices of a product whose output is more than one row tile tall, with
// operands that have one unit stride each and slices of whole k-blocks. TORCHVULKAN_GEMM_PAIR=0 keeps the single-CTA kernel.
static bool pair_kernel_ok(const tvk_gemm_desc* part) {
    const char* e = getenv("TORCHVULKAN_GEMM_PAIR");      // read per call so that a test can switch it
    if (e && atoi(e) == 0) return false;
    if (part->dtype != TVK_F16 && part->dtype != TVK_BF16) return false;
    if (part->m <= tc::BM || part->k % 64 != 0 || part->n % 4 != 0) return false;
    if (!(part->a_cs == 1 || part->a_rs == 1)) return false;
    if (!(part->b_rs == 1 || part->b_cs == 1)) return false;
    return true;
}

// K slices for the pair kernel: a product with so few 256 x 256 tiles that at least two slices of each fit the GPU's CTA
// pairs at once (the weight gradients of a decoder layer, the wide layers of an MLP at a small batch). Such products
// are bound by L2->SM traffic per CTA, and a pair tile pulls two thirds of the bytes of a 128 x 256 tile. 0 = not this kind.
static int pair_splits(const tvk_gemm_desc* d) {
    if (d->batch != 1 || d->k < 2048 || d->k % 64 != 0 || !pair_kernel_ok(d)) return 0;
    const int64_t tiles = ((d->m + 255) / 256) * ((d->n + 255) / 256), pairs = sm_count() / 2, nkb = d->k / 64;
    int best = 0;
    for (int sp = 2; sp <= 8 && tiles * sp <= pairs; sp *= 2)
        if (nkb % sp == 0 && d->k / sp >= 512) best = sp;
    return best;
}

static int tc_splitk_plan(const tvk_gemm_desc* d) {
    static const bool off = getenv("TORCHVULKAN_GEMM_NO_SPLITK") != nullptr;
    // (the fused forms are applied by the finishing pass of the K slices when n % 4 == 0)
    if (off || d->dtype == TVK_F32 || d->c_f32 || d->n_peer_c > 0 || (fused_epilogue(d) && d->n % 4 != 0) || d->batch != 1 || d->k < 2048 || d->k % 64 != 0) return 1;
    static const int forced = [] {
        const char* e = getenv("TORCHVULKAN_GEMM_SPLITS");
        return e ? atoi(e) : 0;
    }();
    if (g_tune.splits >= 1 && g_tune.splits <= 64 && (d->k / 64) % g_tune.splits == 0) return g_tune.splits;
    if (forced >= 1 && forced <= 64 && (d->k / 64) % forced == 0) return forced;
    const int64_t nkb = d->k / 64;
    if (const int p_splits = pair_splits(d)) return p_splits;
    if (const int ws_splits = weight_streaming_splits(d)) return ws_splits;
    const int64_t tiles = ((d->m + tc::BM - 1) / tc::BM) * ((d->n + 127) / 128);
    if (tiles >= 100) return 1;
    int best = 1;
    for (int64_t sp = 2; sp <= nkb / 4 && sp <= 64; ++sp) {
        if (nkb % sp != 0) continue;
        best = (int)sp;
        if (tiles * sp >= 100) break;
    }
    return best;
}

static int run_tc_splitk(const tvk_gemm_desc* d, int splits, void* ws, uint64_t ws_bytes, cudaStream_t s) {
    const uint64_t need = (uint64_t)splits * d->m * d->n * sizeof(float);
    TVK_REQUIRE(ws && ws_bytes >= need, "tvk_gemm: workspace of %llu bytes required, %llu given", (unsigned long long)need, (unsigned long long)ws_bytes);
    const int64_t kc = d->k / splits;
    tvk_gemm_desc part = *d;
    part.batch = splits;
    part.k = kc;
    part.a_bs = kc * d->a_cs;
    part.b_bs = kc * d->b_rs;
    part.c = ws; part.c_rs = d->n; part.c_bs = d->m * d->n; part.c_f32 = 1;
    part.bias = nullptr; part.alpha = 1.f; part.beta = 0.f; part.activation = TVK_ACT_NONE;
    part.aux = nullptr; part.aux_op = TVK_AUX_NONE; part.c2 = nullptr;
    if (!tc_eligible(&part)) return -1;                      // the caller runs the unsplit kernel
    int rc = -2;
    if ((pair_splits(d) == splits || weight_streaming_splits(d) == splits) && pair_kernel_ok(&part)) {
        // CTA pairs: each CTA loads its own rows of A and half of a 256-column tile of B (gemm_tc_2sm.cu)
        const bool a_mn = part.a_cs != 1, b_mn = part.b_rs != 1;
        const uint32_t fmt = d->dtype == TVK_F16 ? 0u : 1u;
        const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) | ((uint32_t)(256 >> 3) << 17) |
                               ((uint32_t)(256 >> 4) << 24);
        CUtensorMap maps[3] = {};
        rc = tc::encode_operand(&maps[2], TVK_F32, ws, part.n, part.m, part.n, splits, part.m * part.n, 32, 32);
        if (rc) return rc;
        if (!a_mn) rc = tc::encode_operand(&maps[0], d->dtype, part.a, part.k, part.m, part.a_rs, splits, part.a_bs, 64, 128);
        else rc = tc::encode_operand(&maps[0], d->dtype, part.a, part.m, part.k, part.a_cs, splits, part.a_bs, 64, 64);
        if (rc) return rc;
        if (!b_mn) rc = tc::encode_operand(&maps[1], d->dtype, part.b, part.k, part.n, part.b_cs, splits, part.b_bs, 64, 128);
        else rc = tc::encode_operand(&maps[1], d->dtype, part.b, part.n, part.k, part.b_rs, splits, part.b_bs, 64, 64);
        if (rc) return rc;
        rc = tc::launch_pair(a_mn, b_mn, maps, part.m, part.n, (int)(kc / 64), splits, idesc, (float*)ws, device_status_word(), g_tune.debug, s);
        if (rc) return rc;
    } else {
        if (weight_streaming_splits(d) == splits) { t_block_bn = 256; t_block_mt = 1; }
        rc = run_tc(&part, nullptr, 0, s);
        t_block_bn = t_block_mt = 0;
        if (rc) return rc;
    }
    simt::Params p = {};
    p.m = d->m; p.n = d->n; p.k = d->k;
    p.c_rs = d->c_rs; p.c_bs = d->c_bs;
    p.bias_rs = d->bias_rs; p.bias_cs = d->bias_cs; p.bias_bs = d->bias_bs;
    p.alpha = d->alpha; p.beta = d->beta; p.act = d->activation;
    p.splits = splits;
    p.aux = d->aux_op ? d->aux : nullptr; p.aux_rs = d->aux_rs; p.aux_op = d->aux_op;
    p.c2 = d->c2;
    const int64_t total = d->m * d->n;
    if (d->n % 4 == 0) {
        int64_t blocks = (total / 4 + 255) / 256;
        if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
        TVK_DISPATCH_FLOAT(d->dtype, T, (simt::splitk_epilogue_vec_kernel<T><<<(unsigned)blocks, 256, 0, s>>>((const float*)ws, (T*)d->c, (const T*)d->bias, p)));
        return launch_status("split-K epilogue");
    }
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
    TVK_DISPATCH_FLOAT(d->dtype, T, (simt::splitk_epilogue_kernel<T><<<(unsigned)blocks, 256, 0, s>>>((const float*)ws, (T*)d->c, (const T*)d->bias, p, 0, 1)));
    return launch_status("split-K epilogue");
}

// The descriptor of the same product with the repacked operands at `base` (A first, then B), both K-major with pitch kp.
static tvk_gemm_desc repacked_desc(const tvk_gemm_desc* d, const Repack& r, void* base) {
    tvk_gemm_desc e = *d;
    if (r.a) { e.a = base; e.a_rs = r.kp; e.a_cs = 1; }
    if (r.b) { e.b = (uint8_t*)base + r.a_bytes; e.b_rs = 1; e.b_cs = r.kp; }
    return e;
}

static int run_repack(const tvk_gemm_desc* d, const Repack& r, void* base, cudaStream_t s) {
    if (r.a) {
        const int64_t total = d->m * r.kp;
        TVK_DISPATCH_FLOAT(d->dtype, T, (simt::repack_kernel<T><<<(unsigned)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096), 256, 0, s>>>(
            (T*)base, (const T*)d->a, d->m, d->k, r.kp, d->a_rs, d->a_cs)));
    }
    if (r.b) {
        const int64_t total = d->n * r.kp;
        TVK_DISPATCH_FLOAT(d->dtype, T, (simt::repack_kernel<T><<<(unsigned)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096), 256, 0, s>>>(
            (T*)((uint8_t*)base + r.a_bytes), (const T*)d->b, d->n, d->k, r.kp, d->b_cs, d->b_rs)));
    }
    return launch_status("operand repack");
}

}  // namespace tvk

using namespace tvk;

extern "C" {

int tvk_debug_gemm_tuning(int bn, int mt, int splits, int group_m, int debug) {
    g_tune.bn = bn; g_tune.mt = mt; g_tune.splits = splits; g_tune.group_m = group_m; g_tune.debug = debug;
    return TVK_OK;
}

int tvk_gemm_path(const tvk_gemm_desc* d, int* path) {
    int rc = validate(d);
    if (rc) return rc;
    if (!path) return set_error(TVK_ERR_INVALID, "tvk_gemm_path: null output");
    *path = choose_path(d);
    if (*path == 0) return set_error(TVK_ERR_UNSUPPORTED, "tvk_gemm: operands cannot be addressed by the tensor-core path");
    return TVK_OK;
}

int tvk_gemm_splits(const tvk_gemm_desc* d, int* splits) {
    int rc = validate(d);
    if (rc) return rc;
    if (!splits) return set_error(TVK_ERR_INVALID, "tvk_gemm_splits: null output");
    *splits = 1;
    if (d->batch == 0 || d->m == 0 || d->n == 0 || d->k == 0) return TVK_OK;
    if (choose_path(d) != 1) return TVK_OK;
    if (!tc_eligible(d)) {
        const Repack r = plan_repack(d);
        if (!(r.a || r.b)) return TVK_OK;
        tvk_gemm_desc e = repacked_desc(d, r, (void*)256);
        *splits = tc_splitk_plan(&e);
        return TVK_OK;
    }
    *splits = tc_splitk_plan(d);
    return TVK_OK;
}

int tvk_gemm_workspace_size(const tvk_gemm_desc* d, uint64_t* bytes) {
    int rc = validate(d);
    if (rc) return rc;
    if (!bytes) return set_error(TVK_ERR_INVALID, "tvk_gemm_workspace_size: null output");
    *bytes = 0;
    if (d->batch == 0 || d->m == 0 || d->n == 0 || d->k == 0) return TVK_OK;
    const int path = choose_path(d);
    if (path == 0) return set_error(TVK_ERR_UNSUPPORTED, "tvk_gemm: operands cannot be addressed by the tensor-core path");
    if (path == 2 && skinny_n_ok(d)) return TVK_OK;
    if (path == 2 && skinny_m_ok(d)) {
        *bytes = skinny_m_workspace(d);
        return TVK_OK;
    }
    if (path == 2) {
        int64_t chunk;
        const int splits = simt::plan_splits(d->batch, d->m, d->n, d->k, &chunk);
        if (splits > 1) {
            // Room for every batch, capped; run_simt processes as many batches per launch as fit.
            uint64_t per_batch = (uint64_t)splits * d->m * d->n * sizeof(float);
            uint64_t all = per_batch * (uint64_t)d->batch;
            const uint64_t cap = (uint64_t)256 << 20;
            *bytes = all <= cap ? all : (per_batch > cap ? per_batch : cap / per_batch * per_batch);
        }
        return TVK_OK;
    }
    if (!tc_eligible(d)) {
        // tensor-core path through repacked copies of the operands TMA cannot address
        const Repack r = plan_repack(d);
        const tvk_gemm_desc e = repacked_desc(d, r, (void*)(uintptr_t)256);
        *bytes = r.a_bytes + r.b_bytes;
        if (tc_splitk_plan(&e) > 1) *bytes += (uint64_t)tc_splitk_plan(&e) * d->m * d->n * sizeof(float);
        return TVK_OK;
    }
    if (tc_splitk_plan(d) > 1) {
        *bytes = (uint64_t)tc_splitk_plan(d) * d->m * d->n * sizeof(float);
        return TVK_OK;
    }
    if (d->dtype == TVK_F32) {
        const int64_t ld = (d->k + 3) / 4 * 4;
        const int64_t a_nb = (d->batch > 1 && d->a_bs != 0) ? d->batch : 1, b_nb = (d->batch > 1 && d->b_bs != 0) ? d->batch : 1;
        *bytes = 2 * align256((uint64_t)a_nb * d->m * ld * 4) + 2 * align256((uint64_t)b_nb * d->n * ld * 4);
    }
    return TVK_OK;
}

int tvk_gemm(const tvk_gemm_desc* d, void* workspace, uint64_t workspace_bytes, void* stream) {
    int rc = validate(d);
    if (rc) return rc;
    if (d->batch == 0 || d->m == 0 || d->n == 0) return TVK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (small_k_ok(d)) return run_small_k(d, s);
    const int path = (d->k == 0) ? 2 : choose_path(d);
    if (path == 0) return set_error(TVK_ERR_UNSUPPORTED, "tvk_gemm: operands cannot be addressed by the tensor-core path");
    if (path == 2) return run_simt(d, workspace, workspace_bytes, s);
    tvk_gemm_desc packed;
    if (!tc_eligible(d)) {
        const Repack r = plan_repack(d);
        const uint64_t need = r.a_bytes + r.b_bytes;
        TVK_REQUIRE((r.a || r.b) && workspace && workspace_bytes >= need && ((uintptr_t)workspace & 255) == 0,
                    "tvk_gemm: a 256-byte aligned workspace of %llu bytes is required, %llu given", (unsigned long long)need, (unsigned long long)workspace_bytes);
        rc = run_repack(d, r, workspace, s);
        if (rc) return rc;
        packed = repacked_desc(d, r, workspace);
        TVK_REQUIRE(tc_eligible(&packed), "tvk_gemm: internal error, repacked operands are not addressable");
        d = &packed;
        workspace = (uint8_t*)workspace + need;
        workspace_bytes -= need;
    }
    const int splits = tc_splitk_plan(d);
    if (splits > 1) {
        rc = run_tc_splitk(d, splits, workspace, workspace_bytes, s);
        if (rc >= 0) return rc;
    }
    return run_tc(d, workspace, workspace_bytes, s);
}

}  // extern "C"
