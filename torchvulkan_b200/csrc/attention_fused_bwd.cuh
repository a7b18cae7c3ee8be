// Fused attention backward for head size 64 and key counts that are multiples of 128: one kernel recomputes the scores
// and forms dV, dK and per-key-block partials of dQ; the probabilities and their gradients never leave the SM.
//
// Replaces, for these shapes, the five GEMMs and the dsoftmax kernel of attention.cu (which stay the path for every other
// shape). Counterpart in the reference: sdpa_backward_vulkan (src/api/ops/attention.cpp:641-749), same conventions as the
// forward: p = exp(s*scale - lse) (0 where masked or lse = +inf), P rounded to the input dtype before it multiplies dO,
// dS = p * (dP - delta) * scale with delta = sum(dO * O), causal masks aligned to the top-left corner (key j visible to query l when j <= l), all query heads
// of a KV group are rows of one matrix (row = g*L + l).
//
// One CTA per (group, block of 128 keys), 576 threads; K_j and V_j stay in shared memory and the CTA walks the 128-row
// query tiles that can see the block:
//   warp 0    TMA: K_j, V_j once; Q_i and dO_i of the next tile into the other half of a double buffer
//   warp 1    tcgen05.mma: S = Q_i.K_j^T and dP = dO_i.V_j^T (tensor-memory columns [0,128) and [128,256)); after the
//             threads have written P and dS: dV_j += P^T.dO_i [256,320), dK_j += dS^T.Q_i [320,384), dQ_i = dS.K_j [384,448)
//             (P^T and dS^T are the same shared-memory tiles read as MN-major operands; dO_i, Q_i and K_j as MN-major B)
//   warps 2-17 four threads per query row (a warp reads the 32 tensor-memory lanes of its quarter, the four warps of a quarter
//             take 32 of the 128 columns each; this part of the kernel is bound by instruction latency, so it wants many
//             warps per scheduler): p and dS from the two rows in tensor memory, written as K-major swizzled
//             tiles; then the row of dQ_i (fp32) to this key block's partial buffer; at the end dV_j and dK_j to global memory.
// dQ is the sum of the partials of the key blocks a tile can see, added and rounded by attn_dq_finalize_kernel.
#pragma once

#include "tc_common.cuh"

namespace tvk {
namespace attn {

constexpr int kBwdWarps = 16;                     // compute warps
constexpr int kBwdThreads = 64 + kBwdWarps * 32;
constexpr int kBwdTmemCols = 512;                 // 448 used; allocated and freed with the same count
constexpr int kBwdTile = 128 * 128;               // bytes of a [128 x 64] two-byte tile
constexpr int kBwdSmemBytes = 2 * kBwdTile /*K,V*/ + 4 * kBwdTile /*Q,dO x2*/ + 4 * kBwdTile /*P, dS*/ + 1024 + 256;
constexpr float kBwdDsScale = 1024.f;             // dS is stored times this so that fp16 keeps it out of its subnormals

struct BwdParams {
    int L, S;
    int rows_per_group;              // G * L (a multiple of 128)
    int tiles_per_group;
    int kblocks;                     // S / 128
    float scale, scale_log2e;
    int causal;
    const float* lse;                // [total_rows]
    const float* delta;              // [total_rows]
    float* dq_part;                  // [kblocks][total_rows][64] fp32, times kBwdDsScale
    int64_t total_rows;
    void* dk;                        // [groups * S, 64]
    void* dv;
    int dtype;
    uint32_t idesc_s, idesc_t, idesc_q;
    int* status;
};

// Can any row of query tile `tile` see a key of block `kb`? (The loop of the kernel and the finalize kernel must agree.)
__host__ __device__ inline bool tile_sees_block(int tile, int kb, int L, int S, int causal) {
    if (!causal) return true;
    const int l_hi = (L % 128 == 0) ? (tile * 128) % L + 127 : L - 1;
    return kb * 128 <= l_hi;
}

__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const BwdParams p) {
    using namespace tc;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sK = smem;
    uint8_t* sV = sK + kBwdTile;
    uint8_t* sQ = sV + kBwdTile;              // [2][Q tile | dO tile]
    uint8_t* sP = sQ + 4 * kBwdTile;          // [2 key half-blocks of 64][128 rows][128 B]
    uint8_t* sDS = sP + 2 * kBwdTile;
    uint64_t* bars = (uint64_t*)(sDS + 2 * kBwdTile);
    uint32_t* tmem_slot = (uint32_t*)(bars + 8);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_kv = smem_u32(bars), bar_q0 = smem_u32(bars + 1) /* and +2 */, bar_s = smem_u32(bars + 3), bar_p = smem_u32(bars + 4),
                   bar_o = smem_u32(bars + 5), bar_free0 = smem_u32(bars + 6) /* and +7 */;

    if (threadIdx.x == 0) {
        mbar_init(bar_kv, 1); mbar_init(bar_q0, 1); mbar_init(bar_q0 + 8, 1); mbar_init(bar_s, 1); mbar_init(bar_p, kBwdWarps); mbar_init(bar_o, 1);
        mbar_init(bar_free0, 1); mbar_init(bar_free0 + 8, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kBwdTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 320, t_dq = tmem_base + 384;

    const int group = blockIdx.x / p.kblocks, kb = blockIdx.x - group * p.kblocks;
    const int64_t grow0 = (int64_t)group * p.rows_per_group;       // first query row of the group
    const int key0 = kb * 128;
    // the tiles this block walks: those that see it (with a causal mask the later ones; the order is ascending)
    int first_tile = 0;
    while (first_tile < p.tiles_per_group && !tile_sees_block(first_tile, kb, p.L, p.S, p.causal)) ++first_tile;
    // (visibility is not monotonic over tiles when the tiles of several heads follow each other, so every tile is tested)

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(bar_kv, 2 * kBwdTile);
            tma_load_2d(smem_u32(sK), &tmap_k, 0, group * p.S + key0, bar_kv);
            tma_load_2d(smem_u32(sV), &tmap_v, 0, group * p.S + key0, bar_kv);
            bool ok = true;
            int it = 0;
            for (int tile = first_tile; tile < p.tiles_per_group && ok; ++tile) {
                if (!tile_sees_block(tile, kb, p.L, p.S, p.causal)) continue;
                const int buf = it & 1;
                // the products of iteration it-2 read this buffer; its own barrier flips once per use, so the parity of the
                // previous use cannot be confused with a later one (bar_o may already be a phase further)
                if (it >= 2) ok = mbar_wait(bar_free0 + 8 * buf, (uint32_t)(((it >> 1) - 1) & 1), abort_flag, p.status, 61);
                if (!ok) break;
                const uint32_t dst = smem_u32(sQ) + buf * 2 * kBwdTile;
                mbar_expect_tx(bar_q0 + 8 * buf, 2 * kBwdTile);
                tma_load_2d(dst, &tmap_q, 0, (int)(grow0 + (int64_t)tile * 128), bar_q0 + 8 * buf);
                tma_load_2d(dst + kBwdTile, &tmap_do, 0, (int)(grow0 + (int64_t)tile * 128), bar_q0 + 8 * buf);
                ++it;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = mbar_wait(bar_kv, 0, abort_flag, p.status, 62);
            int it = 0;
            for (int tile = first_tile; tile < p.tiles_per_group && ok; ++tile) {
                if (!tile_sees_block(tile, kb, p.L, p.S, p.causal)) continue;
                const int buf = it & 1;
                const uint32_t q = smem_u32(sQ) + buf * 2 * kBwdTile, dO = q + kBwdTile;
                ok = mbar_wait(bar_q0 + 8 * buf, (uint32_t)((it >> 1) & 1), abort_flag, p.status, 63);
                if (!ok) break;
                tc_fence_after();
                // S = Q.K^T and dP = dO.V^T: both operands K-major, four steps of 16 over the head size
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    umma<false>(t_s, make_smem_desc(q + ks * 32, 16, 1024), make_smem_desc(smem_u32(sK) + ks * 32, 16, 1024), p.idesc_s, ks > 0 ? 1u : 0u);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    umma<false>(t_dp, make_smem_desc(dO + ks * 32, 16, 1024), make_smem_desc(smem_u32(sV) + ks * 32, 16, 1024), p.idesc_s, ks > 0 ? 1u : 0u);
                umma_commit(bar_s);
                ok = mbar_wait(bar_p, (uint32_t)(it & 1), abort_flag, p.status, 64);
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = it > 0 ? 1u : 0u;
                // dV += P^T.dO and dK += dS^T.Q: contraction over the 128 query rows, 16 per step (two 8-row groups = 2048 B);
                // A is the [rows][keys] tile read MN-major (two 64-key column blocks one tile apart), B is [rows][64] MN-major
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    umma<false>(t_dv, make_smem_desc(smem_u32(sP) + ks * 2048, kBwdTile, 1024), make_smem_desc(dO + ks * 2048, kBwdTile, 1024), p.idesc_t,
                                (acc | (uint32_t)ks) ? 1u : 0u);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    umma<false>(t_dk, make_smem_desc(smem_u32(sDS) + ks * 2048, kBwdTile, 1024), make_smem_desc(q + ks * 2048, kBwdTile, 1024), p.idesc_t,
                                (acc | (uint32_t)ks) ? 1u : 0u);
                // dQ_i = dS.K_j: contraction over the 128 keys; A K-major (two 64-key blocks, 32 B per step), B = K_j MN-major
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    umma<false>(t_dq, make_smem_desc(smem_u32(sDS) + (ks >> 2) * kBwdTile + (ks & 3) * 32, 16, 1024),
                                make_smem_desc(smem_u32(sK) + ks * 2048, kBwdTile, 1024), p.idesc_q, ks > 0 ? 1u : 0u);
                umma_commit(bar_o);
                umma_commit(bar_free0 + 8 * buf);
                ++it;
            }
        }
    } else {
        const int lane_window = (warp & 3) * 32;
        const int r = lane_window + lane;                          // row of the tile (and, at the end, key of the block)
        const int part = (warp - 2) >> 2;                          // which 32 of the 128 columns this warp takes
        const uint32_t tlane = (uint32_t)lane_window << 16;
        bool ok = true;
        int it = 0;
        for (int tile = first_tile; tile < p.tiles_per_group && ok; ++tile) {
            if (!tile_sees_block(tile, kb, p.L, p.S, p.causal)) continue;
            const int64_t row = grow0 + (int64_t)tile * 128 + r;
            const int l = (int)((tile * 128 + r) % p.L);
            const int limit = p.causal ? (l + 1) : p.S;      // keys [0, limit) are visible to this row
            const int nvis = limit - key0 < 0 ? 0 : (limit - key0 > 128 ? 128 : limit - key0);   // visible keys of this block
            const float ls = p.lse[row], dl = p.delta[row];
            const bool dead = !(ls < INFINITY);                            // +inf (or NaN): the row attended to nothing
            const float ls2 = ls * 1.4426950408889634f;
            ok = mbar_wait(bar_s, (uint32_t)(it & 1), abort_flag, p.status, 65);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
#pragma unroll 1
            {
                const int c0 = part * 32;
                uint32_t sv[32], gv[32];
                tmem_ld32(t_s + tlane + (uint32_t)c0, sv);
                tmem_ld32(t_dp + tlane + (uint32_t)c0, gv);
                tmem_ld_wait();
                uint32_t pp[16], dd[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float pr[2], ds[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const bool vis = c0 + 2 * j + e < nvis && !dead;
                        pr[e] = vis ? ex2_approx(fmaf(__uint_as_float(sv[2 * j + e]), p.scale_log2e, -ls2)) : 0.f;
                    }
                    // the forward pass multiplied V by the rounded probabilities: differentiate that function
                    if (p.dtype == TVK_F16) {
                        const __half2 a = __floats2half2_rn(pr[0], pr[1]);
                        pp[j] = *(const uint32_t*)&a;
                        pr[0] = __low2float(a); pr[1] = __high2float(a);
                    } else {
                        const __nv_bfloat162 a = __floats2bfloat162_rn(pr[0], pr[1]);
                        pp[j] = *(const uint32_t*)&a;
                        pr[0] = __low2float(a); pr[1] = __high2float(a);
                    }
#pragma unroll
                    for (int e = 0; e < 2; ++e)
                        ds[e] = fminf(fmaxf(pr[e] * (__uint_as_float(gv[2 * j + e]) - dl) * p.scale * kBwdDsScale, -60000.f), 60000.f);
                    if (p.dtype == TVK_F16) { const __half2 b = __floats2half2_rn(ds[0], ds[1]); dd[j] = *(const uint32_t*)&b; }
                    else { const __nv_bfloat162 b = __floats2bfloat162_rn(ds[0], ds[1]); dd[j] = *(const uint32_t*)&b; }
                }
                // K-major 128-byte-swizzled tiles: row r, 16-byte chunk c of key half-block h sits at chunk position c ^ (r & 7)
                const int off = (c0 >> 6) * kBwdTile + r * 128;
                const int cbase = (c0 & 63) >> 3;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int ch = ((cbase + i) ^ (r & 7)) << 4;
                    *(uint4*)(sP + off + ch) = make_uint4(pp[4 * i], pp[4 * i + 1], pp[4 * i + 2], pp[4 * i + 3]);
                    *(uint4*)(sDS + off + ch) = make_uint4(dd[4 * i], dd[4 * i + 1], dd[4 * i + 2], dd[4 * i + 3]);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p);
            ok = mbar_wait(bar_o, (uint32_t)(it & 1), abort_flag, p.status, 66);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            float* qrow = p.dq_part + ((int64_t)kb * p.total_rows + row) * 64;
            if (part < 2) {
                const int c0 = part * 32;
                uint32_t v[32];
                tmem_ld32(t_dq + tlane + (uint32_t)c0, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *(float4*)(qrow + c0 + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
            }
            tc_fence_before();
            ++it;
        }
        // dV_j and dK_j: row r of the accumulators is key key0 + r (zero when no tile saw the block)
        if (ok) {
            const int64_t krow = (int64_t)group * p.S + key0 + r;
            const float inv = 1.0f / kBwdDsScale;
            {
                const int which = part >> 1;                 // 32 columns of one accumulator per warp of the quarter
                uint16_t* dst = (uint16_t*)(which == 0 ? p.dv : p.dk) + krow * 64;
                const float mul = which == 0 ? 1.f : inv;
                {
                    const int c0 = (part & 1) * 32;
                    uint32_t v[32];
                    if (it > 0) {
                        tmem_ld32((which == 0 ? t_dv : t_dk) + tlane + (uint32_t)c0, v);
                        tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = 0u;
                    }
                    uint32_t packed[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float a = __uint_as_float(v[2 * j]) * mul, b = __uint_as_float(v[2 * j + 1]) * mul;
                        if (p.dtype == TVK_F16) { const __half2 h = __floats2half2_rn(a, b); packed[j] = *(const uint32_t*)&h; }
                        else { const __nv_bfloat162 h = __floats2bfloat162_rn(a, b); packed[j] = *(const uint32_t*)&h; }
                    }
#pragma unroll
                    for (int j = 0; j < 16; j += 4) *(uint4*)(dst + c0 + 2 * j) = make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
                }
            }
        }
    }
    __syncwarp();
    if (*abort_flag) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kBwdTmemCols) : "memory");
    }
}

// dQ[row, :] = (sum over the key blocks the row's tile can see of dq_part[kb][row, :]) / kBwdDsScale, rounded to T.
// One thread per four columns.
template <typename T>
__global__ void __launch_bounds__(256) attn_dq_finalize_kernel(T* __restrict__ dq, const float* __restrict__ part, int64_t total_rows, int rows_per_group,
                                                              int kblocks, int L, int S, int causal) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total_rows * 16) return;
    const int64_t row = idx >> 4;
    const int c = (int)(idx & 15) * 4;
    const int tile = (int)((row % rows_per_group) / 128);
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int kb = 0; kb < kblocks; ++kb) {
        if (!tile_sees_block(tile, kb, L, S, causal)) continue;
        const float4 v = *(const float4*)(part + ((int64_t)kb * total_rows + row) * 64 + c);
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
    }
    const float inv = 1.0f / kBwdDsScale;
    T* o = dq + row * 64 + c;
    o[0] = from_f32<T>(a.x * inv); o[1] = from_f32<T>(a.y * inv); o[2] = from_f32<T>(a.z * inv); o[3] = from_f32<T>(a.w * inv);
}

}  // namespace attn
}  // namespace tvk
