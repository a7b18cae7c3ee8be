// Fused attention forward for head size 64 and up to 256 keys: Q.K^T, softmax and P.V in one kernel, the scores in
// tensor memory, never in HBM.
//
// Replaces, for these shapes, the GEMM -> softmax kernel -> GEMM sequence of attention.cu (which stays the path for
// every other shape and for the backward pass). Counterpart in the reference: fused_forward
// (src/api/ops/attention.cpp:395-480, src/shaders/ops/attention_coop.slang:117-222), whose conventions are kept:
// probabilities are rounded to the input dtype before they multiply V and the denominator sums the rounded values;
// the log-sum-exp is fp32; a query row without a visible key gives out = 0 and lse = +inf; causal masks are aligned
// to the top-left corner (key j is visible to query l when j <= l, attention_coop.slang:53-56); all query heads of a KV group are
// rows of one matrix (row = g*L + l).
//
// One CTA per 128 query rows of one (batch, kv head) group, 320 threads:
//   warp 0   TMA: Q tile [128 x 64], K [256 x 64], V [256 x 64] (each row is one 128-byte swizzled line)
//   warp 1   tcgen05.mma: S = Q.K^T (M=128, N<=256, K=64) into tensor-memory columns [0, 256); later O = P.V
//            (M=128, N=64, K<=256), with V as an MN-major operand (a key's 64 values are the 128-byte row)
//   warps 2-9 the row math, two threads per query row (a warp reads the 32 tensor-memory lanes of its quarter, so two
//            warps share a quarter and take alternate 32-column chunks): two passes over the row of S in tensor memory
//            (max, then exp and sum; the two halves of a row meet through shared memory), P written to shared memory
//            as the K-major swizzled A operand of the second product, then O / sum -> out. The row math is what bounds
//            the kernel (instruction issue and tensor-memory load latency), hence eight warps and the one-instruction
//            ex2.approx exponential on chunks that need no mask.
// O reuses the first 64 tensor-memory columns of S (all rows have been read by then), so a CTA holds 256 columns and
// two CTAs share an SM. With a causal mask only the key blocks some row of the tile can see are multiplied.
#pragma once

#include "tc_common.cuh"

namespace tvk {
namespace attn {

constexpr int kFusedS = 256;                       // key tile (tensor-memory columns of S)
constexpr int kFusedTmemCols = 256;                // allocated and freed with the same count
constexpr int kSmemQ = 128 * 128, kSmemK = kFusedS * 128, kSmemV = kFusedS * 128, kSmemP = 4 * 128 * 128;
// P (64 KB) is written after the first product has finished reading Q and K, so it overlays them: V | [Q K ...] = 96 KB,
// two CTAs per SM (their phases interleave: one multiplies while the other exponentiates).
constexpr int kFusedThreads = 64 + 256;            // producer warp, MMA warp, eight row-math warps
constexpr int kFusedSmemBytes = kSmemV + kSmemP + 1024 + 256 + 2048;      // + row max and row sum of each half (2 x 2 x 128 floats)

struct FusedParams {
    int L, S;                        // queries per head, keys
    int rows_per_group;              // G * L (a multiple of 128)
    int tiles_per_group;
    float scale_log2e;               // softmax scale * log2(e)
    float scale;
    int causal;
    void* out;                       // [total_rows, 64]
    float* lse;                      // [total_rows]
    int dtype;
    uint32_t idesc_qk, idesc_pv;
    int* status;
};

__global__ void __launch_bounds__(kFusedThreads, 2)
attn_fwd_fused_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                      const FusedParams p) {
    using namespace tc;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sV = smem;
    uint8_t* sP = sV + kSmemV;            // 64 KB; Q and K live in its first 48 KB until S has been computed
    uint8_t* sQ = sP;
    uint8_t* sK = sQ + kSmemQ;
    uint64_t* bars = (uint64_t*)(sP + kSmemP);
    uint32_t* tmem_slot = (uint32_t*)(bars + 5);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* xmax = (float*)((uint8_t*)bars + 256);     // [2][128]: row max found by each half
    float* xsum = xmax + 256;                         // [2][128]: sum of the rounded probabilities of each half
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_qk = smem_u32(bars), bar_v = smem_u32(bars + 1), bar_s = smem_u32(bars + 2), bar_p = smem_u32(bars + 3),
                   bar_o = smem_u32(bars + 4);

    if (threadIdx.x == 0) {
        mbar_init(bar_qk, 1); mbar_init(bar_v, 1); mbar_init(bar_s, 1); mbar_init(bar_p, 8); mbar_init(bar_o, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kFusedTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // Under a causal mask the tiles low in a head see few keys and finish early: launch order runs from the last tile of
    // every head to the first, so that the CTAs of the final, partial wave are the short ones.
    int tile_id = (int)blockIdx.x;
    if (p.causal && p.L % 128 == 0) {
        const int tph = p.L / 128, heads = (int)gridDim.x / tph;          // tiles per head; the grid is a whole number of heads
        tile_id = ((int)blockIdx.x % heads) * tph + (tph - 1 - (int)blockIdx.x / heads);
    }
    const int group = tile_id / p.tiles_per_group, tile = tile_id - group * p.tiles_per_group;
    const int64_t row0 = (int64_t)group * p.rows_per_group + (int64_t)tile * 128;     // first query row of the tile
    // keys some row of this tile can see, rounded up to whole 64-key blocks: the extent of both products
    int tile_keys = p.S;
    if (p.causal) {
        const int l_hi = (p.L % 128 == 0) ? (int)((tile * 128) % p.L) + 127 : p.L - 1;     // largest query index in the tile
        const int lim = l_hi + 1;
        tile_keys = lim < 0 ? 0 : (lim > p.S ? p.S : lim);
    }
    const int nk = tile_keys <= 0 ? 64 : (tile_keys + 63) / 64 * 64;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(bar_qk, kSmemQ + kSmemK);
            tma_load_2d(smem_u32(sQ), &tmap_q, 0, (int)row0, bar_qk);
            tma_load_2d(smem_u32(sK), &tmap_k, 0, group * p.S, bar_qk);
            mbar_expect_tx(bar_v, kSmemV);
            tma_load_2d(smem_u32(sV), &tmap_v, 0, group * p.S, bar_v);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = mbar_wait(bar_qk, 0, abort_flag, p.status, 51);
            if (ok) {
                tc_fence_after();
                const uint32_t idesc_qk = (p.idesc_qk & ~(0x3fu << 17)) | ((uint32_t)(nk >> 3) << 17);     // N = nk keys
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    umma<false>(tmem_base, make_smem_desc(smem_u32(sQ) + ks * 32, 16, 1024), make_smem_desc(smem_u32(sK) + ks * 32, 16, 1024), idesc_qk,
                                ks > 0 ? 1u : 0u);
                umma_commit(bar_s);
                ok = mbar_wait(bar_p, 0, abort_flag, p.status, 52) && mbar_wait(bar_v, 0, abort_flag, p.status, 53);
            }
            if (ok) {
                tc_fence_after();
#pragma unroll 1
                for (int kb = 0; kb < nk / 64; ++kb) {
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        // A = P, K-major: k-block kb is a [128 x 128 B] tile. B = V, MN-major: 16 keys per step = two 8-row groups.
                        umma<false>(tmem_base, make_smem_desc(smem_u32(sP) + kb * 16384 + ks * 32, 16, 1024),
                                    make_smem_desc(smem_u32(sV) + (kb * 4 + ks) * 2048, 8192, 1024), p.idesc_pv, (kb | ks) ? 1u : 0u);
                    }
                }
                umma_commit(bar_o);
            }
        }
    } else {
        const int lane_window = (warp & 3) * 32;
        const int half = (warp - 2) >> 2;                                  // which of the two warps of this quarter
        const int r = lane_window + lane;                                  // row of the tile
        const int64_t row = row0 + r;
        const int l = (int)(row % p.L);
        const int limit = p.causal ? (l + 1) : p.S;
        const int nvis = limit < 0 ? 0 : (limit > p.S ? p.S : limit);
        const uint32_t trow = tmem_base + ((uint32_t)lane_window << 16);
        bool ok = mbar_wait(bar_s, 0, abort_flag, p.status, 54);
        ok = __all_sync(0xffffffffu, ok);
        // chunks that no row of this warp can see are skipped in both passes (their P is zero); chunks that every row sees
        // in full need no mask
        const int warp_nvis = __reduce_max_sync(0xffffffffu, nvis), warp_full = __reduce_min_sync(0xffffffffu, nvis);
        float m = -INFINITY, sum = 0.f;
        if (ok) {
            tc_fence_after();
#pragma unroll 1
            for (int c0 = half * 32; c0 < kFusedS; c0 += 64) {
                if (c0 >= warp_nvis) break;
                uint32_t v[32];
                tmem_ld32(trow + (uint32_t)c0, v);
                tmem_ld_wait();
                if (c0 + 32 <= warp_full) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) m = fmaxf(m, __uint_as_float(v[j]));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (c0 + j < nvis) m = fmaxf(m, __uint_as_float(v[j]));
                }
            }
        }
        xmax[half * 128 + r] = m;
        asm volatile("bar.sync 1, 256;" ::: "memory");                     // the eight row-math warps
        m = fmaxf(xmax[r], xmax[128 + r]);
        if (ok) {
            const float mscaled = m * p.scale_log2e;
#pragma unroll 1
            for (int c0 = half * 32; c0 < nk; c0 += 64) {
                uint32_t packed[16];
                if (c0 < warp_nvis) {
                    uint32_t v[32];
                    tmem_ld32(trow + (uint32_t)c0, v);
                    tmem_ld_wait();
                    const bool full = c0 + 32 <= warp_full;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float e0 = ex2_approx(fmaf(__uint_as_float(v[2 * j]), p.scale_log2e, -mscaled));
                        float e1 = ex2_approx(fmaf(__uint_as_float(v[2 * j + 1]), p.scale_log2e, -mscaled));
                        if (!full) {
                            e0 = (c0 + 2 * j < nvis) ? e0 : 0.f;
                            e1 = (c0 + 2 * j + 1 < nvis) ? e1 : 0.f;
                        }
                        if (p.dtype == TVK_F16) {
                            const __half2 h = __floats2half2_rn(e0, e1);
                            packed[j] = *(const uint32_t*)&h;
                            const float2 f = __half22float2(h);
                            sum += f.x + f.y;
                        } else {
                            const __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
                            packed[j] = *(const uint32_t*)&h;
                            const float2 f = __bfloat1622float2(h);
                            sum += f.x + f.y;
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) packed[j] = 0u;
                }
                // K-major 128-byte-swizzled A tile: row r, 16-byte chunk c of k-block kb sits at chunk position c ^ (r & 7)
                uint8_t* prow = sP + (c0 >> 6) * 16384 + r * 128;
                const int cbase = (c0 & 63) >> 3;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    *(uint4*)(prow + (((cbase + i) ^ (r & 7)) << 4)) = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the MMA
            tc_fence_before();
        }
        xsum[half * 128 + r] = sum;
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(bar_p);
        asm volatile("bar.sync 1, 256;" ::: "memory");                     // both halves of every row sum are written
        sum = xsum[r] + xsum[128 + r];
        if (ok) {
            ok = mbar_wait(bar_o, 0, abort_flag, p.status, 55);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            tc_fence_after();
            const float inv = nvis > 0 ? 1.0f / sum : 0.f;
            uint16_t* orow = (uint16_t*)p.out + row * 64;
            const int c0 = half * 32;                                      // each half stores 32 of the 64 output columns
            uint32_t v[32];
            tmem_ld32(trow + (uint32_t)c0, v);
            tmem_ld_wait();
            uint32_t packed[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float a = __uint_as_float(v[2 * j]) * inv, b = __uint_as_float(v[2 * j + 1]) * inv;
                if (p.dtype == TVK_F16) { const __half2 h = __floats2half2_rn(a, b); packed[j] = *(const uint32_t*)&h; }
                else { const __nv_bfloat162 h = __floats2bfloat162_rn(a, b); packed[j] = *(const uint32_t*)&h; }
            }
#pragma unroll
            for (int j = 0; j < 16; j += 4) *(uint4*)(orow + c0 + 2 * j) = make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
            // natural-log log-sum-exp of the scaled scores: m*scale + ln(sum)
            if (half == 0) p.lse[row] = nvis > 0 ? m * p.scale + logf(sum) : INFINITY;
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kFusedTmemCols) : "memory");
    }
}

}  // namespace attn
}  // namespace tvk
