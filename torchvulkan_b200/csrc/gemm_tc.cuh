// The tcgen05 GEMM kernel (shared by gemm.cu, which plans and dispatches, and the gemm_tc_*.cu files, which each
// instantiate one family of it): a persistent, warp-specialised kernel.
//   warp 0      TMA producer: cp.async.bulk.tensor tiles of A and B into a ring of 128-byte-swizzled shared-memory
//               stages, completion on mbarriers
//   warp 1      MMA issuer: one lane issues tcgen05.mma (M=128, N=BN, K=32 bytes per step) with the fp32 accumulator in
//               tensor memory (two accumulator sets where they fit, so the epilogue of block i overlaps the main loop of
//               block i+1); tcgen05.commit frees stages
//   warps 2-9   epilogue: tcgen05.ld the accumulator, alpha / beta*bias / activation (and the fused forms), convert, stage
//               in swizzled shared memory, TMA store
// Replaces the matmul_coop shader (src/shaders/ops/matmul_coop.slang:158-223, 364-415).
#pragma once

#include "common.cuh"
#include "tc_common.cuh"

#include <cuda.h>

namespace tvk {
namespace tc {

struct Params {
    int64_t m, n, batch;
    int num_kb;          // k-blocks (128 bytes of K each) per pass
    int passes;          // 1; 3 for the 3xTF32 split
    int chunk_kb;        // fp32 only: k-blocks per tensor-memory accumulation chain
    int a_mn, b_mn;      // operand is MN-major (its M/N index is the contiguous one)
    int a_batched, b_batched;
    int tiles_m, tiles_n;
    int64_t total_tiles;
    uint32_t idesc;
    void* c;
    int64_t c_rs, c_bs;
    const void* bias;
    int64_t bias_rs, bias_cs, bias_bs;
    float alpha, beta;
    int act;
    int out_dtype;
    int* status;
    int stage_ok;        // C (and every peer copy) is 16-byte aligned with 16-byte multiples as row and batch pitch
    int n_peers;         // further copies of C (same strides) in other devices' memory, written by the epilogue
    int tma_store;       // C is written by TMA stores of 32-row x 128-byte boxes staged in shared memory (tmap_c is valid)
    int group_m;         // tile rows per raster group (tm runs fastest inside a group)
    int debug;           // tuning probes: 1 = the epilogue stores nothing, 2 = nothing is loaded or multiplied, 4 = staged tiles are not stored
    void* c2;            // second output with C's strides: C receives the value before the activation, c2 the activated one
    const void* aux;     // per-element operand of C's shape and dtype for aux_op (row pitch aux_rs, batch pitch aux_bs)
    int64_t aux_rs, aux_bs;
    int aux_op;          // TVK_AUX_*: what the epilogue does with aux
    void* peer_c[7];
    // float8 products only (the scaled product): the accumulator of row r, column c is multiplied by
    // row_scale[r * row_scale_stride] * col_scale[c * col_scale_stride] before alpha / bias; null col_scale = no scales
    const float* row_scale;
    const float* col_scale;
    int row_scale_stride, col_scale_stride;
};

// Threads of the GEMM kernel: producer warp, MMA warp and EIGHT epilogue warps. A warp can only read the 32 tensor-memory
// lanes (rows) of its quarter (warp index mod 4), so two warps share each quarter and take alternate column groups:
// reading tensor memory is latency-bound per warp and the epilogue of a block is exposed when a block fills all of it.
constexpr int kEpiWarps = 8;
constexpr int kGemmThreads = 64 + 32 * kEpiWarps;
// Epilogue staging: every epilogue warp owns a 4 KB buffer of 32 rows x 128 bytes in the 128-byte-swizzle layout (chunk j
// of row r sits at chunk j ^ (r & 7)), from where a group of columns leaves as one TMA store, or as whole 128-byte lines
// towards this device's C and the peers' copies.
constexpr int kOutBufBytes = 32 * 128;
constexpr int kGemmStagingBytes = kEpiWarps * kOutBufBytes;       // 32 KB
constexpr int kGemmStageBudget = 192 * 1024;

__device__ __forceinline__ void tma_store_3d(const void* tmap, uint32_t src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(tmap), "r"(src), "r"(c0), "r"(c1),
                 "r"(c2)
                 : "memory");
}

// Stage and tensor-memory sizing of a CTA that owns MT vertically adjacent 128 x BN tiles (a 128*MT x BN block of C).
// With MT = 2 the two tiles share every B stage, so a block of C costs (128*MT + BN) rows of operands from L2 instead of
// MT * (128 + BN): what bounds the weight-streaming and short-K shapes is that fill, not the tensor core.
template <int BN, int MT> struct GemmCfg {
    static constexpr int kStageA = MT * BM * 128;
    static constexpr int kStageB = BN * 128;
    static constexpr int kStage = kStageA + kStageB;
    static constexpr int kStagesRaw = kGemmStageBudget / kStage;
    static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
    static constexpr int kAccBufs = (2 * MT * BN <= 512) ? 2 : 1;       // accumulator sets: two let the epilogue overlap the next block
    static constexpr int kTmemCols = kAccBufs * MT * BN < 32 ? 32 : kAccBufs * MT * BN;
    static constexpr int kSmemBytes = kStages * kStage + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// ---- epilogue building blocks (one output type per instantiation) -----------------------------------------------------
__device__ __forceinline__ float act_apply(float v, int act) {
    if (act == TVK_ACT_RELU) return (v != v) ? v : fmaxf(v, 0.f);
    if (act == TVK_ACT_GELU) return 0.5f * v * (1.0f + erff(v * 0.7071067811865476f));
    return v;
}
// aux_op of the fused epilogues: v is the scaled (and biased) accumulator, x the element of the aux operand.
__device__ __forceinline__ float aux_apply(float v, float x, int op) {
    if (op == TVK_AUX_GELU_BACKWARD) {          // the same expression as the elementwise gelu_backward kernel
        const float cdf = 0.5f * (1.0f + erff(x * 0.7071067811865476f));
        const float pdf = expf(-0.5f * x * x) * 0.3989422804014327f;
        return v * (cdf + x * pdf);
    }
    if (op == TVK_AUX_RELU_BACKWARD) return (x <= 0.f) ? 0.f : v;
    return v;
}

template <int OUT> __device__ __forceinline__ float epi_load(const uint8_t* p, int64_t i) {
    if constexpr (OUT == TVK_F32) return ((const float*)p)[i];
    else if constexpr (OUT == TVK_F16) return __half2float(((const __half*)p)[i]);
    else return __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
template <int OUT> __device__ __forceinline__ uint32_t epi_pack2(float a, float b) {
    if constexpr (OUT == TVK_F16) { const __half2 h = __floats2half2_rn(a, b); return *(const uint32_t*)&h; }
    else { const __nv_bfloat162 h = __floats2bfloat162_rn(a, b); return *(const uint32_t*)&h; }
}
__device__ __forceinline__ void epi_act(float* v, int act) {
    if (act == TVK_ACT_RELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (v[j] != v[j]) ? v[j] : fmaxf(v[j], 0.f);
    } else if (act == TVK_ACT_GELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0.5f * v[j] * (1.0f + erff(v[j] * 0.7071067811865476f));
    }
}
// v = act(alpha * v + beta * bias[cbase + j]) for the 32 columns of one row starting at column cbase (ncols of them exist).
// brow: the bias row of this output row (bytes), element stride bias_cs.
template <int OUT>
__device__ __forceinline__ void epi_scale_bias_act(float* v, float alpha, float beta, const uint8_t* brow, int64_t bias_cs, int64_t cbase, int ncols, int act) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = alpha * v[j];
    if (brow) {
        if (bias_cs == 0) {                              // one value per output row
            const float bv = beta * epi_load<OUT>(brow, 0);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += bv;
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < ncols) v[j] += beta * epi_load<OUT>(brow, (cbase + j) * bias_cs);
        }
    }
    if (act != TVK_ACT_NONE) epi_act(v, act);
}
// The factors the aux operation multiplies columns [c, c + 32) of one row by, as 16 packed half pairs: they depend on aux
// alone, so they are formed before the accumulator is ready (gelu'(x) lies in [-0.13, 1.13]: half precision keeps 11 bits
// of it, the precision of the result that is stored).
template <int OUT>
__device__ __forceinline__ void epi_aux_factors(const uint8_t* arow, int64_t c, int64_t n, int aux_op, uint32_t* a2) {
    const int ncols = (n - c) < 32 ? (int)(n - c) : 32;
    const uint16_t* ap = (const uint16_t*)arow + c;
    if (ncols == 32 && ((uintptr_t)ap & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 q = __ldg((const uint4*)ap + j);
            a2[4 * j] = q.x; a2[4 * j + 1] = q.y; a2[4 * j + 2] = q.z; a2[4 * j + 3] = q.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t lo = (2 * j < ncols) ? ap[2 * j] : 0u, hi = (2 * j + 1 < ncols) ? ap[2 * j + 1] : 0u;
            a2[j] = lo | (hi << 16);
        }
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        float x0, x1;
        if constexpr (OUT == TVK_F16) { const float2 f = __half22float2(*(const __half2*)&a2[j]); x0 = f.x; x1 = f.y; }
        else { const float2 f = __bfloat1622float2(*(const __nv_bfloat162*)&a2[j]); x0 = f.x; x1 = f.y; }
        const __half2 h = __floats2half2_rn(aux_apply(1.0f, x0, aux_op), aux_apply(1.0f, x1, aux_op));
        a2[j] = *(const uint32_t*)&h;
    }
}
// 32 finished columns of one row into the warp's staging buffer: `mine` is this lane's 128-byte row, sw = lane & 7 the
// swizzle of that row, cin the first of the 32 columns within the 128-byte group.
template <int OUT>
__device__ __forceinline__ void epi_stage(uint8_t* mine, int sw, int cin, const float* v) {
    if constexpr (OUT == TVK_F32) {
#pragma unroll
        for (int j = 0; j < 8; ++j) *(float4*)(mine + ((j ^ sw) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
        const int j0 = cin >> 3;   // first 16-byte chunk of these 32 columns within the row
#pragma unroll
        for (int j = 0; j < 4; ++j)
            *(uint4*)(mine + (((j0 + j) ^ sw) << 4)) = make_uint4(epi_pack2<OUT>(v[8 * j], v[8 * j + 1]), epi_pack2<OUT>(v[8 * j + 2], v[8 * j + 3]),
                                                                   epi_pack2<OUT>(v[8 * j + 4], v[8 * j + 5]), epi_pack2<OUT>(v[8 * j + 6], v[8 * j + 7]));
    }
}
// Conversion and store of 32 columns of one row straight from registers (any n, any alignment). crow: byte address of the
// row's first column in the destination.
template <int OUT>
__device__ __forceinline__ void epi_store_direct(const float* v, uint8_t* crow, int64_t cbase, int ncols) {
    if constexpr (OUT == TVK_F32) {
        float* dst = (float*)crow + cbase;
        if (ncols == 32 && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) *(float4*)(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) if (j < ncols) dst[j] = v[j];
        }
    } else {
        uint16_t* dst = (uint16_t*)crow + cbase;
        if (ncols == 32 && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                *(uint4*)(dst + 8 * j) = make_uint4(epi_pack2<OUT>(v[8 * j], v[8 * j + 1]), epi_pack2<OUT>(v[8 * j + 2], v[8 * j + 3]),
                                                    epi_pack2<OUT>(v[8 * j + 4], v[8 * j + 5]), epi_pack2<OUT>(v[8 * j + 6], v[8 * j + 7]));
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (j < ncols) {
                    const uint32_t pk = epi_pack2<OUT>(v[j], 0.f);
                    dst[j] = (uint16_t)(pk & 0xffffu);
                }
            }
        }
    }
}

// ES = operand element size in bytes (2: f16/bf16, 4: tf32). MT = 128-row tiles per CTA block (1 or 2). OUT = dtype of C
// (TVK_F16 / TVK_BF16 / TVK_F32). FUSED = the epilogue also handles a second output and an aux operand.
// OUT and FUSED are compile-time so that the epilogue's loop holds one straight path: with the output type, the fused
// forms and every fallback selected at run time inside that loop it ran several times slower than the same arithmetic
// in a small loop (measured: 1900 against 280 clocks per 32-column chunk), i.e. it was bound by instruction fetch.
template <int BN, int ES, int MT, int OUT, bool FUSED>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a0, const __grid_constant__ CUtensorMap tmap_a1,
            const __grid_constant__ CUtensorMap tmap_b0, const __grid_constant__ CUtensorMap tmap_b1,
            const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_c2, const Params p) {
    using Cfg = GemmCfg<BN, MT>;
    constexpr int BK = 128 / ES;         // elements of K per stage
    constexpr int CH = 128 / ES;         // elements of M/N per 128-byte row of an MN-major tile
    constexpr int kStages = Cfg::kStages;
    constexpr bool kChunked = (ES == 4) && (BN <= 64);     // fp32: chains of K summed in registers (below)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* outbuf = smem + kStages * Cfg::kStage;                    // 1024-byte aligned: the stages are multiples of 1 KB
    uint64_t* bars = (uint64_t*)(outbuf + kGemmStagingBytes);
    // bars: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * kStages + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kStages);
    const uint32_t tfull0 = smem_u32(bars + 2 * kStages), tempty0 = smem_u32(bars + 2 * kStages + 2);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull0 + 8 * a, 1);
            mbar_init(tempty0 + 8 * a, kChunked ? 4 : kEpiWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0 && lane == 0) {
        // the descriptors are fetched while the barriers and tensor memory are being set up
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a0) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b0) : "memory");
        if (p.passes > 1) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a1) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b1) : "memory");
        }
        if (p.tma_store) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_c) : "memory");
        if (p.tma_store && p.c2) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_c2) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)Cfg::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // fp32 (3xTF32): K is cut into chunks of p.chunk_kb k-blocks, every chunk is one accumulation
    // chain in tensor memory (small lo terms first, hi*hi last) and the epilogue warps sum the
    // chunks in registers. Half types: one chain over all of K.
    static_assert(!(kChunked && MT != 1), "the chunked fp32 epilogue handles one tile per block");
    constexpr int kAccBufs = Cfg::kAccBufs;
    // accumulator set and mbarrier parity of the it-th accumulation of this CTA
    auto acc_of = [&](int64_t it) { return kAccBufs == 2 ? (int)(it & 1) : 0; };
    auto acc_phase_of = [&](int64_t it) { return (uint32_t)((kAccBufs == 2 ? (it >> 1) : it) & 1); };
    const int ckb = kChunked ? p.chunk_kb : p.num_kb;
    auto pass_of = [&](int pi) { return kChunked ? (pi == 0 ? 1 : (pi == 1 ? 2 : 0)) : pi; };
    // Tile index arithmetic in 32 bits (the host refuses launches with 2^31 tiles or more): a 64-bit division costs several
    // hundred clocks, and this runs once per tile in every role.
    const uint32_t tiles_per_batch = (uint32_t)(p.tiles_m * p.tiles_n);
    const uint32_t total_tiles = (uint32_t)p.total_tiles;
    auto decode = [&](uint32_t t, int& b, int& tm, int& tn) {
        const uint32_t bb = t / tiles_per_batch;
        const uint32_t r = t - bb * tiles_per_batch;
        const uint32_t group = (uint32_t)(p.group_m * p.tiles_n);
        const uint32_t g = r / group, rr = r - g * group;
        const uint32_t first_m = g * (uint32_t)p.group_m;
        const uint32_t left = (uint32_t)p.tiles_m - first_m;
        const uint32_t gm = left < (uint32_t)p.group_m ? left : (uint32_t)p.group_m;
        const uint32_t q = rr / gm;
        b = (int)bb;
        tm = (int)(first_m + (rr - q * gm));
        tn = (int)q;
    };

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; t < total_tiles && ok && !(p.debug & 2); t += gridDim.x) {
                int b, tm, tn;
                decode(t, b, tm, tn);
                const int ab = p.a_batched ? b : 0, bb = p.b_batched ? b : 0;
                for (int kb0 = 0; kb0 < p.num_kb && ok; kb0 += ckb) {
                    const int kb1 = (kb0 + ckb) < p.num_kb ? (kb0 + ckb) : p.num_kb;
                    for (int pi = 0; pi < p.passes && ok; ++pi) {
                        const int pass = pass_of(pi);
                        const void* ta = (pass == 1) ? (const void*)&tmap_a1 : (const void*)&tmap_a0;
                        const void* tb = (pass == 2) ? (const void*)&tmap_b1 : (const void*)&tmap_b0;
                        for (int kb = kb0; kb < kb1; ++kb) {
                            ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.status, 1);
                            if (!ok) break;
                            const uint32_t sa = smem_u32(smem + stage * Cfg::kStage);
                            const uint32_t sb = sa + Cfg::kStageA;
                            const uint32_t bar = full0 + 8 * stage;
                            mbar_expect_tx(bar, Cfg::kStage);
                            if (!p.a_mn) {
                                tma_load_3d(sa, ta, kb * BK, tm * (MT * BM), ab, bar);
                            } else {
#pragma unroll
                                for (int j = 0; j < MT * BM / CH; ++j) tma_load_3d(sa + j * (BK * 128), ta, tm * (MT * BM) + j * CH, kb * BK, ab, bar);
                            }
                            if (!p.b_mn) {
                                tma_load_3d(sb, tb, kb * BK, tn * BN, bb, bar);
                            } else {
#pragma unroll
                                for (int j = 0; j < BN / CH; ++j) tma_load_3d(sb + j * (BK * 128), tb, tn * BN + j * CH, kb * BK, bb, bar);
                            }
                            if (++stage == kStages) { stage = 0; phase ^= 1; }
                        }
                    }
                }
            }
            if (ok) {
                // Drain: wait until the MMA warp has released every stage this thread filled, so no
                // copy is still in flight towards shared memory when the CTA exits.
                for (int s = 0; s < kStages && ok; ++s) {
                    ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.status, 2);
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int64_t it = 0;
            // Per k-step advance of the descriptor start address, and the LBO/SBO fields.
            const uint32_t a_step = p.a_mn ? (uint32_t)((32 / ES) * 128) : 32u;
            const uint32_t b_step = p.b_mn ? (uint32_t)((32 / ES) * 128) : 32u;
            // MN-major: LBO is the distance between 128-byte-wide column blocks of the tile, SBO the
            // distance between groups of eight k-rows. K-major: LBO is unused, SBO spans eight rows.
            const uint32_t a_lbo = p.a_mn ? (uint32_t)(BK * 128) : 16u, a_sbo = 1024u;
            const uint32_t b_lbo = p.b_mn ? (uint32_t)(BK * 128) : 16u, b_sbo = 1024u;
            for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                for (int kb0 = 0; kb0 < p.num_kb && ok; kb0 += ckb, ++it) {
                    const int kb1 = (kb0 + ckb) < p.num_kb ? (kb0 + ckb) : p.num_kb;
                    const int acc = acc_of(it);
                    const uint32_t acc_phase = acc_phase_of(it);
                    ok = mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1, abort_flag, p.status, 3);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t tmem_c = tmem_base + (uint32_t)(acc * MT * BN);
                    uint32_t accumulate = 0;
                    for (int pi = 0; pi < p.passes && ok && !(p.debug & 2); ++pi) {
                        for (int kb = kb0; kb < kb1; ++kb) {
                            ok = mbar_wait(full0 + 8 * stage, phase, abort_flag, p.status, 4);
                            if (!ok) break;
                            tc_fence_after();
                            const uint32_t sa = smem_u32(smem + stage * Cfg::kStage);
                            const uint32_t sb = sa + Cfg::kStageA;
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks) {
                                const uint64_t bdesc = make_smem_desc(sb + ks * b_step, b_lbo, b_sbo);
#pragma unroll
                                for (int mt = 0; mt < MT; ++mt) {
                                    // tile mt of the block: its 128 rows (K-major) or its column blocks (MN-major) start BM*128 bytes on
                                    const uint64_t adesc = make_smem_desc(sa + mt * (BM * 128) + ks * a_step, a_lbo, a_sbo);
                                    if constexpr (ES == 1) umma_f8(tmem_c + (uint32_t)(mt * BN), adesc, bdesc, p.idesc, accumulate);
                                    else umma<ES == 4>(tmem_c + (uint32_t)(mt * BN), adesc, bdesc, p.idesc, accumulate);
                                }
                                accumulate = 1;
                            }
                            umma_commit(empty0 + 8 * stage);
                            if (++stage == kStages) { stage = 0; phase ^= 1; }
                        }
                    }
                    if (ok) umma_commit(tfull0 + 8 * acc);
                }
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        constexpr int kEsOut = (OUT == TVK_F32) ? 4 : 2;
        constexpr int gcols = 128 / kEsOut;                  // columns of C in 128 bytes
        constexpr bool kBoxes = (BN % gcols == 0);           // the block is made of whole 128-byte column groups
        const int lane_window = (warp & 3) * 32;   // TMEM lanes this warp may read
        const int half = (warp - 2) >> 2;          // which of the two warps of this quarter: it takes column groups of its parity
        uint8_t* buf = outbuf + (warp - 2) * kOutBufBytes;               // this warp's staging rows
        bool ok = true;
        int64_t it = 0;
        for (uint32_t t = blockIdx.x; t < total_tiles && ok && !(kChunked && half); t += gridDim.x) {
            int b, tm, tn;
            decode(t, b, tm, tn);
            int acc = 0;
            uint32_t acc_phase = 0;
            if constexpr (!kChunked) {
                // (the wait for this accumulator set sits inside the loop below, after the first aux loads are issued)
                acc = acc_of(it);
                acc_phase = acc_phase_of(it);
                ++it;
            }
#pragma unroll 1
            for (int mt = 0; mt < MT; ++mt) {
                const int64_t tile_row0 = ((int64_t)tm * MT + mt) * BM;
                if (mt > 0 && tile_row0 >= p.m) break;      // the lower tile of the last block may lie wholly below C
                const int64_t row = tile_row0 + lane_window + lane;
                const int64_t col0 = (int64_t)tn * BN;
                const bool row_ok = row < p.m;
                const int64_t coff = ((int64_t)b * p.c_bs + row * p.c_rs) * kEsOut;   // byte offset of this row in C
                const uint8_t* brow = p.bias ? (const uint8_t*)p.bias + ((int64_t)b * p.bias_bs + row * p.bias_rs) * kEsOut : nullptr;
                const uint8_t* arow = nullptr;
                if constexpr (FUSED) {
                    if (p.aux_op) arow = (const uint8_t*)p.aux + ((int64_t)b * p.aux_bs + row * p.aux_rs) * 2;
                }

                if constexpr (kChunked) {
                    // The tensor core adds into its accumulator with truncation, so a long chain of MMAs
                    // drifts by about one ulp per step. Each chunk of K is therefore accumulated from zero
                    // in tensor memory and the chunks are summed here in registers with round-to-nearest.
                    float sum[BN];
#pragma unroll
                    for (int j = 0; j < BN; ++j) sum[j] = 0.f;
                    for (int kb0 = 0; kb0 < p.num_kb && ok; kb0 += ckb, ++it) {
                        const int cacc = (int)(it & 1);
                        const uint32_t cphase = (uint32_t)((it >> 1) & 1);
                        ok = mbar_wait(tfull0 + 8 * cacc, cphase, abort_flag, p.status, 5);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll
                        for (int c0 = 0; c0 < BN; c0 += 32) {
                            uint32_t r[32];
                            tmem_ld32(tmem_base + ((uint32_t)lane_window << 16) + (uint32_t)(cacc * BN + c0), r);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 32; ++j) sum[c0 + j] += __uint_as_float(r[j]);
                        }
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tempty0 + 8 * cacc);
                    }
                    if (!ok) break;
#pragma unroll
                    for (int c0 = 0; c0 < BN; c0 += 32) {
                        if (col0 + c0 < p.n && row_ok) {
                            const int ncols = (p.n - col0 - c0) < 32 ? (int)(p.n - col0 - c0) : 32;
                            epi_scale_bias_act<OUT>(&sum[c0], p.alpha, p.beta, brow, p.bias_cs, col0 + c0, ncols, p.act);
                            epi_store_direct<OUT>(&sum[c0], (uint8_t*)p.c + coff, col0 + c0, ncols);
                        }
                    }
                } else {
                    const bool staged = kBoxes && (p.tma_store || p.stage_ok);
                    const uint32_t tacc = tmem_base + ((uint32_t)lane_window << 16) + (uint32_t)((acc * MT + mt) * BN);
                    // With a second output the accumulator is read twice: first for C (no activation), then for c2 (activated).
                    const int n_out = (FUSED && p.c2) ? 2 : 1;
                    // this warp's chunks of 32 columns in order: both chunks of every column group of its parity (the other warp
                    // of the quarter takes the other groups)
                    auto next_chunk = [&](int c0) {
                        int c = c0 + 32;
                        if (gcols == 32 || (c % gcols) == 0) c += gcols;
                        return c;
                    };
                    const int c_first = half * gcols;
#pragma unroll 1
                    for (int which = 0; which < n_out; ++which) {
                        uint32_t acur[16], anext[16];
                        if constexpr (FUSED) {
                            if (arow && row_ok && c_first < BN && col0 + c_first < p.n) {
                                epi_aux_factors<OUT>(arow, col0 + c_first, p.n, p.aux_op, acur);
                                const int c2nd = next_chunk(c_first);
                                if (c2nd < BN && col0 + c2nd < p.n) epi_aux_factors<OUT>(arow, col0 + c2nd, p.n, p.aux_op, anext);
                            }
                        }
                        if (mt == 0 && which == 0) {
                            // (the first aux factors are formed while this warp would otherwise wait for the accumulator)
                            ok = mbar_wait(tfull0 + 8 * acc, acc_phase, abort_flag, p.status, 5);
                            ok = __all_sync(0xffffffffu, ok);
                            if (!ok) break;
                            tc_fence_after();
                        }
                        uint8_t* cbase_ptr = (FUSED && which) ? (uint8_t*)p.c2 : (uint8_t*)p.c;
                        const void* tm_out = (FUSED && which) ? (const void*)&tmap_c2 : (const void*)&tmap_c;
#pragma unroll 1
                        for (int c0 = c_first; c0 < BN; c0 = next_chunk(c0)) {
                            if (col0 + c0 >= p.n) break;                   // uniform across the warp
                            const int64_t cbase = col0 + c0;
                            const int ncols = (p.n - cbase) < 32 ? (int)(p.n - cbase) : 32;
                            uint32_t r[32];
                            tmem_ld32(tacc + (uint32_t)c0, r);
                            tmem_ld_wait();
                            float v[32];
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                            if (row_ok) {
                                if constexpr (ES == 1) {
                                    if (p.col_scale) {
                                        const float rsc = __ldg(p.row_scale + row * p.row_scale_stride);
                                        if (p.col_scale_stride == 0) {
                                            const float sc = rsc * __ldg(p.col_scale);
#pragma unroll
                                            for (int j = 0; j < 32; ++j) v[j] *= sc;
                                        } else {
#pragma unroll
                                            for (int j = 0; j < 32; ++j)
                                                if (j < ncols) v[j] *= rsc * __ldg(p.col_scale + cbase + j);
                                        }
                                    }
                                }
                                if constexpr (FUSED) {
                                    epi_scale_bias_act<OUT>(v, p.alpha, p.beta, brow, p.bias_cs, cbase, ncols, TVK_ACT_NONE);
                                    if (arow) {
                                        // the incoming gradient times the derivative of the activation at the saved pre-activation
#pragma unroll
                                        for (int j = 0; j < 16; ++j) {
                                            const float2 f = __half22float2(*(const __half2*)&acur[j]);
                                            v[2 * j] *= f.x;
                                            v[2 * j + 1] *= f.y;
                                        }
                                    }
                                    if (which == n_out - 1) epi_act(v, p.act);
                                } else {
                                    epi_scale_bias_act<OUT>(v, p.alpha, p.beta, brow, p.bias_cs, cbase, ncols, p.act);
                                }
                            }
                            if constexpr (FUSED) {
                                // the factors stay two chunks ahead of the accumulator reads
#pragma unroll
                                for (int j = 0; j < 16; ++j) acur[j] = anext[j];
                                const int cn2 = next_chunk(next_chunk(c0));
                                if (arow && row_ok && cn2 < BN && col0 + cn2 < p.n) epi_aux_factors<OUT>(arow, col0 + cn2, p.n, p.aux_op, anext);
                            }
                            if (p.debug & 1) continue;
                            const int g0 = c0 / gcols * gcols;
                            // Groups of 128 bytes per row go through this warp's staging rows and leave as one TMA store (which clips
                            // rows >= m and columns >= n) or, towards peers, as whole 128-byte lines (whole groups only).
                            if (!staged || (!p.tma_store && col0 + g0 + gcols > p.n)) {
                                if (row_ok) {
                                    epi_store_direct<OUT>(v, cbase_ptr + coff, cbase, ncols);
                                    if (!(FUSED && which))
                                        for (int q = 0; q < p.n_peers; ++q) epi_store_direct<OUT>(v, (uint8_t*)p.peer_c[q] + coff, cbase, ncols);
                                }
                                continue;
                            }
                            if (c0 == g0 && p.tma_store) {
                                // the previous store of this warp must have finished reading the buffer
                                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                                __syncwarp();
                            }
                            epi_stage<OUT>(buf + lane * 128, lane & 7, c0 - g0, v);
                            if (!(c0 + 32 == g0 + gcols || (p.tma_store && cbase + 32 >= p.n))) continue;
                            if (p.tma_store) {
                                if (p.debug & 4) continue;                   // probe: staged, never stored
                                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                                __syncwarp();
                                if (lane == 0 && tile_row0 + lane_window < p.m) {
                                    tma_store_3d(tm_out, smem_u32(buf), (int)(col0 + g0), (int)(tile_row0 + lane_window), b);
                                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                                }
                                continue;
                            }
                            // whole 128-byte lines towards this device's C and the peers' copies (the pushed all-gather)
                            __syncwarp();
                            uint4 line[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int rr = 4 * i + (lane >> 3);
                                line[i] = *(const uint4*)(buf + rr * 128 + ((((lane & 7) ^ (rr & 7))) << 4));
                            }
                            const int64_t row0 = tile_row0 + lane_window;
                            const int64_t off0 = ((int64_t)b * p.c_bs + row0 * p.c_rs + col0 + g0) * kEsOut + (lane & 7) * 16;
                            const int64_t row_bytes = p.c_rs * kEsOut;
                            const int np = (FUSED && which) ? 0 : p.n_peers;
                            // qi == -1 is this device's C; the others push the same lines into the peers' copies over NVLink,
                            // every CTA starting at another peer so that 148 CTAs do not all write to one GPU at a time
                            const int rot = np > 0 ? (int)((blockIdx.x + (unsigned)warp) % (unsigned)np) : 0;
                            for (int qi = -1; qi < np; ++qi) {
                                const int q = qi < 0 ? -1 : (qi + rot >= np ? qi + rot - np : qi + rot);
                                uint8_t* base = (q < 0 ? cbase_ptr : (uint8_t*)p.peer_c[q]) + off0;
#pragma unroll
                                for (int i = 0; i < 8; ++i) {
                                    const int rr = 4 * i + (lane >> 3);
                                    if (row0 + rr < p.m) *(uint4*)(base + rr * row_bytes) = line[i];
                                }
                            }
                            __syncwarp();
                        }
                    }
                    if (!ok) break;
                }
            }   // mt
            if constexpr (!kChunked) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
            }
        }
        // every TMA store of this warp has finished reading its staging rows before shared memory is handed back (the
        // writes themselves complete with the grid)
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }

    // ------------------------------ teardown ------------------------------
    __syncwarp();
    if (*abort_flag) {
        // Let copies and MMAs that were already issued finish before shared and tensor memory
        // are handed back.
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::kTmemCols) : "memory");
    }
}

template <int BN, int ES, int MT, int OUT, bool FUSED>
static int launch(const CUtensorMap* maps, const Params& p, cudaStream_t s) {
    using Cfg = GemmCfg<BN, MT>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        TVK_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<BN, ES, MT, OUT, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes + kGemmStagingBytes));
        attr_set[dev] = true;
    }
    int64_t grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
    gemm_kernel<BN, ES, MT, OUT, FUSED><<<(unsigned)grid, kGemmThreads, Cfg::kSmemBytes + kGemmStagingBytes, s>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], p);
    return launch_status("tcgen05 gemm");
}

// One family = one (operand size, output type, fused) combination over every block shape; each family is compiled in a
// translation unit of its own (gemm_tc_*.cu) so that they build in parallel.
template <int ES, int OUT, bool FUSED>
static int launch_family(int bn, int mt, const CUtensorMap* maps, const Params& p, cudaStream_t s) {
    if constexpr (ES == 4) {
        if (bn >= 64) return launch<64, 4, 1, OUT, FUSED>(maps, p, s);
        return launch<32, 4, 1, OUT, FUSED>(maps, p, s);
    } else {
        switch (bn) {
            case 256: return mt == 2 ? launch<256, ES, 2, OUT, FUSED>(maps, p, s) : launch<256, ES, 1, OUT, FUSED>(maps, p, s);
            case 128: return mt == 2 ? launch<128, ES, 2, OUT, FUSED>(maps, p, s) : launch<128, ES, 1, OUT, FUSED>(maps, p, s);
            case 64: return mt == 2 ? launch<64, ES, 2, OUT, FUSED>(maps, p, s) : launch<64, ES, 1, OUT, FUSED>(maps, p, s);
            case 32: return mt == 2 ? launch<32, ES, 2, OUT, FUSED>(maps, p, s) : launch<32, ES, 1, OUT, FUSED>(maps, p, s);
        }
        return set_error(TVK_ERR_INVALID, "tvk_gemm: internal tile selection error");
    }
}

// Defined one per translation unit (gemm_tc_*.cu). bn in {32, 64, 128, 256}, mt in {1, 2}.
int launch_f16(int bn, int mt, const CUtensorMap* maps, const Params& p, cudaStream_t s);
int launch_f16_fused(int bn, int mt, const CUtensorMap* maps, const Params& p, cudaStream_t s);
int launch_bf16(int bn, int mt, const CUtensorMap* maps, const Params& p, cudaStream_t s);
int launch_bf16_fused(int bn, int mt, const CUtensorMap* maps, const Params& p, cudaStream_t s);
int launch_half_f32out(int bn, int mt, const CUtensorMap* maps, const Params& p, cudaStream_t s);   // f16/bf16 operands, fp32 C
int launch_tf32(int bn, int mt, const CUtensorMap* maps, const Params& p, cudaStream_t s);          // 3xTF32
int launch_f8_f32out(int bn, int mt, const CUtensorMap* maps, const Params& p, cudaStream_t s);     // float8 operands (kind::f8f6f4), fp32 C
int launch_f8_f16out(int bn, int mt, const CUtensorMap* maps, const Params& p, cudaStream_t s);     // float8 operands, fp16 C
int launch_f8_bf16out(int bn, int mt, const CUtensorMap* maps, const Params& p, cudaStream_t s);    // float8 operands, bf16 C

// K-sliced product on CTA pairs (gemm_tc_2sm.cu): 256 x 256 tiles of fp32 partial sums, one per pair and K slice.
struct Params2sm;
int launch_pair(bool a_mn, bool b_mn, const CUtensorMap* maps, int64_t m, int64_t n, int num_kb, int splits, uint32_t idesc, float* partial, int* status, int debug, cudaStream_t s);

}  // namespace tc
}  // namespace tvk
