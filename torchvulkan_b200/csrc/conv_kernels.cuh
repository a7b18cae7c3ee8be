// Device code of the implicit-GEMM convolution (used by conv.cu): layout transposes, weight
// packing, and the two tcgen05 kernels.
//
// Activations are staged channels-last ([N, H, W, C], C padded to a multiple of 64) so that one TMA
// box {64 channels, tw, th, tn} is exactly one 128-byte-swizzled K-major operand tile: the pixel
// (n, h, w) is the row, the 64 channels are the 128 contraction bytes. A filter tap only shifts the
// start coordinate of the box on the W and H axes (outer dimensions, so the 16-byte rule on the
// innermost coordinate always holds), padding is the TMA's out-of-bounds zero fill, and a stride-2
// convolution is the box's element stride. No im2col buffer exists anywhere.
#pragma once

#include "tc_common.cuh"

namespace tvk {
namespace conv {

constexpr int kMaxTaps = 64;

// ---- layout helpers ---------------------------------------------------------------------
// src [N, C, HW] -> dst [N, HW, Cp] (channels >= C written as zero). grid (ceil(HW/32), ceil(Cp/32), N), block (32, 8)
template <typename T>
__global__ void nchw_to_nhwc_kernel(T* __restrict__ dst, const T* __restrict__ src, int C, int HW, int Cp) {
    __shared__ T tile[32][33];
    const int n = blockIdx.z;
    const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int c = c0 + j, p = p0 + threadIdx.x;
        T v = T(0);
        if (c < C && p < HW) v = src[((int64_t)n * C + c) * HW + p];
        tile[j][threadIdx.x] = v;
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int p = p0 + j, c = c0 + threadIdx.x;
        if (p < HW && c < Cp) dst[((int64_t)n * HW + p) * Cp + c] = tile[threadIdx.x][j];
    }
}

// The same move in 16-byte packets for 16-bit elements, HW a multiple of 8 and 16-byte aligned buffers: a CTA of 256 threads
// carries a tile of 64 channels x 64 pixels through shared memory. It reads eight pixels of one channel per load, scatters
// them into a [pixel][channel] tile whose 16-byte channel packets are XOR-swizzled by the pixel's packet index (so the eight
// lanes that hold the same channels of different pixel packets hit different banks), and writes eight channels of one pixel
// per store. Channels >= C come out as zero. grid (ceil(HW/64), ceil(Cp/64), N).
__global__ void __launch_bounds__(256) nchw_to_nhwc_packet_kernel(uint16_t* __restrict__ dst, const uint16_t* __restrict__ src, int C, int HW, int Cp) {
    __shared__ __align__(16) uint16_t tile[64 * 64];
    const int n = blockIdx.z;
    const int p0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int idx = threadIdx.x + 256 * k;
        const int c = idx >> 3, pp = idx & 7;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (c0 + c < C && p0 + pp * 8 < HW) v = __ldcs((const uint4*)(src + ((int64_t)n * C + c0 + c) * HW + p0 + pp * 8));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        const int col = ((((c >> 3) ^ pp) & 7) << 3) + (c & 7);
#pragma unroll
        for (int j = 0; j < 8; ++j) tile[(pp * 8 + j) * 64 + col] = (uint16_t)((j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xffffu));
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int idx = threadIdx.x + 256 * k;
        const int p = idx >> 3, cpk = idx & 7;
        if (p0 + p < HW && c0 + cpk * 8 < Cp) {
            const uint4 v = *(const uint4*)(tile + p * 64 + (((cpk ^ (p >> 3)) & 7) << 3));
            __stcs((uint4*)(dst + ((int64_t)n * HW + p0 + p) * Cp + c0 + cpk * 8), v);
        }
    }
}

// src [N, HW, Cp] -> dst [N, C, HW]. grid (ceil(HW/32), ceil(C/32), N), block (32, 8)
template <typename T>
__global__ void nhwc_to_nchw_kernel(T* __restrict__ dst, const T* __restrict__ src, int C, int HW, int Cp) {
    __shared__ T tile[32][33];
    const int n = blockIdx.z;
    const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int p = p0 + j, c = c0 + threadIdx.x;
        T v = T(0);
        if (p < HW && c < C) v = src[((int64_t)n * HW + p) * Cp + c];
        tile[j][threadIdx.x] = v;
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int c = c0 + j, p = p0 + threadIdx.x;
        if (c < C && p < HW) dst[((int64_t)n * C + c) * HW + p] = tile[threadIdx.x][j];
    }
}

// Filters OIHW [O, I, T] (T = KH*KW) -> [O, T, Ip] (forward operand, contraction over (tap, i)) when
// transposed == 0, or -> [I, T, Op] (input-gradient operand, contraction over (tap, o)) when 1.
// The source is OIHW (src_channels_last == 0) or the same shape in channels-last memory, [O, T, I].
template <typename T>
__global__ void pack_filter_kernel(T* __restrict__ dst, const T* __restrict__ src, int O, int I, int taps, int pad_to, int transposed,
                                   int src_channels_last) {
    const int64_t rows = transposed ? I : O, inner = transposed ? O : I;
    const int64_t total = rows * taps * pad_to;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t c = idx % pad_to, t = (idx / pad_to) % taps, r = idx / ((int64_t)pad_to * taps);
        T v = T(0);
        if (c < inner) {
            const int64_t o = transposed ? c : r, i = transposed ? r : c;
            v = src_channels_last ? src[(o * taps + t) * I + i] : src[(o * I + i) * taps + t];
        }
        dst[idx] = v;
    }
}

// [rows, C] -> [rows, Cp] with zero channels appended (channels-last input whose channel count is not a multiple of 8)
template <typename T>
__global__ void pad_channels_kernel(T* __restrict__ dst, const T* __restrict__ src, int64_t rows, int C, int Cp) {
    const int64_t total = rows * Cp;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = idx / Cp;
        const int c = (int)(idx - r * Cp);
        dst[idx] = c < C ? src[r * C + c] : T(0);
    }
}

// partial fp32 [splits][taps][O][Ip] -> dw OIHW [O, I, taps] (or channels-last [O, taps, I]) in T. Threads walk the
// partials in their own memory order (input channel fastest), so the reads of each slice are coalesced, and the loads of
// eight slices are issued together before they are added in slice order (a dependent load-add chain over up to 64 slices,
// with one 4-byte value used per 32-byte sector, made this kernel 11-16 us for a 64x64x3x3 filter).
template <typename T>
__global__ void wgrad_finalize_kernel(T* __restrict__ dw, const float* __restrict__ partial, int splits, int taps, int O, int I, int Ip,
                                      int dst_channels_last) {
    const int64_t total = (int64_t)taps * O * I, slice = (int64_t)taps * O * Ip;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = idx % I, o = (idx / I) % O, t = idx / ((int64_t)I * O);
        const float* src = partial + (t * O + o) * Ip + i;
        float s = 0.f;
        int k = 0;
        for (; k + 8 <= splits; k += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = src[(int64_t)(k + u) * slice];
#pragma unroll
            for (int u = 0; u < 8; ++u) s += v[u];
        }
        for (; k < splits; ++k) s += src[(int64_t)k * slice];
        const int64_t dst = dst_channels_last ? ((o * taps + t) * I + i) : ((o * I + i) * taps + t);
        dw[dst] = from_f32<T>(s);
    }
}

// ---- forward / input-gradient kernel --------------------------------------------------------
struct FwdParams {
    // tile grid over the output pixels (n, ho, wo) this launch produces, and over output channels
    int tn, th, tw;                  // tile shape, tn*th*tw == 128, powers of two
    int tiles_w, tiles_h, tiles_n, tiles_c;
    int64_t total_tiles;
    int Nimg, Ho, Wo;                // extent of the pixel grid covered by this launch
    int in_stride;                   // input coordinate = pixel coordinate * in_stride + tap offset
    int ntaps, cblocks;              // contraction = ntaps x cblocks blocks of 64 channels
    int8_t dh[kMaxTaps], dw[kMaxTaps];
    int16_t wtap[kMaxTaps];          // index of the tap inside the packed filter (k offset = wtap * cblocks * 64)
    // output addressing: pixel (n, ho, wo), channel c -> out[((n*OH + ho*os + oh0)*OW + wo*os + ow0)*OC + c]
    // with out_nchw set: out[((n*Cout + c)*OH + ho*os + oh0)*OW + wo*os + ow0], the caller's own NCHW tensor
    int OH, OW, os, oh0, ow0, OC, Cout;
    void* out;
    int out_nchw;
    int dtype;
    uint32_t idesc;
    int* status;
};

template <int BN>
__global__ void __launch_bounds__(tc::kThreads, 1)
conv_fwd_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, const FwdParams p) {
    using namespace tc;
    using Cfg = Config<BN>;
    constexpr int kStages = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + kStages * Cfg::kStage);
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * kStages + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kStages);
    const uint32_t tfull0 = smem_u32(bars + 2 * kStages), tempty0 = smem_u32(bars + 2 * kStages + 2);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)Cfg::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto decode = [&](int64_t t, int& tcx, int& twx, int& thx, int& tnx) {
        tcx = (int)(t % p.tiles_c); t /= p.tiles_c;
        twx = (int)(t % p.tiles_w); t /= p.tiles_w;
        thx = (int)(t % p.tiles_h); t /= p.tiles_h;
        tnx = (int)t;
    };
    const int nkb = p.ntaps * p.cblocks;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
                int tcx, twx, thx, tnx;
                decode(t, tcx, twx, thx, tnx);
                const int w0 = twx * p.tw * p.in_stride, h0 = thx * p.th * p.in_stride, n0 = tnx * p.tn;
                for (int tap = 0; tap < p.ntaps && ok; ++tap) {
                    for (int cb = 0; cb < p.cblocks; ++cb) {
                        ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.status, 11);
                        if (!ok) break;
                        const uint32_t sa = smem_u32(smem + stage * Cfg::kStage), sb = sa + Cfg::kStageA, bar = full0 + 8 * stage;
                        mbar_expect_tx(bar, Cfg::kStage);
                        tma_load_4d(sa, &tmap_x, cb * 64, w0 + p.dw[tap], h0 + p.dh[tap], n0, bar);
                        tma_load_2d(sb, &tmap_w, (p.wtap[tap] * p.cblocks + cb) * 64, tcx * BN, bar);
                        if (++stage == kStages) { stage = 0; phase ^= 1; }
                    }
                }
            }
            for (int s = 0; s < kStages && ok; ++s) {
                ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.status, 12);
                if (++stage == kStages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int64_t it = 0;
            for (int64_t t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++it) {
                const int acc = (int)(it & 1);
                ok = mbar_wait(tempty0 + 8 * acc, (uint32_t)((it >> 1) & 1) ^ 1, abort_flag, p.status, 13);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_c = tmem_base + (uint32_t)(acc * BN);
                uint32_t accumulate = 0;
                for (int kb = 0; kb < nkb; ++kb) {
                    ok = mbar_wait(full0 + 8 * stage, phase, abort_flag, p.status, 14);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * Cfg::kStage), sb = sa + Cfg::kStageA;
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        umma<false>(tmem_c, make_smem_desc(sa + ks * 32, 16, 1024), make_smem_desc(sb + ks * 32, 16, 1024), p.idesc, accumulate);
                        accumulate = 1;
                    }
                    umma_commit(empty0 + 8 * stage);
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit(tfull0 + 8 * acc);
            }
        }
    } else {
        const int lane_window = (warp & 3) * 32;
        bool ok = true;
        int64_t it = 0;
        for (int64_t t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++it) {
            int tcx, twx, thx, tnx;
            decode(t, tcx, twx, thx, tnx);
            const int acc = (int)(it & 1);
            ok = mbar_wait(tfull0 + 8 * acc, (uint32_t)((it >> 1) & 1), abort_flag, p.status, 15);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            // row of the tile -> output pixel
            const int r = lane_window + lane;
            const int ww = r % p.tw, hh = (r / p.tw) % p.th, nn = r / (p.tw * p.th);
            const int wo = twx * p.tw + ww, ho = thx * p.th + hh, n = tnx * p.tn + nn;
            const bool row_ok = wo < p.Wo && ho < p.Ho && n < p.Nimg;
            const int64_t pix = ((int64_t)n * p.OH + (int64_t)ho * p.os + p.oh0) * p.OW + (int64_t)wo * p.os + p.ow0;
            uint16_t* orow = (uint16_t*)p.out + pix * p.OC;
            const int col0 = tcx * BN;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (col0 + c0 >= p.Cout) break;
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)lane_window << 16) + (uint32_t)(acc * BN + c0), v);
                tmem_ld_wait();
                if (row_ok) {
                    const int cbase = col0 + c0;
                    const int ncols = (p.Cout - cbase) < 32 ? (p.Cout - cbase) : 32;
                    uint32_t packed[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float a = __uint_as_float(v[2 * j]), b = __uint_as_float(v[2 * j + 1]);
                        if (p.dtype == TVK_F16) { __half2 h = __floats2half2_rn(a, b); packed[j] = *(uint32_t*)&h; }
                        else { __nv_bfloat162 h = __floats2bfloat162_rn(a, b); packed[j] = *(uint32_t*)&h; }
                    }
                    uint16_t* dst = orow + cbase;
                    if (p.out_nchw) {
                        const int64_t plane = (int64_t)p.OH * p.OW;
                        uint16_t* q = (uint16_t*)p.out + ((int64_t)n * p.Cout + cbase) * plane + ((int64_t)ho * p.os + p.oh0) * p.OW + (int64_t)wo * p.os + p.ow0;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (2 * j < ncols) q[(int64_t)(2 * j) * plane] = (uint16_t)(packed[j] & 0xffffu);
                            if (2 * j + 1 < ncols) q[(int64_t)(2 * j + 1) * plane] = (uint16_t)(packed[j] >> 16);
                        }
                    } else if (ncols == 32 && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4) *(uint4*)(dst + 2 * j) = make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (j < ncols) dst[j] = (uint16_t)((j & 1) ? (packed[j >> 1] >> 16) : (packed[j >> 1] & 0xffffu));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::kTmemCols) : "memory");
    }
}

// ---- weight-gradient kernel -----------------------------------------------------------------
// dW[tap][o][i] = sum over pixels of dY[pixel, o] * X[pixel shifted by the tap, i]: a GEMM with
// M = output channels (128 per tile), N = input channels (BN per tile) and the pixels as the
// contraction, 64 pixels (a tn x th x tw box) per k-block. Both operands are MN-major tiles: one
// k-row is one pixel, its 64 channels are the 128 bytes of the row. The pixel range is split over
// `splits` CTAs per (tap, o-tile, i-tile); each writes an fp32 partial (summed by
// wgrad_finalize_kernel), as the reference does with its split-K partials (src/api/ops/conv.cpp:1034-1060).
struct WgradParams {
    int tn, th, tw;                  // k-block pixel box, tn*th*tw == 64
    int blocks_w, blocks_h, blocks_n;
    int64_t kblocks;                 // blocks_w * blocks_h * blocks_n
    int splits;
    int64_t kb_per_split;
    int ntaps, tiles_o, tiles_i;
    int64_t total_items;             // ntaps * tiles_o * tiles_i * splits
    int in_stride;
    int8_t dh[kMaxTaps], dw[kMaxTaps];
    int O, I, Ip;                    // valid output / input channels, padded input channels (partial pitch)
    float* partial;                  // [splits][ntaps][O][Ip]
    uint32_t idesc;
    int* status;
};

template <int BN>
__global__ void __launch_bounds__(tc::kThreads, 1)
conv_wgrad_kernel(const __grid_constant__ CUtensorMap tmap_dy, const __grid_constant__ CUtensorMap tmap_x, const WgradParams p) {
    using namespace tc;
    using Cfg = Config<BN>;
    constexpr int kStages = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + kStages * Cfg::kStage);
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * kStages + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kStages);
    const uint32_t tfull0 = smem_u32(bars + 2 * kStages), tempty0 = smem_u32(bars + 2 * kStages + 2);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)Cfg::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto decode = [&](int64_t t, int& split, int& ti, int& to, int& tap) {
        split = (int)(t % p.splits); t /= p.splits;
        ti = (int)(t % p.tiles_i); t /= p.tiles_i;
        to = (int)(t % p.tiles_o); t /= p.tiles_o;
        tap = (int)t;
    };
    auto kb_range = [&](int split, int64_t& k0, int64_t& k1) {
        k0 = (int64_t)split * p.kb_per_split;
        k1 = k0 + p.kb_per_split;
        if (k1 > p.kblocks) k1 = p.kblocks;
        if (k0 > k1) k0 = k1;
    };

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < p.total_items && ok; t += gridDim.x) {
                int split, ti, to, tap;
                decode(t, split, ti, to, tap);
                int64_t k0, k1;
                kb_range(split, k0, k1);
                for (int64_t kb = k0; kb < k1; ++kb) {
                    const int bw = (int)(kb % p.blocks_w), bh = (int)((kb / p.blocks_w) % p.blocks_h), bn = (int)(kb / ((int64_t)p.blocks_w * p.blocks_h));
                    ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.status, 21);
                    if (!ok) break;
                    const uint32_t sa = smem_u32(smem + stage * Cfg::kStage), sb = sa + Cfg::kStageA, bar = full0 + 8 * stage;
                    mbar_expect_tx(bar, Cfg::kStage);
                    const int wo0 = bw * p.tw, ho0 = bh * p.th, n0 = bn * p.tn;
#pragma unroll
                    for (int j = 0; j < 2; ++j) tma_load_4d(sa + j * 8192, &tmap_dy, to * 128 + j * 64, wo0, ho0, n0, bar);
#pragma unroll
                    for (int j = 0; j < BN / 64; ++j)
                        tma_load_4d(sb + j * 8192, &tmap_x, ti * BN + j * 64, wo0 * p.in_stride + p.dw[tap], ho0 * p.in_stride + p.dh[tap], n0, bar);
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
            for (int s = 0; s < kStages && ok; ++s) {
                ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.status, 22);
                if (++stage == kStages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int64_t it = 0;
            for (int64_t t = blockIdx.x; t < p.total_items && ok; t += gridDim.x, ++it) {
                int split, ti, to, tap;
                decode(t, split, ti, to, tap);
                int64_t k0, k1;
                kb_range(split, k0, k1);
                const int acc = (int)(it & 1);
                ok = mbar_wait(tempty0 + 8 * acc, (uint32_t)((it >> 1) & 1) ^ 1, abort_flag, p.status, 23);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_c = tmem_base + (uint32_t)(acc * BN);
                uint32_t accumulate = 0;
                for (int64_t kb = k0; kb < k1; ++kb) {
                    ok = mbar_wait(full0 + 8 * stage, phase, abort_flag, p.status, 24);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * Cfg::kStage), sb = sa + Cfg::kStageA;
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        // MN-major tiles: 16 k-rows (pixels) per step = 2048 bytes; column blocks 8192 bytes apart
                        umma<false>(tmem_c, make_smem_desc(sa + ks * 2048, 8192, 1024), make_smem_desc(sb + ks * 2048, 8192, 1024), p.idesc, accumulate);
                        accumulate = 1;
                    }
                    umma_commit(empty0 + 8 * stage);
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit(tfull0 + 8 * acc);   // with an empty pixel range this still hands the (untouched) accumulator over
            }
        }
    } else {
        const int lane_window = (warp & 3) * 32;
        bool ok = true;
        int64_t it = 0;
        for (int64_t t = blockIdx.x; t < p.total_items && ok; t += gridDim.x, ++it) {
            int split, ti, to, tap;
            decode(t, split, ti, to, tap);
            int64_t k0, k1;
            kb_range(split, k0, k1);
            const int acc = (int)(it & 1);
            ok = mbar_wait(tfull0 + 8 * acc, (uint32_t)((it >> 1) & 1), abort_flag, p.status, 25);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int o = to * 128 + lane_window + lane;
            float* prow = p.partial + (((int64_t)split * p.ntaps + tap) * p.O + o) * p.Ip + (int64_t)ti * BN;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (ti * BN + c0 >= p.Ip) break;
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)lane_window << 16) + (uint32_t)(acc * BN + c0), v);
                tmem_ld_wait();
                if (o < p.O) {
                    const bool empty = k0 >= k1;   // nothing was accumulated: the partial is zero
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *(float4*)(prow + c0 + j) = empty ? make_float4(0.f, 0.f, 0.f, 0.f)
                                                          : make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::kTmemCols) : "memory");
    }
}

}  // namespace conv
}  // namespace tvk
