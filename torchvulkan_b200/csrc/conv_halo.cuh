// 3x3, stride 1, padding 1 convolution with at most 64 input and 64 output channels (the first stage of a
// CIFAR-sized ResNet: 32x32 images, 64 channels), forward and input gradient.
//
// The general kernel (conv_kernels.cuh) issues one TMA box per filter tap and channel block, so a 64-channel
// layer spends its time issuing eighteen small copies per 128-pixel tile and re-reading every input pixel nine
// times from L2. Here
//   * the nine 64x64 filter taps (72 KB) are loaded once per CTA and stay in shared memory;
//   * a tile is 16 rows x 8 columns of output pixels, and ONE TMA box brings its 18 x 10 input halo (zero filled
//     outside the image) into shared memory: 180 rows of 128 bytes (64 channels), 128-byte swizzled;
//   * the A operand of tap (dh, dw) is that same halo read through a shared-memory descriptor that starts
//     (dh+1)*10 + (dw+1) rows later, with 8-row groups (one image row of the tile) 10 rows apart. The swizzle is
//     a function of the shared-memory address, so a descriptor that starts on any 128-byte row reads what the
//     TMA wrote.
// Per tile: 1 copy instead of 18, 23 KB instead of 216 KB into shared memory, 36 MMAs back to back.
#pragma once

#include "tc_common.cuh"

namespace tvk {
namespace conv {

constexpr int kHaloW = 8, kHaloH = 16;                               // output tile: 16 rows x 8 columns = 128 pixels
constexpr int kHaloRows = (kHaloW + 2) * (kHaloH + 2);                // 180 input pixels
constexpr int kHaloBytes = kHaloRows * 128;                           // 23040
constexpr int kHaloStage = (kHaloBytes + 1023) / 1024 * 1024;         // 23552: stages stay 1024-byte aligned
constexpr int kHaloStages = 4;
constexpr int kHaloFilterBytes = 9 * 64 * 128;                        // nine K-major 64 x 64 tiles
constexpr int kHaloSmemBytes = kHaloFilterBytes + kHaloStages * kHaloStage + 1024 + 256 + tc::kStagingBytes;   // + epilogue staging rows

struct HaloParams {
    int N, H, W;                     // images and their extent (input and output extents are equal)
    int tiles_w, tiles_h;
    int64_t total_tiles;
    int8_t dh[9], dw[9];             // input offset of tap t (rows, columns), each in [-1, 1]
    int16_t wtap[9];                 // which 64-column block of the packed filter tap t multiplies
    int OC, Cout;                    // output channel pitch and count (<= 64)
    void* out;                       // channels-last [N, H, W, OC], or [N, Cout, H, W] when out_nchw is set
    int out_nchw;                    // the epilogue writes the caller's NCHW tensor itself (no staged copy, no transpose launch)
    int dtype;
    uint32_t idesc;
    int* status;
};

__global__ void __launch_bounds__(tc::kThreads, 1)
conv3x3_halo_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, const HaloParams p) {
    using namespace tc;
    constexpr int BN = 64;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* filt = smem;                                             // 72 KB
    uint8_t* halo = smem + kHaloFilterBytes;                          // kHaloStages x kHaloStage
    uint64_t* bars = (uint64_t*)(halo + kHaloStages * kHaloStage);
    // bars: full[S], empty[S], tmem_full[2], tmem_empty[2], filter
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * kHaloStages + 5);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kHaloStages);
    const uint32_t tfull0 = smem_u32(bars + 2 * kHaloStages), tempty0 = smem_u32(bars + 2 * kHaloStages + 2);
    const uint32_t fbar = smem_u32(bars + 2 * kHaloStages + 4);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kHaloStages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 4); }
        mbar_init(fbar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(128u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto decode = [&](int64_t t, int& tx, int& ty, int& n) {
        tx = (int)(t % p.tiles_w); t /= p.tiles_w;
        ty = (int)(t % p.tiles_h); t /= p.tiles_h;
        n = (int)t;
    };

    if (warp == 0) {
        if (lane == 0) {
            // the filter: nine boxes of 64 rows x 64 channels, once
            mbar_expect_tx(fbar, kHaloFilterBytes);
            for (int t = 0; t < 9; ++t) tma_load_2d(smem_u32(filt + t * 8192), &tmap_w, t * 64, 0, fbar);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
                int tx, ty, n;
                decode(t, tx, ty, n);
                ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.status, 31);
                if (!ok) break;
                const uint32_t bar = full0 + 8 * stage;
                mbar_expect_tx(bar, kHaloBytes);
                tma_load_4d(smem_u32(halo + stage * kHaloStage), &tmap_x, 0, tx * kHaloW - 1, ty * kHaloH - 1, n, bar);
                if (++stage == kHaloStages) { stage = 0; phase ^= 1; }
            }
            for (int s = 0; s < kHaloStages && ok; ++s) {
                ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.status, 32);
                if (++stage == kHaloStages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // per-tap operand offsets, kept in registers (a runtime index into the parameter arrays would go through local memory)
            uint32_t aoff[9], boff[9];
#pragma unroll
            for (int tap = 0; tap < 9; ++tap) {
                aoff[tap] = (uint32_t)(((p.dh[tap] + 1) * (kHaloW + 2) + (p.dw[tap] + 1)) * 128);
                boff[tap] = (uint32_t)p.wtap[tap] * 8192u;
            }
            bool ok = mbar_wait(fbar, 0, abort_flag, p.status, 33);
            int stage = 0;
            uint32_t phase = 0;
            int64_t it = 0;
            for (int64_t t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++it) {
                const int acc = (int)(it & 1);
                ok = mbar_wait(tempty0 + 8 * acc, (uint32_t)((it >> 1) & 1) ^ 1, abort_flag, p.status, 34);
                if (!ok) break;
                ok = mbar_wait(full0 + 8 * stage, phase, abort_flag, p.status, 35);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_c = tmem_base + (uint32_t)(acc * BN);
                const uint32_t sa = smem_u32(halo + stage * kHaloStage), sb = smem_u32(filt);
                uint32_t accumulate = 0;
#pragma unroll
                for (int tap = 0; tap < 9; ++tap) {
                    const uint32_t a0 = sa + aoff[tap];
                    const uint32_t b0 = sb + boff[tap];
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        // A: 8-row groups (one image row of the tile) are (kHaloW + 2) halo rows = 1280 bytes apart
                        umma<false>(tmem_c, make_smem_desc(a0 + ks * 32, 16, (kHaloW + 2) * 128), make_smem_desc(b0 + ks * 32, 16, 1024), p.idesc, accumulate);
                        accumulate = 1;
                    }
                }
                umma_commit(empty0 + 8 * stage);
                umma_commit(tfull0 + 8 * acc);
                if (++stage == kHaloStages) { stage = 0; phase ^= 1; }
            }
        }
    } else {
        const int lane_window = (warp & 3) * 32;
        // full 64-channel rows of a 64-channel-pitch output go through this warp's staging rows for 128-byte line stores
        const bool staged = !p.out_nchw && p.Cout == 64 && p.OC == 64 && ((uintptr_t)p.out & 15) == 0;
        uint8_t* stg = (uint8_t*)bars + 256 + (warp - 2) * (32 * kStagingPitch);
        bool ok = true;
        int64_t it = 0;
        for (int64_t t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++it) {
            int tx, ty, n;
            decode(t, tx, ty, n);
            const int acc = (int)(it & 1);
            ok = mbar_wait(tfull0 + 8 * acc, (uint32_t)((it >> 1) & 1), abort_flag, p.status, 36);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int r = lane_window + lane;
            const int w = tx * kHaloW + (r & (kHaloW - 1)), h = ty * kHaloH + (r >> 3);
            const bool row_ok = w < p.W && h < p.H;
            uint16_t* orow = (uint16_t*)p.out + (((int64_t)n * p.H + h) * p.W + w) * p.OC;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (c0 >= p.Cout) break;
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)lane_window << 16) + (uint32_t)(acc * BN + c0), v);
                tmem_ld_wait();
                if (row_ok) {
                    const int ncols = (p.Cout - c0) < 32 ? (p.Cout - c0) : 32;
                    uint32_t packed[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float a = __uint_as_float(v[2 * j]), b = __uint_as_float(v[2 * j + 1]);
                        if (p.dtype == TVK_F16) { __half2 hh = __floats2half2_rn(a, b); packed[j] = *(uint32_t*)&hh; }
                        else { __nv_bfloat162 hh = __floats2bfloat162_rn(a, b); packed[j] = *(uint32_t*)&hh; }
                    }
                    uint16_t* dst = orow + c0;
                    if (p.out_nchw) {
                        // a lane is a pixel: per channel the eight pixels of a tile row are 16 contiguous bytes of the plane
                        const int64_t plane = (int64_t)p.H * p.W;
                        uint16_t* q = (uint16_t*)p.out + ((int64_t)n * p.Cout + c0) * plane + (int64_t)h * p.W + w;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (2 * j < ncols) q[(int64_t)(2 * j) * plane] = (uint16_t)(packed[j] & 0xffffu);
                            if (2 * j + 1 < ncols) q[(int64_t)(2 * j + 1) * plane] = (uint16_t)(packed[j] >> 16);
                        }
                    } else if (staged) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4)
                            *(uint4*)(stg + lane * kStagingPitch + c0 * 2 + j * 4) = make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
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
            if (lane == 0) mbar_arrive(tempty0 + 8 * acc);      // the accumulator is in registers / staging rows now
            if (staged) {
                // 64 channels = one 128-byte line per pixel: eight lanes write a pixel, four pixels per instruction
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int rr = lane_window + 4 * i + (lane >> 3);
                    const int ww = tx * kHaloW + (rr & (kHaloW - 1)), hh = ty * kHaloH + (rr >> 3);
                    const uint4 line = *(const uint4*)(stg + (4 * i + (lane >> 3)) * kStagingPitch + (lane & 7) * 16);
                    if (ww < p.W && hh < p.H)
                        *(uint4*)((uint8_t*)p.out + ((((int64_t)n * p.H + hh) * p.W + ww) << 7) + (lane & 7) * 16) = line;
                }
                __syncwarp();
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(128u) : "memory");
    }
}

// ---- weight gradient of the same layers -----------------------------------------------------------------
// dW[o][kh][kw][i] = sum over pixels of dY[pixel, o] * X[pixel + (kh-1, kw-1), i]. A work item is one filter row kh
// and one range of 8x8 pixel blocks. Per block it loads the dY tile (64 pixels x 64 channels, 8 KB) and the 8 x 10
// input rows that filter row touches (10 KB), and issues four MMAs (one per 16 pixels) whose N dimension is
// 192 = the three taps of the row x 64 input channels: tap kw is the same shared-memory rows shifted by one pixel,
// so the three taps are three "column blocks" of one MN-major descriptor that lie 128 bytes apart. M is 128 with the
// 64 output channels mapped twice (leading byte offset 0): accumulator lanes 64..127 repeat lanes 0..63 and are
// not read. Partials go to [splits][9][O][64] in fp32 and are summed by wgrad_finalize_kernel.
constexpr int kWgStageA = 64 * 128;                      // dY: 64 pixels
constexpr int kWgStageB = 80 * 128;                      // X: 8 rows x 10 columns of pixels
constexpr int kWgStage = kWgStageA + kWgStageB;          // 18432, a multiple of 1024
constexpr int kWgStages = 8;
constexpr int kWgSmemBytes = kWgStages * kWgStage + 1024 + 256;

struct HaloWgradParams {
    int N, H, W;
    int blocks_w, blocks_h;
    int64_t kblocks;                 // blocks_w * blocks_h * N
    int splits;
    int64_t kb_per_split;
    int total_items;                 // 3 * splits
    int O;                           // output channels (<= 64)
    float* partial;                  // [splits][9][O][64]
    uint32_t idesc;
    int* status;
};

__global__ void __launch_bounds__(tc::kThreads, 1)
conv3x3_wgrad_rows_kernel(const __grid_constant__ CUtensorMap tmap_dy, const __grid_constant__ CUtensorMap tmap_x, const HaloWgradParams p) {
    using namespace tc;
    constexpr int BNW = 192;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + kWgStages * kWgStage);
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * kWgStages + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kWgStages);
    const uint32_t tfull0 = smem_u32(bars + 2 * kWgStages), tempty0 = smem_u32(bars + 2 * kWgStages + 2);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWgStages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

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
            for (int item = blockIdx.x; item < p.total_items && ok; item += gridDim.x) {
                const int kh = item % 3, split = item / 3;
                int64_t k0, k1;
                kb_range(split, k0, k1);
                for (int64_t kb = k0; kb < k1; ++kb) {
                    const int bw = (int)(kb % p.blocks_w), bh = (int)((kb / p.blocks_w) % p.blocks_h), n = (int)(kb / ((int64_t)p.blocks_w * p.blocks_h));
                    ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.status, 41);
                    if (!ok) break;
                    const uint32_t sa = smem_u32(smem + stage * kWgStage), sb = sa + kWgStageA, bar = full0 + 8 * stage;
                    mbar_expect_tx(bar, kWgStage);
                    tma_load_4d(sa, &tmap_dy, 0, bw * 8, bh * 8, n, bar);
                    tma_load_4d(sb, &tmap_x, 0, bw * 8 - 1, bh * 8 - 1 + kh, n, bar);
                    if (++stage == kWgStages) { stage = 0; phase ^= 1; }
                }
            }
            for (int s = 0; s < kWgStages && ok; ++s) {
                ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.status, 42);
                if (++stage == kWgStages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int it = 0;
            for (int item = blockIdx.x; item < p.total_items && ok; item += gridDim.x, ++it) {
                const int split = item / 3;
                int64_t k0, k1;
                kb_range(split, k0, k1);
                const int acc = it & 1;
                ok = mbar_wait(tempty0 + 8 * acc, (uint32_t)((it >> 1) & 1) ^ 1, abort_flag, p.status, 43);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_c = tmem_base + (uint32_t)(acc * 256);
                uint32_t accumulate = 0;
                for (int64_t kb = k0; kb < k1; ++kb) {
                    ok = mbar_wait(full0 + 8 * stage, phase, abort_flag, p.status, 44);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * kWgStage), sb = sa + kWgStageA;
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        // 16 pixels per step = two image rows of the block: 2 x 1024 bytes of dY, 2 x 1280 bytes of X rows
                        umma<false>(tmem_c, make_smem_desc(sa + ks * 2048, 0, 1024), make_smem_desc(sb + ks * 2560, 128, 1280), p.idesc, accumulate);
                        accumulate = 1;
                    }
                    umma_commit(empty0 + 8 * stage);
                    if (++stage == kWgStages) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit(tfull0 + 8 * acc);
            }
        }
    } else {
        const int lane_window = (warp & 3) * 32;
        bool ok = true;
        int it = 0;
        for (int item = blockIdx.x; item < p.total_items && ok; item += gridDim.x, ++it) {
            const int kh = item % 3, split = item / 3;
            int64_t k0, k1;
            kb_range(split, k0, k1);
            const int acc = it & 1;
            ok = mbar_wait(tfull0 + 8 * acc, (uint32_t)((it >> 1) & 1), abort_flag, p.status, 45);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int o = lane_window + lane;
            if (lane_window < 64) {                      // lanes 64..127 hold the repeated rows
#pragma unroll 1
                for (int c0 = 0; c0 < BNW; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((uint32_t)lane_window << 16) + (uint32_t)(acc * 256 + c0), v);
                    tmem_ld_wait();
                    if (o < p.O) {
                        const int kw = c0 >> 6, i0 = c0 & 63;
                        float* prow = p.partial + ((((int64_t)split * 9 + kh * 3 + kw) * p.O + o) << 6) + i0;
                        const bool empty = k0 >= k1;
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *(float4*)(prow + j) = empty ? make_float4(0.f, 0.f, 0.f, 0.f)
                                                         : make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace conv
}  // namespace tvk
