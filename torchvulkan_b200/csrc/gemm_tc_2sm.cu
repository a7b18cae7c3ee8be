// K-sliced product on CTA pairs: tcgen05.mma.cta_group::2, one 256 x 256 tile of fp32 partial sums per pair and K slice.
//
// For one or two 128-row tiles against a large weight matrix (the forward and input-gradient products of a wide layer at
// a small batch; the reference runs them through the same matmul shader as every other shape,
// src/api/ops/matmul.cpp:373-582) what bounds the single-CTA kernel is the rate at which one SM pulls its operands through
// L2 (about 90 GB/s per SM): a 128 x 256 tile needs 128 rows of A and 256 rows of B per k-block. A CTA pair shares the B
// tile - each CTA loads its own 128 rows of A and HALF of the 256 rows of B, and the pair's tensor cores read both halves
// - so a CTA pulls 256 rows per k-block for the same 128 x 256 outputs: two thirds of the bytes.
//
// Roles per CTA (192 threads): warp 0 TMA producer (both CTAs' copies of a stage are counted on ONE barrier, in the issuing
// CTA), warp 1 MMA issuer (CTA 0 of the pair only), warps 2-5 epilogue (tensor memory -> fp32 partials in global memory).
// The finishing pass of the K slices (simt::splitk_epilogue_vec_kernel) applies bias, activation and the fused forms.
// Every wait is bounded and reports through the device status word; both CTAs of a pair always reach the closing cluster
// barrier. Each CTA loads its own operands; nothing is broadcast between them.
#include "gemm_tc.cuh"

namespace tvk {
namespace tc {

constexpr int k2smStages = 6;
constexpr int k2smStageA = 128 * 128, k2smStageB = 128 * 128, k2smStage = k2smStageA + k2smStageB;       // bytes per CTA and stage
constexpr int k2smOutBuf = 32 * 128;                                    // per epilogue warp: 32 rows x 32 fp32 columns, 128-byte swizzle
constexpr int k2smSmemBytes = k2smStages * k2smStage + 4 * k2smOutBuf + 1024 + 256;
constexpr int k2smTmemCols = 256;

struct Params2sm {
    int64_t m, n;
    int num_kb;              // k-blocks of 64 per K slice
    int tiles_m, tiles_n;    // 256-row and 256-column tiles
    int splits;              // K slices (the batch index of the tensor maps)
    uint32_t idesc;
    float* partial;          // [splits][m][n]
    int* status;
    int debug;               // probes (results undefined): 1 no stores, 2 no MMAs (commits only), 16 every CTA writes the tensor-memory address it was given into partial[blockIdx.x]
};

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_c,
                 const Params2sm p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* outbuf = smem + k2smStages * k2smStage;
    uint64_t* bars = (uint64_t*)(outbuf + 4 * k2smOutBuf);
    // full[S] (CTA 0's counts the TMA bytes of both CTAs), empty[S], tfull, tempty
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * k2smStages;
    const uint32_t tfull = empty0 + 8 * k2smStages, tempty = tfull + 8;
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * k2smStages + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const uint32_t pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const uint32_t tiles_per_slice = (uint32_t)(p.tiles_m * p.tiles_n);
    const uint32_t total_tiles = tiles_per_slice * (uint32_t)p.splits;
    // tile t -> K slice b, row tile tm (fastest: neighbouring pairs share a tile of B), column tile tn
    auto decode = [&](uint32_t t, int& b, int& tm, int& tn) {
        const uint32_t bb = t / tiles_per_slice, r = t - bb * tiles_per_slice;
        b = (int)bb;
        tn = (int)(r / (uint32_t)p.tiles_m);
        tm = (int)(r - (uint32_t)tn * (uint32_t)p.tiles_m);
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < k2smStages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(tfull, 1);
        mbar_init(tempty, 8);                 // four epilogue warps in each CTA of the pair
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0 && lane == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_c) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)k2smTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                       // both CTAs' barriers are initialised before anything arrives on them from the other side
    tc_fence_after();
    const uint32_t own_tmem = *tmem_slot;
    // the accumulator lives at the address the issuing CTA allocated, in both CTAs' tensor memory
    const uint32_t tmem_base = rank == 0 ? own_tmem : ld_remote_u32(map_to_cta(smem_u32(tmem_slot), 0));

    if (warp == 0) {
        // ------------------------------ TMA producer (both CTAs) ------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (uint32_t t = pair; t < total_tiles && ok; t += npairs) {
                int b, tm, tn;
                decode(t, b, tm, tn);
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    ok = mbar_wait_cluster(empty0 + 8 * stage, phase ^ 1, abort_flag, p.status, 61);
                    if (!ok) break;
                    const uint32_t sa = smem_u32(smem + stage * k2smStage), sb = sa + k2smStageA;
                    // both CTAs' copies of this stage are counted on the issuing CTA's barrier, which expects the bytes of both
                    const uint32_t bar = map_to_cta(full0 + 8 * stage, 0);
                    if (rank == 0) mbar_expect_tx(full0 + 8 * stage, 2 * k2smStage);
                    if (!A_MN) {
                        tma_load_3d_pair(sa, &tmap_a, kb * 64, tm * 256 + (int)rank * 128, b, bar);
                    } else {
                        tma_load_3d_pair(sa, &tmap_a, tm * 256 + (int)rank * 128, kb * 64, b, bar);
                        tma_load_3d_pair(sa + 64 * 128, &tmap_a, tm * 256 + (int)rank * 128 + 64, kb * 64, b, bar);
                    }
                    if (!B_MN) {
                        tma_load_3d_pair(sb, &tmap_b, kb * 64, tn * 256 + (int)rank * 128, b, bar);
                    } else {
                        tma_load_3d_pair(sb, &tmap_b, tn * 256 + (int)rank * 128, kb * 64, b, bar);
                        tma_load_3d_pair(sb + 64 * 128, &tmap_b, tn * 256 + (int)rank * 128 + 64, kb * 64, b, bar);
                    }
                    if (++stage == k2smStages) { stage = 0; phase ^= 1; }
                }
            }
            if (ok) {
                // drain: no copy may still be in flight towards shared memory when the CTA exits
                for (int s = 0; s < k2smStages && ok; ++s) {
                    ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.status, 62);
                    if (++stage == k2smStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ------------------------------ MMA issuer (CTA 0 of the pair) ------------------------------
            int stage = 0;
            uint32_t phase = 0, tphase = 0;
            bool ok = true;
            // per k-step advance of the descriptor start address and the distance between 64-wide column blocks (MN-major)
            const uint32_t a_step = A_MN ? (uint32_t)(16 * 128) : 32u, b_step = B_MN ? (uint32_t)(16 * 128) : 32u;
            const uint32_t a_lbo = A_MN ? (uint32_t)(64 * 128) : 16u, b_lbo = B_MN ? (uint32_t)(64 * 128) : 16u;
            for (uint32_t t = pair; t < total_tiles && ok; t += npairs) {
                ok = mbar_wait_cluster(tempty, tphase ^ 1, abort_flag, p.status, 64);       // both epilogues have drained the accumulator
                if (!ok) break;
                tc_fence_after();
                uint32_t accumulate = 0;
                for (int kb = 0; kb < p.num_kb; ++kb) {
                    ok = mbar_wait_cluster(full0 + 8 * stage, phase, abort_flag, p.status, 65);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * k2smStage), sb = sa + k2smStageA;
#pragma unroll
                    for (int ks = 0; ks < 4 && !(p.debug & 2); ++ks) {
                        umma_pair(tmem_base, make_smem_desc(sa + ks * a_step, a_lbo, 1024), make_smem_desc(sb + ks * b_step, b_lbo, 1024), p.idesc, accumulate);
                        accumulate = 1;
                    }
                    // the stage is free again in both CTAs
                    umma_commit_pair(empty0 + 8 * stage);
                    umma_commit_pair(map_to_cta(empty0 + 8 * stage, 1));
                    if (++stage == k2smStages) { stage = 0; phase ^= 1; }
                }
                if (ok) {
                    umma_commit_pair(tfull);
                    umma_commit_pair(map_to_cta(tfull, 1));
                }
                tphase ^= 1;
            }
        }
    } else {
        // ------------------------------ epilogue (both CTAs): 128 rows x 256 columns of fp32 partial sums ------------------------------
        const int lane_window = (warp & 3) * 32;
        uint32_t tphase = 0;
        bool ok = true;
        const uint32_t tempty_issuer = rank == 0 ? tempty : map_to_cta(tempty, 0);
        for (uint32_t t = pair; t < total_tiles && ok; t += npairs) {
            int b, tm, tn;
            decode(t, b, tm, tn);
            ok = mbar_wait_cluster(tfull, tphase, abort_flag, p.status, 67);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tphase ^= 1;
            tc_fence_after();
            const int64_t row0 = (int64_t)tm * 256 + (int64_t)rank * 128 + lane_window;       // first row of this warp's 32
            const int64_t col0 = (int64_t)tn * 256;
            uint8_t* buf = outbuf + (warp - 2) * k2smOutBuf;
#pragma unroll 1
            for (int c0 = 0; c0 < 256; c0 += 32) {
                if (col0 + c0 >= p.n) break;
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)lane_window << 16) + (uint32_t)c0, v);
                tmem_ld_wait();
                if (p.debug & 1) continue;
                // 32 rows x 128 bytes staged in the swizzled layout (chunk j of row r at j ^ (r & 7)), then one TMA store
                // (rows and columns beyond the matrix are clipped by the tensor map)
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    *(uint4*)(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0 && row0 < p.m) {
                    tma_store_3d(&tmap_c, smem_u32(buf), (int)(col0 + c0), (int)row0, b);
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(tempty);
                else mbar_arrive_remote(tempty_issuer);
            }
        }
    }
    __syncwarp();
    if (warp >= 2 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");      // this warp's stores have left shared memory and landed
    if (*abort_flag) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    // neither CTA leaves (and frees its barriers and tensor memory) while the other may still signal it or multiply from its shared memory
    cluster_sync_all();
    tc_fence_after();
    if ((p.debug & 16) && threadIdx.x == 0) ((uint32_t*)p.partial)[blockIdx.x] = own_tmem;      // probe: the address each CTA's allocation returned
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(own_tmem), "r"((uint32_t)k2smTmemCols) : "memory");
    }
}

// maps[0]: A, box {64 k, 128 rows} (K-major) or {64 rows, 64 k} (MN-major); maps[1]: B likewise over its columns; maps[2]: the fp32
// partials [splits][m][n], box {32 columns, 32 rows}; batch = K slice
int launch_pair(bool a_mn, bool b_mn, const CUtensorMap* maps, int64_t m, int64_t n, int num_kb, int splits, uint32_t idesc, float* partial, int* status, int debug,
                cudaStream_t s) {
    Params2sm p = {};
    p.debug = debug;
    p.m = m; p.n = n; p.num_kb = num_kb; p.tiles_m = (int)((m + 255) / 256); p.tiles_n = (int)((n + 255) / 256); p.splits = splits; p.idesc = idesc;
    p.partial = partial; p.status = status;
    static bool attr_done[4] = {false, false, false, false};
    const int64_t total = (int64_t)p.tiles_m * p.tiles_n * p.splits;
    int pairs = sm_count() / 2;
    if (pairs > total) pairs = (int)total;
    if (pairs < 1) pairs = 1;
    const int which = (a_mn ? 2 : 0) | (b_mn ? 1 : 0);
    const void* fns[4] = {(const void*)gemm_pair_kernel<false, false>, (const void*)gemm_pair_kernel<false, true>, (const void*)gemm_pair_kernel<true, false>,
                          (const void*)gemm_pair_kernel<true, true>};
    if (!attr_done[which]) {
        cudaError_t e = cudaFuncSetAttribute(fns[which], cudaFuncAttributeMaxDynamicSharedMemorySize, k2smSmemBytes);
        if (e != cudaSuccess) return set_error(TVK_ERR_CUDA, "cudaFuncSetAttribute (pair gemm) failed: %s", cudaGetErrorString(e));
        attr_done[which] = true;
    }
    switch (which) {
        case 0: gemm_pair_kernel<false, false><<<2 * pairs, kThreads, k2smSmemBytes, s>>>(maps[0], maps[1], maps[2], p); break;
        case 1: gemm_pair_kernel<false, true><<<2 * pairs, kThreads, k2smSmemBytes, s>>>(maps[0], maps[1], maps[2], p); break;
        case 2: gemm_pair_kernel<true, false><<<2 * pairs, kThreads, k2smSmemBytes, s>>>(maps[0], maps[1], maps[2], p); break;
        default: gemm_pair_kernel<true, true><<<2 * pairs, kThreads, k2smSmemBytes, s>>>(maps[0], maps[1], maps[2], p); break;
    }
    return launch_status("pair gemm");
}

}  // namespace tc
}  // namespace tvk
