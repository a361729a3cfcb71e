// Two-CTA (cta_group::2) tcgen05 GEMM for kernels launched with thread-block clusters of 2.
//
// A cluster computes a 256 x 256 output tile: CTA rank r of the pair owns rows [r*128, r*128+128)
// of the tile (its own TMEM holds that 128 x 256 FP32 accumulator) and stages, per 64-deep K
// block, its own 128 x 64 slice of A plus 128 of the 256 B columns (32 KiB instead of the 48 KiB
// a single-CTA 128 x 256 tile needs).  One thread of the even CTA issues
// tcgen05.mma.cta_group::2 (M = 256), which reads A from each CTA's shared memory and gathers the
// two B halves; this halves the B traffic into shared memory, the resource that bounds the
// single-CTA tile.  Protocol:
//   * both CTAs' TMA loads complete on the EVEN CTA's full barrier (cta_group::2 loads, barrier
//     address with the peer bit cleared); the even CTA's producer posts the 64 KiB expect_tx;
//   * the even CTA's MMA thread waits on that barrier, issues the MMAs, and commits with a
//     cluster-multicast arrive so the slot's empty barrier (and, per tile, the accumulator's
//     full barrier) fires in both CTAs;
//   * the epilogue warps of both CTAs arrive on the even CTA's accumulator-empty barrier
//     (remote mbarrier arrive for the odd CTA).
// Every wait is bounded exactly like the single-CTA path.
#pragma once
#include "tk_device.cuh"

namespace tk {

constexpr int kSlot2A = BM * BK * 2;           // 16 KiB: this CTA's 128 rows of A
constexpr int kSlot2B = 128 * BK * 2;          // 16 KiB: this CTA's 128 columns of B
constexpr int kSlot2Bytes = kSlot2A + kSlot2B;
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu; // clears the CTA-rank bit of a shared-window address

__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t cta) {
    asm volatile("{\n .reg .b32 ra;\n mapa.shared::cluster.u32 ra, %0, %1;\n mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n}"
                 :: "r"(smem_u32(bar)), "r"(cta) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar) & kPeerBitMask), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc2_commit_both(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :: "r"(smem_u32(bar)), "h"(static_cast<uint16_t>(3)) : "memory");
}
__device__ __forceinline__ void tc2_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void ctx_init2(Ctx& c, uint32_t* sync, uint32_t* status, uint64_t timeout_ns, uint32_t arrivals, SharedState* sh, uint8_t* dyn) {
    c.sync = sync; c.status = status; c.timeout_ns = timeout_ns; c.sh = sh;
    c.arrivals = arrivals ? arrivals : gridDim.x;
    c.slots = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn) + 1023) & ~uintptr_t(1023));
    c.stage_id = 0; c.slot = 0; c.slot_phase = 0; c.acc = 0; c.acc_phase = 0; c.tmem = 0; c.epi = nullptr;
    c.stamps = nullptr; c.flags = 0;
    c.warp = threadIdx.x >> 5; c.lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        sh->abort = 0;
        for (int i = 0; i < kStages2; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&sh->tmem_full[i], 1); mbar_init(&sh->tmem_empty[i], 2 * (kEpiThreads / 32)); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (c.warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&sh->tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();            // the peer's barriers are initialised before anything signals them
    tc_fence_after();
    c.tmem = *reinterpret_cast<volatile uint32_t*>(&sh->tmem_base);
}

__device__ __forceinline__ void ctx_finish2(Ctx& c) {
    tc_fence_before();
    __syncthreads();
    if (c.aborted()) {
        const uint64_t start = global_timer_ns();
        while (global_timer_ns() - start < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync();            // neither CTA frees TMEM or leaves while the peer may still touch it
    if (c.warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(c.tmem), "r"(kTmemCols) : "memory");
    }
}

// Pair-tile rasterisation: groups of kGroupM2 pair rows walked column by column.
template <int GROUP>
__device__ __forceinline__ void pair_coords(int64_t t, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int64_t per_group = static_cast<int64_t>(GROUP) * tiles_n;
    const int group = static_cast<int>(t / per_group);
    const int first = group * GROUP;
    const int rows = min(GROUP, tiles_m - first);
    const int within = static_cast<int>(t - static_cast<int64_t>(group) * per_group);
    tm = first + within % rows;
    tn = within / rows;
}

// C[M,N] = A[M,K] * B[K,N].  Tensor maps: K-major operands use a {64 (K), 128 rows} box,
// MN-major operands a {64 (MN), 64 (K)} box per 64-wide atom (two atoms per CTA per operand).
// `item_base` is the unit's position in the stage's item list counted in CTAs (even).
template <bool A_MN, bool B_MN, int FMT, int GROUP, typename Epi, typename Bg, typename Params>
__device__ __forceinline__ void gemm_tc2(Ctx& c, const Params& P, const CUtensorMap* map_a, const CUtensorMap* map_b,
                                         int M, int N, int K, int64_t item_base) {
    constexpr int TM = 256, TN = 256;
    const int tiles_m = (M + TM - 1) / TM, tiles_n = (N + TN - 1) / TN;
    const int64_t tiles = static_cast<int64_t>(tiles_m) * tiles_n;
    const int kblocks = (K + BK - 1) / BK;
    const uint32_t rank = cluster_ctarank();
    const int64_t clusters = gridDim.x / 2;
    const int64_t cluster_id = blockIdx.x / 2;
    int64_t first = (cluster_id - item_base / 2) % clusters;
    if (first < 0) first += clusters;
    SharedState* sh = c.sh;

    if (c.warp == 0) {
        if (c.lane == 0) {
            for (int64_t t = first; t < tiles && !c.aborted(); t += clusters) {
                int tm, tn; pair_coords<GROUP>(t, tiles_m, tiles_n, tm, tn);
                const int row0 = tm * TM + static_cast<int>(rank) * 128;     // this CTA's A rows
                const int col0 = tn * TN + static_cast<int>(rank) * 128;     // this CTA's B columns
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!c.wait(&sh->empty[c.slot], c.slot_phase ^ 1, kErrSmemEmpty)) break;
                    uint8_t* sa = c.slots + c.slot * kSlot2Bytes;
                    uint8_t* sb = sa + kSlot2A;
                    if (rank == 0) mbar_expect_tx(&sh->full[c.slot], 2 * kSlot2Bytes);
                    if constexpr (A_MN) {
                        tma_load_2d_pair(sa, map_a, &sh->full[c.slot], row0, kb * BK);
                        tma_load_2d_pair(sa + 8192, map_a, &sh->full[c.slot], row0 + 64, kb * BK);
                    } else {
                        tma_load_2d_pair(sa, map_a, &sh->full[c.slot], kb * BK, row0);
                    }
                    if constexpr (B_MN) {
                        tma_load_2d_pair(sb, map_b, &sh->full[c.slot], col0, kb * BK);
                        tma_load_2d_pair(sb + 8192, map_b, &sh->full[c.slot], col0 + 64, kb * BK);
                    } else {
                        tma_load_2d_pair(sb, map_b, &sh->full[c.slot], kb * BK, col0);
                    }
                    c.advance_slot2();
                }
            }
        }
        __syncwarp();
    } else if (c.warp == 1) {
        if (rank == 0 && c.lane == 0) {
            constexpr uint32_t idesc = umma_idesc(FMT, A_MN ? 1 : 0, B_MN ? 1 : 0, TM, TN);
            for (int64_t t = first; t < tiles && !c.aborted(); t += clusters) {
                if (!c.wait(&sh->tmem_empty[c.acc], c.acc_phase ^ 1, kErrTmemEmpty)) break;
                tc_fence_after();
                const uint32_t d_tmem = c.tmem + c.acc * kMaxBN;
                bool ok = true;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!c.wait(&sh->full[c.slot], c.slot_phase, kErrSmemFull)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(c.slots + c.slot * kSlot2Bytes);
                    const uint32_t sb = sa + kSlot2A;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t da = A_MN ? umma_desc(sa + k * 2048, 8192, 1024) : umma_desc(sa + k * 32, 16, 1024);
                        const uint64_t db = B_MN ? umma_desc(sb + k * 2048, 8192, 1024) : umma_desc(sb + k * 32, 16, 1024);
                        tc2_mma_f16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tc2_commit_both(&sh->empty[c.slot]);
                    c.advance_slot2();
                }
                if (!ok) break;
                tc2_commit_both(&sh->tmem_full[c.acc]);
                c.advance_acc();
            }
        }
        __syncwarp();
    } else if (c.warp < 2 + kEpiWarps) {
        const int quarter = c.warp & 3;
        const int chunk0 = (c.warp - 2) >> 2;          // wide epilogue: warps 6..9 start one chunk later ...
        constexpr int kChunkStep = kEpiWarps / 4;      // ... and every warp takes every other chunk
        for (int64_t t = first; t < tiles && !c.aborted(); t += clusters) {
            int tm, tn; pair_coords<GROUP>(t, tiles_m, tiles_n, tm, tn);
            if (chunk0 == 0 && t + clusters < tiles) {
                int pm, pn; pair_coords<GROUP>(t + clusters, tiles_m, tiles_n, pm, pn);
                const int prow = pm * TM + static_cast<int>(rank) * 128 + quarter * 32 + c.lane;
                if (prow < M && pn * TN < N) Epi::prefetch(P, prow, pn * TN, min(TN, N - pn * TN));
            }
            const int row0 = tm * TM + static_cast<int>(rank) * 128 + quarter * 32;
            typename EpiOps<Epi>::type operands;
            if constexpr (Epi::kPipelined || Epi::kFetchFirst) {               // in flight during the wait
                if (tn * TN + 32 * chunk0 < N) epilogue_fetch<Epi>(c, P, row0, tn * TN + 32 * chunk0, min(32, N - tn * TN - 32 * chunk0), operands);
            }
            if (!c.wait(&sh->tmem_full[c.acc], c.acc_phase, kErrTmemFull)) break;
            tc_fence_after();
            const uint32_t taddr = c.tmem + c.acc * kMaxBN + (static_cast<uint32_t>(quarter * 32) << 16);
            epilogue_tile<TN, Epi>(c, P, taddr, row0, tn * TN, N, operands, chunk0, kChunkStep);
            tc_fence_before();
            __syncwarp();
            if (c.lane == 0) {
                if (rank == 0) mbar_arrive(&sh->tmem_empty[c.acc]);
                else mbar_arrive_remote(&sh->tmem_empty[c.acc], 0);
            }
            c.advance_acc();
        }
    }
}

}  // namespace tk
