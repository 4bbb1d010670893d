// bf16 GEMM for sm_100a on the 5th-generation tensor cores.
//
//   D[m, n] (+)= alpha * sum_k A(m, k) * B(n, k)
//
// One persistent CTA per SM walks a list of 128 x 256 output tiles. Operand tiles are brought
// into 128-byte-swizzled shared memory by TMA (each CTA fetches its own tiles), a single thread
// issues tcgen05.mma into one of two 256-column TMEM accumulators, and four epilogue warps drain
// the other accumulator with tcgen05.ld while the next tile is being multiplied.
//
// Either operand may be "K-major" (the reduction index is the contiguous one, the layout of
// y = x W^T) or "MN-major" (the reduction index walks rows, the layout of dx = dy W and of
// dW = dy^T x), so forward, data-gradient and weight-gradient products all read the tensors in
// place. The tile list is either derived from (M, N, K) or read from device memory, which is how
// the grouped (per-expert) products of an MoE layer run without a host round trip.
//
// Replaces what the reference obtains from cuBLAS (F.linear) and from torch's grouped_mm
// (halo/kernels/grouped_mm.py:30-51, halo/kernels/expert_gemm.py:14-35).
#include "gemm_sm100.cuh"

#include <stdio.h>

namespace halo {

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ GemmParams p) {
    if (status_poisoned(p.status)) return;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[kStages], bar_empty[kStages], bar_tfull[2], bar_tempty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bar_tfull[a]), 1);
            mbar_init(smem_u32(&bar_tempty[a]), 4);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    const int total = p.list ? *p.list_count : p.tiles_m * p.tiles_n;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            GemmWork w;
            for (int idx = blockIdx.x; fetch_work(p, idx, total, w) && !abort_flag;
                 idx += gridDim.x) {
                for (int kb = 0; kb < w.k_iters; ++kb) {
                    if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, &abort_flag, p.status))
                        break;
                    const uint32_t full = smem_u32(&bar_full[stage]);
                    const uint32_t sa = tiles_base + stage * kStageBytes;
                    const uint32_t sb = sa + kATileBytes;
                    mbar_expect_tx(full, kStageBytes);
                    if (A_MN) {
                        tma_load_2d(sa, &tmA, full, w.a_mn, w.a_k + kb * kBlockK);
                        tma_load_2d(sa + 8192, &tmA, full, w.a_mn + 64, w.a_k + kb * kBlockK);
                    } else {
                        tma_load_2d(sa, &tmA, full, w.a_k + kb * kBlockK, w.a_mn);
                    }
                    if (B_MN) {
                        tma_load_2d(sb, &tmB, full, w.b_mn, w.b_k + kb * kBlockK);
                        tma_load_2d(sb + 8192, &tmB, full, w.b_mn + 64, w.b_k + kb * kBlockK);
                        tma_load_2d(sb + 16384, &tmB, full, w.b_mn2, w.b_k + kb * kBlockK);
                        tma_load_2d(sb + 24576, &tmB, full, w.b_mn2 + 64, w.b_k + kb * kBlockK);
                    } else {
                        tma_load_2d(sb, &tmB, full, w.b_k + kb * kBlockK, w.b_mn);
                        tma_load_2d(sb + 16384, &tmB, full, w.b_k + kb * kBlockK, w.b_mn2);
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_bf16(kBlockM, kBlockN, A_MN ? 1 : 0, B_MN ? 1 : 0);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            GemmWork w;
            for (int idx = blockIdx.x; fetch_work(p, idx, total, w) && !abort_flag;
                 idx += gridDim.x) {
                if (!mbar_wait(smem_u32(&bar_tempty[acc]), acc_phase ^ 1u, &abort_flag, p.status))
                    break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kBlockN;
                bool ok = true;
                for (int kb = 0; kb < w.k_iters; ++kb) {
                    if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &abort_flag, p.status)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = tiles_base + stage * kStageBytes;
                    const uint32_t sb = sa + kATileBytes;
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k) {
                        const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, 8192, 1024)
                                                 : make_smem_desc(sa + k * 32, 16, 1024);
                        const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024)
                                                 : make_smem_desc(sb + k * 32, 16, 1024);
                        tc_mma_f16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&bar_empty[stage]));  // stage reusable once these MMAs retire
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                tc_commit(smem_u32(&bar_tfull[acc]));  // accumulator complete
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> global ----------------
        const int quarter = warp & 3;  // TMEM lanes this warp may read: [32*quarter, 32*quarter+32)
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t epi_stage = tiles_base + kStages * kStageBytes + quarter * kEpiStageBytesPerWarp;
        int acc = 0;
        uint32_t acc_phase = 0;
        GemmWork w;
        for (int idx = blockIdx.x; fetch_work(p, idx, total, w) && !abort_flag; idx += gridDim.x) {
            if (!mbar_wait(smem_u32(&bar_tfull[acc]), acc_phase, &abort_flag, p.status)) break;
            tc_fence_after();
            const uint32_t t_row = tmem_base + acc * kBlockN + (uint32_t(quarter * 32) << 16);
            epilogue_tile(p, w, t_row, row_in_tile, epi_stage);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[acc]));
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        // give copies that may still be in flight time to land before the CTA's memory is reused
        uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}


// ---------------------------------------------------------------------------------------------
// CTA-pair form (tcgen05 cta_group::2). Two CTAs of a cluster share one 256 x 256 output tile: CTA r of the pair
// stages rows [128 r, 128 r + 128) of the A tile and rows [128 r, 128 r + 128) of the B tile (its half of N), the
// even CTA issues M = 256 MMAs that read both CTAs' shared memory and write 128 accumulator rows into each CTA's
// TMEM, and each CTA's epilogue warps store their own 128 rows. Per 64-wide k-block a CTA pulls 32 KB from L2
// instead of 48 KB, which is what the single-CTA kernel is short of, and six stages fit instead of four.
// Synchronisation: the pair's TMA loads all complete on the even CTA's "full" barrier (which expects both CTAs'
// bytes); tcgen05.commit multicasts "stage free" and "accumulator ready" to both CTAs; the epilogue warps of both
// CTAs arrive on the even CTA's "accumulator free" barrier. No TMA load uses cluster multicast.
// ---------------------------------------------------------------------------------------------
constexpr int kPairStages = 6;
constexpr int kPairStageBytes = 2 * kATileBytes;  // 128 x 64 of A and 128 x 64 of B
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + 4 * 32 * 256;   // + the epilogue's transposition buffers

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of `local_smem_addr` in the shared memory of CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// tile load whose completion may be counted on the peer CTA's barrier (no multicast: one destination)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
        "{%3, %4}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive on the barrier at this shared-memory offset in every CTA of `cta_mask` once the MMAs issued so far are done
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"(cta_mask)
                 : "memory");
}

// Dense tile walk of the pair kernel: 256-row tiles, groups of 4 tile-rows, column-first inside a group.
__device__ __forceinline__ bool fetch_work_pair(const GemmParams& p, int idx, int total, GemmWork& w) {
    if (idx >= total) return false;
    if (p.list) {
        w = p.list[idx];
        return true;
    }
    const int tiles_m = (p.M + 255) / 256;
    const int group_m = 4;
    const int per_group = group_m * p.tiles_n;
    const int g = idx / per_group;
    const int first_m = g * group_m;
    const int gsz = min(tiles_m - first_m, group_m);
    const int in_g = idx - g * per_group;
    const int tm = first_m + in_g % gsz;
    const int tn = in_g / gsz;
    w.a_mn = tm * 256;
    w.a_k = 0;
    w.b_k = 0;
    w.k_iters = (p.K + kBlockK - 1) / kBlockK;
    w.c_row = tm * 256;
    w.m_valid = min(256, p.M - tm * 256);
    w.pad0 = w.pad1 = 0;
    if (epi_is_glu(p.epi)) {
        w.b_mn = tn * 128;
        w.b_mn2 = p.swiglu_f + tn * 128;
        w.c_col = tn * 128;
        w.n_valid = min(128, p.swiglu_f - tn * 128);
    } else {
        w.b_mn = tn * kBlockN;
        w.b_mn2 = tn * kBlockN + 128;
        w.c_col = tn * kBlockN;
        w.n_valid = min(kBlockN, p.N - tn * kBlockN);
    }
    return true;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[kPairStages], bar_empty[kPairStages], bar_tfull[2], bar_tempty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();      // 0: issues the MMAs, 1: its peer
    const bool leader = rank == 0;
    const uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const bool poisoned = status_poisoned(p.status);   // both CTAs read the same word: they agree

    if (threadIdx.x == 0) {
        abort_flag = poisoned ? 1 : 0;
        for (int s = 0; s < kPairStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);    // the even CTA's: its producer's arrive + both CTAs' bytes
            mbar_init(smem_u32(&bar_empty[s]), 1);   // one multicast commit
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bar_tfull[a]), 1);   // one multicast commit
            mbar_init(smem_u32(&bar_tempty[a]), 8);  // the even CTA's: four epilogue warps of each CTA
        }
        mbar_fence_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(&tmem_base_slot), kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the peer's barriers exist before anything is signalled across the pair
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    const int total = p.list ? *p.list_count : ((p.M + 255) / 256) * p.tiles_n;
    const int first = blockIdx.x >> 1, step = gridDim.x >> 1;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs, each for its halves) ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            GemmWork w;
            for (int idx = first; fetch_work_pair(p, idx, total, w) && !abort_flag; idx += step) {
                const int a_mn = w.a_mn + int(rank) * 128;
                const int b_mn = rank ? w.b_mn2 : w.b_mn;
                for (int kb = 0; kb < w.k_iters; ++kb) {
                    if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, &abort_flag, p.status)) break;
                    if (leader) mbar_expect_tx(smem_u32(&bar_full[stage]), 2 * kPairStageBytes);
                    const uint32_t full = map_to_cta(smem_u32(&bar_full[stage]), 0);
                    const uint32_t sa = tiles_base + stage * kPairStageBytes;
                    const uint32_t sb = sa + kATileBytes;
                    if (A_MN) {
                        tma_load_2d_pair(sa, &tmA, full, a_mn, w.a_k + kb * kBlockK);
                        tma_load_2d_pair(sa + 8192, &tmA, full, a_mn + 64, w.a_k + kb * kBlockK);
                    } else {
                        tma_load_2d_pair(sa, &tmA, full, w.a_k + kb * kBlockK, a_mn);
                    }
                    if (B_MN) {
                        tma_load_2d_pair(sb, &tmB, full, b_mn, w.b_k + kb * kBlockK);
                        tma_load_2d_pair(sb + 8192, &tmB, full, b_mn + 64, w.b_k + kb * kBlockK);
                    } else {
                        tma_load_2d_pair(sb, &tmB, full, w.b_k + kb * kBlockK, b_mn);
                    }
                    if (++stage == kPairStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (even CTA only) ----------------
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = make_idesc_bf16(256, kBlockN, A_MN ? 1 : 0, B_MN ? 1 : 0);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            GemmWork w;
            for (int idx = first; fetch_work_pair(p, idx, total, w) && !abort_flag; idx += step) {
                if (!mbar_wait(smem_u32(&bar_tempty[acc]), acc_phase ^ 1u, &abort_flag, p.status)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kBlockN;
                bool ok = true;
                for (int kb = 0; kb < w.k_iters; ++kb) {
                    if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &abort_flag, p.status)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = tiles_base + stage * kPairStageBytes;
                    const uint32_t sb = sa + kATileBytes;
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k) {
                        const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, 8192, 1024)
                                                 : make_smem_desc(sa + k * 32, 16, 1024);
                        const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024)
                                                 : make_smem_desc(sb + k * 32, 16, 1024);
                        tc_mma_f16_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tc_commit_pair(smem_u32(&bar_empty[stage]), 3);   // both CTAs' producers may refill the stage
                    if (++stage == kPairStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                tc_commit_pair(smem_u32(&bar_tfull[acc]), 3);         // both CTAs' epilogues may read
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ---------------- epilogue (both CTAs, each its own 128 rows) ----------------
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t epi_stage = tiles_base + kPairStages * kPairStageBytes + quarter * kEpiStageBytesPerWarp;
        int acc = 0;
        uint32_t acc_phase = 0;
        GemmWork w;
        for (int idx = first; fetch_work_pair(p, idx, total, w) && !abort_flag; idx += step) {
            if (!mbar_wait(smem_u32(&bar_tfull[acc]), acc_phase, &abort_flag, p.status)) break;
            tc_fence_after();
            const uint32_t t_row = tmem_base + acc * kBlockN + (uint32_t(quarter * 32) << 16);
            GemmWork mine = w;
            mine.c_row = w.c_row + int(rank) * 128;
            mine.m_valid = max(0, min(128, w.m_valid - int(rank) * 128));
            epilogue_tile(p, mine, t_row, row_in_tile, epi_stage);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&bar_tempty[acc]), 0));
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (abort_flag && !poisoned) {
        uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    cluster_sync_all();          // nothing of the pair is in flight towards the other CTA's memory any more
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------
// Tile lists for grouped (per-expert) products, built on the device from the expert segments.
// Segment e occupies rows [seg_start[e], seg_start[e] + seg_rows[e]) of the grouped operand;
// seg_start is a multiple of 128 and the rows between segments are zero.
// ---------------------------------------------------------------------------------------------

// Rows grouped along M:  C[rows of e] = A[rows of e] * op(B_e).
//   b_mn_stride / b_k_stride: how far expert e's weights sit along B's N / reduction coordinate.
__global__ void plan_grouped_m_kernel(const int* __restrict__ seg_start,
                                      const int* __restrict__ seg_rows, int num_experts, int n_cols,
                                      int k_dim, int b_mn_stride, int b_k_stride, int swiglu_f,
                                      GemmWork* __restrict__ list, int* __restrict__ count,
                                      int max_items, int tile_m) {
    // tile_m: 128 (one CTA per tile) or 256 (a CTA pair per tile; the second half of a segment's last tile may
    // reach past the segment's padded rows, in which case only 128 rows of it are stored)
    __shared__ int base[1025];
    const int tile_n = swiglu_f ? 128 : kBlockN;
    const int width = swiglu_f ? swiglu_f : n_cols;
    const int tiles_n = (width + tile_n - 1) / tile_n;
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < num_experts; ++e) {
            base[e] = acc;
            acc += ((seg_rows[e] + tile_m - 1) / tile_m) * tiles_n;
        }
        base[num_experts] = acc;
        *count = min(acc, max_items);
    }
    __syncthreads();
    for (int e = 0; e < num_experts; ++e) {
        const int rows = seg_rows[e];
        const int n_items = base[e + 1] - base[e];
        for (int i = threadIdx.x; i < n_items; i += blockDim.x) {
            if (base[e] + i >= max_items) continue;
            const int tm = i / tiles_n, tn = i % tiles_n;
            GemmWork w;
            w.a_mn = seg_start[e] + tm * tile_m;
            w.a_k = 0;
            w.b_k = e * b_k_stride;
            w.k_iters = (k_dim + kBlockK - 1) / kBlockK;
            w.c_row = w.a_mn;
            // whole 128-row blocks are written: the pad rows of a segment are zero on input, so they come
            // out as zeros and later reductions over padded row ranges stay finite
            const int padded = (rows + kBlockM - 1) / kBlockM * kBlockM;
            w.m_valid = min(tile_m, padded - tm * tile_m);
            if (swiglu_f) {
                w.b_mn = e * b_mn_stride + tn * 128;
                w.b_mn2 = e * b_mn_stride + swiglu_f + tn * 128;
                w.c_col = tn * 128;
                w.n_valid = min(128, swiglu_f - tn * 128);
            } else {
                w.b_mn = e * b_mn_stride + tn * kBlockN;
                w.b_mn2 = w.b_mn + 128;
                w.c_col = tn * kBlockN;
                w.n_valid = min(kBlockN, n_cols - tn * kBlockN);
            }
            w.pad0 = w.pad1 = 0;
            list[base[e] + i] = w;
        }
    }
}

// Rows grouped along the reduction:  C_e[m, n] = sum_{r in rows of e} A[r, m] * B[r, n]
// (the per-expert weight gradient dW_e = dY_e^T X_e). C is viewed as [E * m_dim, n_dim].
__global__ void plan_grouped_k_kernel(const int* __restrict__ seg_start,
                                      const int* __restrict__ seg_rows, int num_experts, int m_dim,
                                      int n_dim, GemmWork* __restrict__ list,
                                      int* __restrict__ count, int max_items, int tile_m) {
    const int tiles_m = (m_dim + tile_m - 1) / tile_m;
    const int tiles_n = (n_dim + kBlockN - 1) / kBlockN;
    const int per_e = tiles_m * tiles_n;
    const int total = min(per_e * num_experts, max_items);
    if (blockIdx.x == 0 && threadIdx.x == 0) *count = total;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int e = i / per_e, r = i % per_e;
        const int tm = r / tiles_n, tn = r % tiles_n;
        GemmWork w;
        w.a_mn = tm * tile_m;
        w.b_mn = tn * kBlockN;
        w.b_mn2 = w.b_mn + 128;
        w.a_k = seg_start[e];
        w.b_k = seg_start[e];
        w.k_iters = (seg_rows[e] + kBlockK - 1) / kBlockK;
        w.c_row = e * m_dim + tm * tile_m;
        w.c_col = tn * kBlockN;
        w.m_valid = min(tile_m, m_dim - tm * tile_m);
        w.n_valid = min(kBlockN, n_dim - tn * kBlockN);
        w.pad0 = w.pad1 = 0;
        list[i] = w;
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D bf16 tensor [rows, cols] with `ld` elements between rows; box = 64 columns x box_rows.
int make_tmap_bf16(CUtensorMap* m, const void* base, long long rows, long long cols, long long ld,
                   int box_rows) {
    // The encoder is a driver call: make sure this thread has the device's context current
    // (a fresh autograd worker thread may not have made any runtime call yet).
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -4;
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return -1;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (ld % 8) != 0) return -2;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        fprintf(stderr, "halo: cuTensorMapEncodeTiled failed (%d): base=%p rows=%lld cols=%lld ld=%lld box_rows=%d\n",
                (int)r, base, rows, cols, ld, box_rows);
        return -3;
    }
    return 0;
}

static int g_num_sms = 0;
static int num_sms() {
    if (!g_num_sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
        if (g_num_sms <= 0) g_num_sms = 148;
    }
    return g_num_sms;
}

constexpr int kGemmSmemBytes = kStages * kStageBytes + 1024 + 4 * kEpiStageBytesPerWarp;

template <bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                       cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_bf16_kernel<A_MN, B_MN>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kGemmSmemBytes) != cudaSuccess)
            return -10;
        configured = true;
    }
    gemm_bf16_kernel<A_MN, B_MN><<<grid, kGemmThreads, kGemmSmemBytes, stream>>>(ta, tb, p);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

static int dispatch_gemm(int a_mn, int b_mn, const CUtensorMap& ta, const CUtensorMap& tb,
                         const GemmParams& p, int grid, cudaStream_t s) {
    if (!a_mn && !b_mn) return launch_gemm<false, false>(ta, tb, p, grid, s);
    if (!a_mn && b_mn) return launch_gemm<false, true>(ta, tb, p, grid, s);
    if (a_mn && b_mn) return launch_gemm<true, true>(ta, tb, p, grid, s);
    return launch_gemm<true, false>(ta, tb, p, grid, s);
}

template <bool A_MN, bool B_MN>
static int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int n_pairs,
                            cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_bf16_pair_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kPairSmemBytes) != cudaSuccess)
            return -10;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * n_pairs, 1, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = kPairSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, gemm_bf16_pair_kernel<A_MN, B_MN>, ta, tb, p) != cudaSuccess) return -11;
    return 0;
}

static int dispatch_gemm_pair(int a_mn, int b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                              int n_pairs, cudaStream_t s) {
    if (!a_mn && !b_mn) return launch_gemm_pair<false, false>(ta, tb, p, n_pairs, s);
    if (!a_mn && b_mn) return launch_gemm_pair<false, true>(ta, tb, p, n_pairs, s);
    if (a_mn && b_mn) return launch_gemm_pair<true, true>(ta, tb, p, n_pairs, s);
    return launch_gemm_pair<true, false>(ta, tb, p, n_pairs, s);
}

// HALO_GEMM_PAIR: 1 (default) = the CTA-pair kernel where it measured faster, 0 = never, 2 = everywhere
static int g_use_pair = -1;
static bool use_pair() {
    if (g_use_pair < 0) {
        const char* e = getenv("HALO_GEMM_PAIR");
        g_use_pair = e ? atoi(e) : 1;
    }
    return g_use_pair != 0;
}

}  // namespace halo

using namespace halo;

extern "C" {

// Dense product. A is [a_rows, a_cols] with leading dimension lda, likewise B.
//   a_mn_major = 0: A is [M, K] (K contiguous);  1: A is [K, M] (M contiguous)
//   b_mn_major = 0: B is [N, K] (K contiguous);  1: B is [K, N] (N contiguous)
// epi selects the epilogue (store / accumulate, bf16 / fp32, SwiGLU). For SwiGLU, B is the
// stacked [2F, K] weight (gate rows then up rows), N must be 2F and C is [M, F].
int halo_gemm_bf16(const void* A, const void* B, void* C, void* aux, int M, int N, int K,
                   long long lda, long long ldb, long long ldc, long long ld_aux, int a_mn_major,
                   int b_mn_major, int epi, float alpha, int* status, void* stream) {
    if (M <= 0 || N <= 0 || K < 0) return 0;
    CUtensorMap ta, tb;
    int rc;
    if (a_mn_major) rc = make_tmap_bf16(&ta, A, K, M, lda, 64);
    else rc = make_tmap_bf16(&ta, A, M, K, lda, 128);
    if (rc) return rc;
    if (b_mn_major) rc = make_tmap_bf16(&tb, B, K, N, ldb, 64);
    else rc = make_tmap_bf16(&tb, B, N, K, ldb, 128);
    if (rc) return rc * 10;
    GemmParams p{};
    p.C = C; p.aux = aux; p.ldc = ldc; p.ld_aux = ld_aux; p.epi = epi; p.alpha = alpha;
    p.M = M; p.N = N; p.K = K;
    p.tiles_m = (M + kBlockM - 1) / kBlockM;
    if (epi_is_glu(epi)) {
        if (N % 2) return -20;
        p.swiglu_f = N / 2;
        p.tiles_n = (p.swiglu_f + 127) / 128;
    } else {
        p.swiglu_f = 0;
        p.tiles_n = (N + kBlockN - 1) / kBlockN;
    }
    p.list = nullptr; p.list_count = nullptr; p.status = status;
    // measured: the pair kernel wins on mainloop-bound products with narrow outputs; wide outputs (the vocabulary
    // head, large square products), short reductions and the SwiGLU epilogue run faster on the single-CTA kernel
    if (use_pair() && (g_use_pair == 2 || (p.tiles_n <= 24 && K >= 1536 && !epi_is_glu(epi)))) {
        const long long pair_tiles = (long long)((M + 255) / 256) * p.tiles_n;
        const int max_pairs = num_sms() / 2;
        return dispatch_gemm_pair(a_mn_major, b_mn_major, ta, tb, p, (int)(pair_tiles < max_pairs ? pair_tiles : max_pairs),
                                  (cudaStream_t)stream);
    }
    long long tiles = (long long)p.tiles_m * p.tiles_n;
    int grid = (int)(tiles < num_sms() ? tiles : num_sms());
    return dispatch_gemm(a_mn_major, b_mn_major, ta, tb, p, grid, (cudaStream_t)stream);
}

// Row-parallel product fused with the reduce-scatter's transfer: C_partial = A B^T is never stored locally; every
// tile goes into slot `rank` of its owner's staging area (see GemmParams). `stage_ptrs`: HOST array of n_ranks
// device pointers (rank d's [n_ranks][rows_per_rank][N] bf16 staging area as mapped into this process). After the
// kernel and a barrier over the ranks, each rank sums its n_ranks slots.
int halo_gemm_bf16_reduce_scatter(const void* A, const void* B, void* const* stage_ptrs, int n_ranks, int rank,
                                  int M, int N, int K, long long lda, long long ldb, int b_mn_major, int* status,
                                  void* stream) {
    if (n_ranks < 2 || n_ranks > 8 || M % n_ranks) return -21;
    const int rows = M / n_ranks;
    if (rows % kBlockM || N % 8) return -22;
    CUtensorMap ta, tb;
    int rc = make_tmap_bf16(&ta, A, M, K, lda, 128);
    if (rc) return rc;
    if (b_mn_major) rc = make_tmap_bf16(&tb, B, K, N, ldb, 64);
    else rc = make_tmap_bf16(&tb, B, N, K, ldb, 128);
    if (rc) return rc * 10;
    GemmParams p{};
    p.C = nullptr; p.aux = nullptr; p.ldc = N; p.ld_aux = 0; p.epi = kEpiStoreBf16; p.alpha = 1.f;
    p.M = M; p.N = N; p.K = K;
    p.tiles_m = M / kBlockM;
    p.tiles_n = (N + kBlockN - 1) / kBlockN;
    p.swiglu_f = 0;
    p.list = nullptr; p.list_count = nullptr; p.status = status;
    for (int i = 0; i < n_ranks; ++i) p.c_peers[i] = stage_ptrs[i];
    p.rs_ranks = n_ranks; p.rs_rank = rank; p.rs_rows = rows;
    long long tiles = (long long)p.tiles_m * p.tiles_n;
    int grid = (int)(tiles < num_sms() ? tiles : num_sms());
    return dispatch_gemm(0, b_mn_major, ta, tb, p, grid, (cudaStream_t)stream);
}

// Product over a device-resident tile list (see plan_grouped_*). The operands are described as
// plain 2-D tensors; the list carries every coordinate.
int halo_gemm_bf16_list(const void* A, long long a_rows, long long a_cols, long long lda,
                        const void* B, long long b_rows, long long b_cols, long long ldb, void* C,
                        void* aux, long long ldc, long long ld_aux, int a_mn_major, int b_mn_major,
                        int epi, float alpha, int swiglu_f, const void* list, const int* list_count,
                        int* status, void* stream, int pair) {
    CUtensorMap ta, tb;
    int rc = make_tmap_bf16(&ta, A, a_rows, a_cols, lda, a_mn_major ? 64 : 128);
    if (rc) return rc;
    rc = make_tmap_bf16(&tb, B, b_rows, b_cols, ldb, b_mn_major ? 64 : 128);
    if (rc) return rc * 10;
    GemmParams p{};
    p.C = C; p.aux = aux; p.ldc = ldc; p.ld_aux = ld_aux; p.epi = epi; p.alpha = alpha;
    p.swiglu_f = swiglu_f;
    p.list = reinterpret_cast<const GemmWork*>(list);
    p.list_count = list_count;
    p.status = status;
    // `pair`: the list holds 256-row tiles planned for the CTA-pair kernel (see halo_plan_grouped_*)
    if (pair) return dispatch_gemm_pair(a_mn_major, b_mn_major, ta, tb, p, num_sms() / 2, (cudaStream_t)stream);
    return dispatch_gemm(a_mn_major, b_mn_major, ta, tb, p, num_sms(), (cudaStream_t)stream);
}

// As halo_gemm_bf16_list with the clamped-GLU epilogue: `bias` is the expert bias bank [E, 2F] in bf16, read through
// the tile's B coordinates (the list must have been planned with swiglu_f = F and b_mn_stride = 2F, so that a tile's
// gate / up column origins are also its origins in the bias bank).
int halo_gemm_bf16_list_glu(const void* A, long long a_rows, long long a_cols, long long lda,
                            const void* B, long long b_rows, long long b_cols, long long ldb, void* C,
                            void* aux, long long ldc, long long ld_aux, int swiglu_f, const void* bias, float limit,
                            float glu_alpha, const void* list, const int* list_count, int* status, void* stream) {
    if (!bias || swiglu_f <= 0 || swiglu_f % 8) return -1;
    CUtensorMap ta, tb;
    int rc = make_tmap_bf16(&ta, A, a_rows, a_cols, lda, 128);
    if (rc) return rc;
    rc = make_tmap_bf16(&tb, B, b_rows, b_cols, ldb, 128);
    if (rc) return rc * 10;
    GemmParams p{};
    p.C = C; p.aux = aux; p.ldc = ldc; p.ld_aux = ld_aux; p.epi = kEpiClampedGlu; p.alpha = 1.f;
    p.swiglu_f = swiglu_f;
    p.list = reinterpret_cast<const GemmWork*>(list);
    p.list_count = list_count;
    p.status = status;
    p.glu_bias = bias; p.glu_limit = limit; p.glu_alpha = glu_alpha;
    return dispatch_gemm(0, 0, ta, tb, p, num_sms(), (cudaStream_t)stream);
}

int halo_plan_grouped_m(const int* seg_start, const int* seg_rows, int num_experts, int n_cols,
                        int k_dim, int b_mn_stride, int b_k_stride, int swiglu_f, void* list,
                        int* count, int max_items, void* stream, int pair) {
    if (num_experts > 1024) return -1;
    plan_grouped_m_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(
        seg_start, seg_rows, num_experts, n_cols, k_dim, b_mn_stride, b_k_stride, swiglu_f,
        reinterpret_cast<GemmWork*>(list), count, max_items, pair ? 256 : kBlockM);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int halo_plan_grouped_k(const int* seg_start, const int* seg_rows, int num_experts, int m_dim,
                        int n_dim, void* list, int* count, int max_items, void* stream, int pair) {
    plan_grouped_k_kernel<<<32, 256, 0, (cudaStream_t)stream>>>(
        seg_start, seg_rows, num_experts, m_dim, n_dim, reinterpret_cast<GemmWork*>(list), count,
        max_items, pair ? 256 : kBlockM);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int halo_gemm_work_bytes() { return (int)sizeof(GemmWork); }

// 1 unless HALO_GEMM_PAIR=0: callers of the list entry points may plan 256-row tiles for the CTA-pair kernel
int halo_gemm_pair_enabled() { return use_pair() ? g_use_pair : 0; }

}  // extern "C"
