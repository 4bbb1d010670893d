// Causal flash attention for packed (variable-length) rows on sm_100a, head_dim 128, grouped-query
// heads. Forward and backward run on tcgen05 tensor cores with the score tiles in tensor memory:
//
//   forward   one CTA per (128-query tile, head): S = Q K^T lands in TMEM, four softmax warps
//             read it with tcgen05.ld, write P (bf16) into swizzled shared memory, a second MMA
//             forms P V in TMEM, and the running output is rescaled in registers.
//   backward  two deterministic kernels (no atomics): one owns a 128-key tile of one kv head and
//             accumulates dK, dV in TMEM over every query tile / head that sees it; the other owns
//             a 128-query tile and accumulates dQ in TMEM over its key tiles.
//
// Documents are delimited by the tile work list (built from cu_seqlens): a query tile only visits
// key tiles of its own document, so packed rows never attend across documents.
// K/V tiles are fetched per CTA with TMA (no cluster broadcast).
//
// Stands where the reference calls FlashAttention-4 / FlashAttention-2 varlen kernels
// (halo/models/attention/selection.py:94-100, 383-462).
#include "sm100_common.cuh"

#include <stdio.h>
#include <stdlib.h>

namespace halo {

constexpr int kHd = 128;
constexpr float kLog2e = 1.4426950408889634f;

int make_tmap_bf16(CUtensorMap* m, const void* base, long long rows, long long cols, long long ld,
                   int box_rows);  // gemm_sm100.cu

// 2^x on the special-function unit (one MUFU op; inputs here are <= 8 after max subtraction)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (M = 128 rows on the 128 lanes, 16 bf16 of the reduction as 8 packed
// 32-bit columns) is read from tensor memory.
__device__ __forceinline__ void tc_mma_f16_tmem_a(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                  uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// A warp writes its 32 TMEM lanes x 16 consecutive 32-bit columns; thread i writes lane i.
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// byte offset of the 16-byte chunk holding column `col` (multiple of 8) of row `row` inside a
// [rows x 64] bf16 half-tile stored with the 128-byte swizzle
__device__ __forceinline__ uint32_t swz_off(int row, int col) {
    return (uint32_t)(row * 128 + ((((col >> 3) ^ row) & 7) << 4));
}

// Context parallelism: the kernels work in the packed row's GLOBAL row numbers (masks, document ends, tile starts);
// only addresses are translated. A row belongs to one piece of the row; a piece has an owner rank and a first row in that
// rank's local order. Queries, outputs and statistics are local tensors; a key / value tile is read from its owner's
// published buffer through that rank's tensor map (plain per-CTA TMA loads; the memory may be a peer GPU's).
// Two tables are passed: one for query rows (always this rank's real pieces) and one for key rows. The key table is either
// the same pieces with one tensor map per owner (every tile read crosses NVLink: good when few foreign rows are touched),
// or a single piece covering the whole row, owned by nobody (`my_rank = -1`), when the needed foreign rows were first
// fetched once into a local mirror indexed by global row; dK / dV then all go to the staging buffer at their global rows.
struct CpMap {
    int n_pieces;
    int my_rank;
    int bound[17];   // global first row of every piece, then the row's length
    int owner[16];
    int loc[16];     // first row of the piece in its owner's local order
    int stage[16];   // row of a foreign piece's first row in this rank's dK / dV staging buffer (-1: none)
};
struct PeerMaps {
    CUtensorMap k[8];
    CUtensorMap v[8];
};
// What a context-parallel instantiation takes beyond the plain kernel's arguments; the plain instantiation carries one
// unused byte instead, so its parameter block (and its launch cost on lists of many short CTAs) stays what it was.
template <bool kCP>
struct CpArgs {
    PeerMaps peers;
    CpMap cp;      // query rows
    CpMap cpk;     // key rows
};
template <>
struct CpArgs<false> {
    char unused;
};

__device__ __forceinline__ int cp_piece(const CpMap& m, int row) {
    int pc = 0;
    while (pc + 1 < m.n_pieces && row >= m.bound[pc + 1]) ++pc;
    return pc;
}

struct FwdWork {
    int q0;        // first query row of the tile
    int kv0;       // first key row the tile may see (its document's first row)
    int n_kv;      // number of 128-key tiles to visit; the last one is the diagonal tile
    int q_end;     // one past the document's last row
};

struct AttnParams {
    const FwdWork* work;
    void* O;              // [T, Hq*128] bf16
    float* lse;           // [Hq, T]
    long long ldo;
    long long T;
    int Hq, Hkv;
    float scale;          // 1/sqrt(head_dim)
    int* status;
    int window;           // > 0: a query sees only the last `window` keys up to itself (sliding-window layers); 0: all earlier keys
    const float* sinks;   // [Hq] or null: one extra logit per head that joins every row's softmax and carries no value
};

// Softmax denominator with the head's sink logit: l is the sum of exp(score - m_nat) over the keys, m_nat the row's
// reference maximum in natural-log units. The exponent is capped so that a sink far above every score gives a large
// finite denominator (an output of zeros) rather than infinity.
__device__ __forceinline__ float add_sink(float l, float m_nat, const float* sinks, int head) {
    return sinks ? l + __expf(fminf(sinks[head] - m_nat, 80.f)) : l;
}

constexpr int kFwdThreads = 192;
constexpr int kTileBytes = 128 * 128 * 2;                              // 32 KiB: a 128x128 bf16 tile
constexpr int kFwdSmem = kTileBytes * (1 + 1 + 2 * 2) + 1024;          // Q, P, 2 x (K, V)

__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_q, bar_kv_full[2], bar_kv_empty[2], bar_s_full, bar_p_ready, bar_o_full;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = base, sP = base + kTileBytes, sKV = base + 2 * kTileBytes;
    const int head = blockIdx.x;
    const int kv_head = head / (p.Hq / p.Hkv);
    const FwdWork w = p.work[blockIdx.y];

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar_q), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&bar_kv_full[s]), 1);
            mbar_init(smem_u32(&bar_kv_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_s_full), 1);
        mbar_init(smem_u32(&bar_p_ready), 128);
        mbar_init(smem_u32(&bar_o_full), 1);
        mbar_fence_init();
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(&tmem_slot), 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tS = tmem_slot, tO = tmem_slot + 128;

    if (warp == 4) {
        if (lane == 0) {
            // ---------------- TMA producer ----------------
            mbar_expect_tx(smem_u32(&bar_q), kTileBytes);
            tma_load_2d(sQ, &tmQ, smem_u32(&bar_q), head * kHd, w.q0);
            tma_load_2d(sQ + 16384, &tmQ, smem_u32(&bar_q), head * kHd + 64, w.q0);
            for (int j = 0; j < w.n_kv; ++j) {
                const int st = j & 1;
                if (!mbar_wait(smem_u32(&bar_kv_empty[st]), ((j >> 1) & 1) ^ 1u, &abort_flag, p.status)) break;
                const uint32_t full = smem_u32(&bar_kv_full[st]);
                const uint32_t sK = sKV + st * 2 * kTileBytes, sV = sK + kTileBytes;
                const int kr = w.kv0 + j * 128;
                mbar_expect_tx(full, 2 * kTileBytes);
                tma_load_2d(sK, &tmK, full, kv_head * kHd, kr);
                tma_load_2d(sK + 16384, &tmK, full, kv_head * kHd + 64, kr);
                tma_load_2d(sV, &tmV, full, kv_head * kHd, kr);
                tma_load_2d(sV + 16384, &tmV, full, kv_head * kHd + 64, kr);
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {
            // ---------------- MMA issuer ----------------
            constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);   // S = Q K^T
            constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, 0, 1);   // O = P V  (V is N-major)
            bool ok = mbar_wait(smem_u32(&bar_q), 0, &abort_flag, p.status);
            for (int j = 0; ok && j < w.n_kv; ++j) {
                const int st = j & 1;
                const uint32_t sK = sKV + st * 2 * kTileBytes, sV = sK + kTileBytes;
                if (!mbar_wait(smem_u32(&bar_kv_full[st]), (j >> 1) & 1, &abort_flag, p.status)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
                    tc_mma_f16(tS, make_smem_desc(sQ + off, 16, 1024), make_smem_desc(sK + off, 16, 1024),
                               idesc_s, ks != 0);
                }
                tc_commit(smem_u32(&bar_s_full));
                if (!mbar_wait(smem_u32(&bar_p_ready), j & 1, &abort_flag, p.status)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    // P: K-major A, 16 keys per step; V: N-major B, 16 key rows (2048 bytes) per step
                    const uint32_t offp = (ks >> 2) * 16384 + (ks & 3) * 32;
                    tc_mma_f16(tO, make_smem_desc(sP + offp, 16, 1024),
                               make_smem_desc(sV + ks * 2048, 16384, 1024), idesc_o, ks != 0);
                }
                tc_commit(smem_u32(&bar_o_full));
                tc_commit(smem_u32(&bar_kv_empty[st]));
            }
        }
    } else {
        // ---------------- softmax / output warps: thread = query row ----------------
        const int row = warp * 32 + lane;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const float c = p.scale * kLog2e;
        float m = -INFINITY, l = 0.f;
        float acc[128];
#pragma unroll
        for (int i = 0; i < 128; ++i) acc[i] = 0.f;
        bool ok = true;
        for (int j = 0; j < w.n_kv; ++j) {
            if (!mbar_wait(smem_u32(&bar_s_full), j & 1, &abort_flag, p.status)) { ok = false; break; }
            tc_fence_after();
            const bool diag = (j == w.n_kv - 1);
            float mx = m;
#pragma unroll 1
            for (int cc = 0; cc < 128; cc += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tS + lane_base + cc, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float s = __uint_as_float(r[i]);
                    if (!diag || cc + i <= row) mx = fmaxf(mx, s);
                }
            }
            const float alpha = fast_exp2((m - mx) * c);
            const float mc = mx * c;
            float rs = 0.f;
#pragma unroll 1
            for (int cc = 0; cc < 128; cc += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tS + lane_base + cc, r);
                tmem_ld_wait();
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0 = fast_exp2(__uint_as_float(r[i]) * c - mc);
                    float p1 = fast_exp2(__uint_as_float(r[i + 1]) * c - mc);
                    if (diag) {
                        if (cc + i > row) p0 = 0.f;
                        if (cc + i + 1 > row) p1 = 0.f;
                    }
                    pk[i >> 1] = pack_bf16(p0, p1);
                    // sum what the second MMA will actually see
                    const __nv_bfloat162 pb = *reinterpret_cast<__nv_bfloat162*>(&pk[i >> 1]);
                    const float2 pf = __bfloat1622float2(pb);
                    rs += pf.x + pf.y;
                }
                const uint32_t half = sP + (cc >> 6) * 16384;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint32_t a = half + swz_off(row, (cc & 63) + q * 8);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(pk[4 * q]),
                                 "r"(pk[4 * q + 1]), "r"(pk[4 * q + 2]), "r"(pk[4 * q + 3])
                                 : "memory");
                }
            }
            l = l * alpha + rs;
            m = mx;
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(smem_u32(&bar_p_ready));
            if (!mbar_wait(smem_u32(&bar_o_full), j & 1, &abort_flag, p.status)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int cc = 0; cc < 128; cc += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tO + lane_base + cc, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[cc + i] = acc[cc + i] * alpha + __uint_as_float(r[i]);
            }
        }
        const long long grow = (long long)w.q0 + row;
        if (ok && grow < w.q_end) {
            l = add_sink(l, m * p.scale, p.sinks, head);
            const float inv = 1.f / l;
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.O) + grow * p.ldo + head * kHd;
#pragma unroll
            for (int i = 0; i < 128; i += 8) {
                *reinterpret_cast<uint4*>(out + i) =
                    make_uint4(pack_bf16(acc[i] * inv, acc[i + 1] * inv), pack_bf16(acc[i + 2] * inv, acc[i + 3] * inv),
                               pack_bf16(acc[i + 4] * inv, acc[i + 5] * inv), pack_bf16(acc[i + 6] * inv, acc[i + 7] * inv));
            }
            p.lse[(long long)head * p.T + grow] = m * p.scale + logf(l);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_slot, 256);
    }
}

// ---------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------
// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (t, h)
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                  float* __restrict__ delta, long long T, int Hq, long long ld_do, long long ld_o) {
    const int lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (wid >= T * Hq) return;
    const long long t = wid / Hq;
    const int h = (int)(wid % Hq);
    const uint2 a = *reinterpret_cast<const uint2*>(dO + t * ld_do + h * kHd + lane * 4);
    const uint2 b = *reinterpret_cast<const uint2*>(O + t * ld_o + h * kHd + lane * 4);
    const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&b);
    float s = 0.f;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        const float2 x = __bfloat1622float2(ah[q]), y = __bfloat1622float2(bh[q]);
        s += x.x * y.x + x.y * y.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) delta[(long long)h * T + t] = s;
}

struct BwdKvWork {
    int kv0;      // first key row of the 128-key tile
    int q_begin;  // first query row that can see it (== kv0)
    int n_q;      // number of 64-query sub-tiles to visit, starting at q_begin
    int q_end;    // one past the document's last row
};

struct BwdParams {
    const void* work;
    const float* lse;    // [Hq, T]
    const float* delta;  // [Hq, T]
    void* dQ;            // [T, ld_dq]
    void* dK;
    void* dV;
    long long ld_dq, ld_dk, ld_dv;
    long long T;
    int Hq, Hkv;
    float scale;
    int* status;
    void* dK_stage;      // context parallelism: dK / dV of key tiles another rank owns ([rows, ld_stage])
    void* dV_stage;
    long long ld_stage;
    int window;          // as in the forward
};

struct BwdKvWorkCp {     // context parallelism: the local queries that see a key tile, as up to two runs (one per local piece)
    int kv0, q_begin, n_q, q_end;
    int q_begin2, n_q2, pad0, pad1;
};

constexpr int kBwdThreads = 192;
constexpr int kHalfTile = 64 * 128 * 2;  // 16 KiB: a 64 x 128 bf16 tile
// K, V (32 KiB each), P^T and dS^T (128 x 64, 16 KiB each), 2 stages of (Q, dO) 64 x 128
constexpr int kBwdKvSmem = 2 * kTileBytes + 2 * kHalfTile + 2 * 2 * kHalfTile + 1024;

// One CTA per (128-key tile, kv head). For every q head of the group and every 64-query sub-tile:
//   S^T = K Q^T, dP^T = V dO^T  (TMEM, 64 columns each)
//   P^T = exp(S^T * scale - lse),  dS^T = P^T * (dP^T - delta) * scale
//   dV += P^T dO,  dK += dS^T Q   (TMEM accumulators, 128 columns each)
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                     const BwdParams p) {
    if (status_poisoned(p.status)) return;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_kv, bar_q_full[2], bar_q_empty[2], bar_s_full, bar_p_ready, bar_ds_ready,
        bar_dv_done, bar_acc_done, bar_stats;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;
    __shared__ float s_lse[2][64], s_delta[2][64];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sK = base, sV = base + kTileBytes, sPT = base + 2 * kTileBytes,
                   sDS = sPT + kHalfTile, sQdO = sDS + kHalfTile;
    const int kv_head = blockIdx.x;
    const int group = p.Hq / p.Hkv;
    const BwdKvWork w = reinterpret_cast<const BwdKvWork*>(p.work)[blockIdx.y];
    const int n_iter = w.n_q * group;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar_kv), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&bar_q_full[s]), 1);
            mbar_init(smem_u32(&bar_q_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_s_full), 1);
        mbar_init(smem_u32(&bar_p_ready), 128);
        mbar_init(smem_u32(&bar_ds_ready), 128);
        mbar_init(smem_u32(&bar_dv_done), 1);
        mbar_init(smem_u32(&bar_acc_done), 1);
        mbar_init(smem_u32(&bar_stats), 64);
        mbar_fence_init();
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(&tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tS = tmem_slot, tDP = tmem_slot + 64, tDV = tmem_slot + 128, tDK = tmem_slot + 256;

    if (warp == 4) {
        if (lane == 0) {
            mbar_expect_tx(smem_u32(&bar_kv), 2 * kTileBytes);
            tma_load_2d(sK, &tmK, smem_u32(&bar_kv), kv_head * kHd, w.kv0);
            tma_load_2d(sK + 16384, &tmK, smem_u32(&bar_kv), kv_head * kHd + 64, w.kv0);
            tma_load_2d(sV, &tmV, smem_u32(&bar_kv), kv_head * kHd, w.kv0);
            tma_load_2d(sV + 16384, &tmV, smem_u32(&bar_kv), kv_head * kHd + 64, w.kv0);
            for (int it = 0; it < n_iter; ++it) {
                const int st = it & 1;
                if (!mbar_wait(smem_u32(&bar_q_empty[st]), ((it >> 1) & 1) ^ 1u, &abort_flag, p.status)) break;
                const int h = kv_head * group + it % group;
                const int qr = w.q_begin + (it / group) * 64;
                const uint32_t full = smem_u32(&bar_q_full[st]);
                const uint32_t sQ = sQdO + st * 2 * kHalfTile, sdO = sQ + kHalfTile;
                mbar_expect_tx(full, 2 * kHalfTile);
                // 64 rows x 128 columns as two 64 x 64 boxes, 8 KiB each
                tma_load_2d(sQ, &tmQ, full, h * kHd, qr);
                tma_load_2d(sQ + 8192, &tmQ, full, h * kHd + 64, qr);
                tma_load_2d(sdO, &tmdO, full, h * kHd, qr);
                tma_load_2d(sdO + 8192, &tmdO, full, h * kHd + 64, qr);
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {
            constexpr uint32_t idesc_st = make_idesc_bf16(128, 64, 0, 0);   // [keys x q] = K Q^T, V dO^T
            constexpr uint32_t idesc_acc = make_idesc_bf16(128, 128, 0, 1); // [keys x hd] = P^T dO, dS^T Q
            bool ok = mbar_wait(smem_u32(&bar_kv), 0, &abort_flag, p.status);
            for (int it = 0; ok && it < n_iter; ++it) {
                const int st = it & 1;
                const uint32_t sQ = sQdO + st * 2 * kHalfTile, sdO = sQ + kHalfTile;
                if (!mbar_wait(smem_u32(&bar_q_full[st]), (it >> 1) & 1, &abort_flag, p.status)) break;
                // the previous iteration's dK product must have drained dS^T / S before they are reused
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t offa = (ks >> 2) * 16384 + (ks & 3) * 32;  // K / V: 128-row halves
                    const uint32_t offb = (ks >> 2) * 8192 + (ks & 3) * 32;   // Q / dO: 64-row halves
                    tc_mma_f16(tS, make_smem_desc(sK + offa, 16, 1024), make_smem_desc(sQ + offb, 16, 1024),
                               idesc_st, ks != 0);
                }
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t offa = (ks >> 2) * 16384 + (ks & 3) * 32;
                    const uint32_t offb = (ks >> 2) * 8192 + (ks & 3) * 32;
                    tc_mma_f16(tDP, make_smem_desc(sV + offa, 16, 1024), make_smem_desc(sdO + offb, 16, 1024),
                               idesc_st, ks != 0);
                }
                tc_commit(smem_u32(&bar_s_full));
                if (!mbar_wait(smem_u32(&bar_p_ready), it & 1, &abort_flag, p.status)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    // A = P^T [128 keys x 64 q] K-major; B = dO [64 q x 128 hd] N-major (two 64-wide halves)
                    tc_mma_f16(tDV, make_smem_desc(sPT + ks * 32, 16, 1024),
                               make_smem_desc(sdO + ks * 2048, 8192, 1024), idesc_acc, (it | ks) != 0);
                }
                tc_commit(smem_u32(&bar_dv_done));
                if (!mbar_wait(smem_u32(&bar_ds_ready), it & 1, &abort_flag, p.status)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    tc_mma_f16(tDK, make_smem_desc(sDS + ks * 32, 16, 1024),
                               make_smem_desc(sQ + ks * 2048, 8192, 1024), idesc_acc, (it | ks) != 0);
                }
                tc_commit(smem_u32(&bar_q_empty[st]));
                if (it == n_iter - 1) tc_commit(smem_u32(&bar_acc_done));
            }
        }
    } else {
        // thread = key row of the tile
        const int key = warp * 32 + lane;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const float c = p.scale * kLog2e;
        const long long key_abs = (long long)w.kv0 + key;
        bool ok = true;
        for (int it = 0; it < n_iter; ++it) {
            const int h = kv_head * group + it % group;
            const int qr = w.q_begin + (it / group) * 64;
            // stage the row statistics of this query sub-tile
            if (threadIdx.x < 64) {
                const long long qa = (long long)qr + threadIdx.x;
                const bool in = qa < w.q_end;
                s_lse[it & 1][threadIdx.x] = in ? p.lse[(long long)h * p.T + qa] * kLog2e : INFINITY;
                s_delta[it & 1][threadIdx.x] = in ? p.delta[(long long)h * p.T + qa] : 0.f;
                mbar_arrive(smem_u32(&bar_stats));
            }
            if (!mbar_wait(smem_u32(&bar_stats), it & 1, &abort_flag, p.status)) { ok = false; break; }
            if (!mbar_wait(smem_u32(&bar_s_full), it & 1, &abort_flag, p.status)) { ok = false; break; }
            tc_fence_after();
            const bool need_mask = (qr < w.kv0 + 128);
            float pv[64];
#pragma unroll
            for (int cc = 0; cc < 64; cc += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tS + lane_base + cc, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float pe = fast_exp2(__uint_as_float(r[i]) * c - s_lse[it & 1][cc + i]);
                    if (need_mask && (long long)qr + cc + i < key_abs) pe = 0.f;
                    pv[cc + i] = pe;
                }
            }
            // P^T was released by the wait on bar_dv_done that ended the previous iteration; dS^T by
            // bar_s_full, whose commit follows (and therefore covers) the previous dK product.
            // P^T -> shared (bf16, K-major A operand: [128 keys x 64 q], one 128-byte row per key)
#pragma unroll
            for (int q8 = 0; q8 < 8; ++q8) {
                const uint32_t a = sPT + swz_off(key, q8 * 8);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a),
                             "r"(pack_bf16(pv[q8 * 8], pv[q8 * 8 + 1])), "r"(pack_bf16(pv[q8 * 8 + 2], pv[q8 * 8 + 3])),
                             "r"(pack_bf16(pv[q8 * 8 + 4], pv[q8 * 8 + 5])), "r"(pack_bf16(pv[q8 * 8 + 6], pv[q8 * 8 + 7]))
                             : "memory");
            }
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(smem_u32(&bar_p_ready));
            // dS^T = P^T * (dP^T - delta) * scale
#pragma unroll
            for (int cc = 0; cc < 64; cc += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tDP + lane_base + cc, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    pv[cc + i] = pv[cc + i] * (__uint_as_float(r[i]) - s_delta[it & 1][cc + i]) * p.scale;
            }
#pragma unroll
            for (int q8 = 0; q8 < 8; ++q8) {
                const uint32_t a = sDS + swz_off(key, q8 * 8);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a),
                             "r"(pack_bf16(pv[q8 * 8], pv[q8 * 8 + 1])), "r"(pack_bf16(pv[q8 * 8 + 2], pv[q8 * 8 + 3])),
                             "r"(pack_bf16(pv[q8 * 8 + 4], pv[q8 * 8 + 5])), "r"(pack_bf16(pv[q8 * 8 + 6], pv[q8 * 8 + 7]))
                             : "memory");
            }
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(smem_u32(&bar_ds_ready));
            // P^T may be overwritten next iteration only after the dV product has read it
            if (!mbar_wait(smem_u32(&bar_dv_done), it & 1, &abort_flag, p.status)) { ok = false; break; }
        }
        if (ok && mbar_wait(smem_u32(&bar_acc_done), 0, &abort_flag, p.status)) {
            tc_fence_after();
            // tcgen05.ld is warp-collective: every lane issues the loads, only the stores are guarded
            const bool live = key_abs < w.q_end;
            __nv_bfloat16* dk = reinterpret_cast<__nv_bfloat16*>(p.dK) + key_abs * p.ld_dk + kv_head * kHd;
            __nv_bfloat16* dv = reinterpret_cast<__nv_bfloat16*>(p.dV) + key_abs * p.ld_dv + kv_head * kHd;
#pragma unroll 1
            for (int cc = 0; cc < 128; cc += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tDK + lane_base + cc, r);
                tmem_ld_wait();
                if (live) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8)
                        *reinterpret_cast<uint4*>(dk + cc + i) = make_uint4(
                            pack_bf16(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                            pack_bf16(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])),
                            pack_bf16(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5])),
                            pack_bf16(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7])));
                }
                tmem_ld_32x32(tDV + lane_base + cc, r);
                tmem_ld_wait();
                if (live) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8)
                        *reinterpret_cast<uint4*>(dv + cc + i) = make_uint4(
                            pack_bf16(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                            pack_bf16(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])),
                            pack_bf16(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5])),
                            pack_bf16(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7])));
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_slot, 512);
    }
}

struct BwdQWork {
    int q0;     // first query row of the 128-query tile
    int kv0;    // first key row of its document
    int n_kv;   // number of 64-key sub-tiles to visit
    int q_end;  // one past the document's last row
};

// Q, dO (32 KiB each), dS (128 x 64, 16 KiB), 2 stages of (K, V) 64 x 128
constexpr int kBwdQSmem = 2 * kTileBytes + kHalfTile + 2 * 2 * kHalfTile + 1024;

// One CTA per (128-query tile, head):  S = Q K^T, dP = dO V^T (64 key columns each),
//   dS = P * (dP - delta) * scale,  dQ += dS K  (TMEM accumulator)
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const BwdParams p) {
    if (status_poisoned(p.status)) return;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_q, bar_kv_full[2], bar_kv_empty[2], bar_s_full, bar_ds_ready, bar_dq_done,
        bar_acc_done;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = base, sdO = base + kTileBytes, sDS = base + 2 * kTileBytes, sKV = sDS + kHalfTile;
    const int head = blockIdx.x;
    const int kv_head = head / (p.Hq / p.Hkv);
    const BwdQWork w = reinterpret_cast<const BwdQWork*>(p.work)[blockIdx.y];

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar_q), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&bar_kv_full[s]), 1);
            mbar_init(smem_u32(&bar_kv_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_s_full), 1);
        mbar_init(smem_u32(&bar_ds_ready), 128);
        mbar_init(smem_u32(&bar_dq_done), 1);
        mbar_init(smem_u32(&bar_acc_done), 1);
        mbar_fence_init();
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(&tmem_slot), 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tS = tmem_slot, tDP = tmem_slot + 64, tDQ = tmem_slot + 128;

    if (warp == 4) {
        if (lane == 0) {
            mbar_expect_tx(smem_u32(&bar_q), 2 * kTileBytes);
            tma_load_2d(sQ, &tmQ, smem_u32(&bar_q), head * kHd, w.q0);
            tma_load_2d(sQ + 16384, &tmQ, smem_u32(&bar_q), head * kHd + 64, w.q0);
            tma_load_2d(sdO, &tmdO, smem_u32(&bar_q), head * kHd, w.q0);
            tma_load_2d(sdO + 16384, &tmdO, smem_u32(&bar_q), head * kHd + 64, w.q0);
            for (int j = 0; j < w.n_kv; ++j) {
                const int st = j & 1;
                if (!mbar_wait(smem_u32(&bar_kv_empty[st]), ((j >> 1) & 1) ^ 1u, &abort_flag, p.status)) break;
                const uint32_t full = smem_u32(&bar_kv_full[st]);
                const uint32_t sK = sKV + st * 2 * kHalfTile, sV = sK + kHalfTile;
                const int kr = w.kv0 + j * 64;
                mbar_expect_tx(full, 2 * kHalfTile);
                tma_load_2d(sK, &tmK, full, kv_head * kHd, kr);
                tma_load_2d(sK + 8192, &tmK, full, kv_head * kHd + 64, kr);
                tma_load_2d(sV, &tmV, full, kv_head * kHd, kr);
                tma_load_2d(sV + 8192, &tmV, full, kv_head * kHd + 64, kr);
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, 0, 0);     // [q x keys]
            constexpr uint32_t idesc_dq = make_idesc_bf16(128, 128, 0, 1);   // [q x hd] = dS K
            bool ok = mbar_wait(smem_u32(&bar_q), 0, &abort_flag, p.status);
            for (int j = 0; ok && j < w.n_kv; ++j) {
                const int st = j & 1;
                const uint32_t sK = sKV + st * 2 * kHalfTile, sV = sK + kHalfTile;
                if (!mbar_wait(smem_u32(&bar_kv_full[st]), (j >> 1) & 1, &abort_flag, p.status)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t offa = (ks >> 2) * 16384 + (ks & 3) * 32;
                    const uint32_t offb = (ks >> 2) * 8192 + (ks & 3) * 32;
                    tc_mma_f16(tS, make_smem_desc(sQ + offa, 16, 1024), make_smem_desc(sK + offb, 16, 1024),
                               idesc_s, ks != 0);
                }
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t offa = (ks >> 2) * 16384 + (ks & 3) * 32;
                    const uint32_t offb = (ks >> 2) * 8192 + (ks & 3) * 32;
                    tc_mma_f16(tDP, make_smem_desc(sdO + offa, 16, 1024), make_smem_desc(sV + offb, 16, 1024),
                               idesc_s, ks != 0);
                }
                tc_commit(smem_u32(&bar_s_full));
                if (!mbar_wait(smem_u32(&bar_ds_ready), j & 1, &abort_flag, p.status)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    // A = dS [128 q x 64 keys] K-major; B = K [64 keys x 128 hd] N-major
                    tc_mma_f16(tDQ, make_smem_desc(sDS + ks * 32, 16, 1024),
                               make_smem_desc(sK + ks * 2048, 8192, 1024), idesc_dq, (j | ks) != 0);
                }
                tc_commit(smem_u32(&bar_dq_done));
                tc_commit(smem_u32(&bar_kv_empty[st]));
                if (j == w.n_kv - 1) tc_commit(smem_u32(&bar_acc_done));
            }
        }
    } else {
        const int row = warp * 32 + lane;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const float c = p.scale * kLog2e;
        const long long q_abs = (long long)w.q0 + row;
        const bool in = q_abs < w.q_end;
        const float lse2 = in ? p.lse[(long long)head * p.T + q_abs] * kLog2e : INFINITY;
        const float dl = in ? p.delta[(long long)head * p.T + q_abs] : 0.f;
        bool ok = true;
        for (int j = 0; j < w.n_kv; ++j) {
            if (!mbar_wait(smem_u32(&bar_s_full), j & 1, &abort_flag, p.status)) { ok = false; break; }
            tc_fence_after();
            const int k0 = w.kv0 + j * 64;
            const bool need_mask = (k0 + 64 > w.q0);
            float pv[64];
#pragma unroll
            for (int cc = 0; cc < 64; cc += 32) {
                uint32_t r[32], d[32];
                tmem_ld_32x32(tS + lane_base + cc, r);
                tmem_ld_32x32(tDP + lane_base + cc, d);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float pe = fast_exp2(__uint_as_float(r[i]) * c - lse2);
                    if (need_mask && (long long)k0 + cc + i > q_abs) pe = 0.f;
                    pv[cc + i] = pe * (__uint_as_float(d[i]) - dl) * p.scale;
                }
            }
            // the previous dQ product must have finished reading dS before it is overwritten
            if (j > 0 && !mbar_wait(smem_u32(&bar_dq_done), (j - 1) & 1, &abort_flag, p.status)) { ok = false; break; }
#pragma unroll
            for (int q8 = 0; q8 < 8; ++q8) {
                const uint32_t a = sDS + swz_off(row, q8 * 8);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a),
                             "r"(pack_bf16(pv[q8 * 8], pv[q8 * 8 + 1])), "r"(pack_bf16(pv[q8 * 8 + 2], pv[q8 * 8 + 3])),
                             "r"(pack_bf16(pv[q8 * 8 + 4], pv[q8 * 8 + 5])), "r"(pack_bf16(pv[q8 * 8 + 6], pv[q8 * 8 + 7]))
                             : "memory");
            }
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(smem_u32(&bar_ds_ready));
        }
        if (ok && mbar_wait(smem_u32(&bar_acc_done), 0, &abort_flag, p.status)) {
            tc_fence_after();
            __nv_bfloat16* dq = reinterpret_cast<__nv_bfloat16*>(p.dQ) + q_abs * p.ld_dq + head * kHd;
#pragma unroll 1
            for (int cc = 0; cc < 128; cc += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tDQ + lane_base + cc, r);
                tmem_ld_wait();
                if (in) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8)
                        *reinterpret_cast<uint4*>(dq + cc + i) = make_uint4(
                            pack_bf16(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                            pack_bf16(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])),
                            pack_bf16(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5])),
                            pack_bf16(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7])));
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_slot, 256);
    }
}

// ---------------------------------------------------------------------------------------------
// Backward, second form. Same tiling and the same deterministic split into a dK/dV kernel and a dQ kernel as above,
// rebuilt around the fact that one step is a chain of latencies (products -> TMEM loads -> exp / mask / scale ->
// shared-memory stores -> products), not of throughput:
//   * the score / dP accumulators (tensor memory) and the P^T / dS^T operand tiles (shared memory) exist twice, and TWO
//     groups of eight element-wise warps alternate steps (group g takes the steps with it % 2 == g and always works on
//     copy g), so two steps' chains are in flight and the products of step i+1 are issued before the element-wise pass
//     of step i has finished;
//   * inside a group each thread owns one row and 32 of its 64 columns, so it holds 32 score values, not 64;
//   * the streamed operand tiles (Q, dO for dK/dV; K, V for dQ) have three / four stages, so that their loads are in
//     flight two steps ahead and the round trip to L2 never sits between two steps.
//   warp 0: TMA producer, warp 1: MMA issuer, warps 2..17: element-wise
//   (group = (warp - 2) / 8, TMEM lane quarter = warp & 3, column half = ((warp - 2) % 8) / 4)
// ---------------------------------------------------------------------------------------------
constexpr int kBwd2Threads = 576;
constexpr int kBwd2Ew = 256;                      // element-wise threads of one group
constexpr int kBwd2EwWarps = kBwd2Ew / 32;        // a warp arrives on a barrier once, through its first lane

// All lanes of the warp have finished what the barrier publishes (their loads from tensor memory, their stores and
// proxy fences); one lane arrives for the warp. 256 separate arrivals on one barrier word, three times a step, cost
// more than the step's arithmetic.
__device__ __forceinline__ void warp_arrive(uint32_t bar, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}

__device__ __forceinline__ void ew_bar_sync(int group) {   // named barrier of one group's eight warps
    asm volatile("bar.sync %0, %1;" ::"r"(2 + group), "n"(kBwd2Ew) : "memory");
}

// K, V (32 KiB each), 5 stages of (Q, dO) 64 x 128 (16 KiB each). P^T and dS^T never touch shared memory: every
// element-wise thread writes its row of them (bf16 pairs) with tcgen05.st over the tensor-memory columns its scores
// came from, and the dV / dK products take their A operand from there. (Measured per step of this kernel before:
// the MMA thread spent 2,100 of 3,700 cycles blocked in issue, because operand fetches, the element-wise stores and the
// TMA writes share one 128-byte-per-clock shared-memory port.)
constexpr int kBwdKv2Stages = 5;
constexpr int kBwdKv2Tiles = 2 * kTileBytes + kBwdKv2Stages * 2 * kHalfTile;     // 229,376
constexpr int kBwdKv2Smem = kBwdKv2Tiles + 2048;                                                 // barriers, scalars, statistics

template <bool kCP, bool kWin = false>
__global__ void __launch_bounds__(kBwd2Threads, 1)
attn_bwd_dkdv2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                      const BwdParams p, const __grid_constant__ CpArgs<kCP> ca) {
    if (status_poisoned(p.status)) return;
    extern __shared__ __align__(1024) uint8_t smem_b2[];
    const uint32_t base = smem_u32(smem_b2);
    if (base & 1023u) {
        if (threadIdx.x == 0 && p.status) atomicCAS(p.status, kStatusOk, kStatusBadArgument);
        return;
    }
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_b2 + kBwdKv2Tiles);
    enum { kKv = 0, kQFull = 1, kQEmpty = 6, kSFull = 11, kPReady = 13, kDsReady = 15, kAccDone = 17, kNumBars = 18 };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + kNumBars + 1);
    float* s_lse = reinterpret_cast<float*>(bars + kNumBars + 2);          // [2 groups][64]
    float* s_delta = s_lse + 128;                                          // [2 groups][64]
    auto bar = [&](int i) { return smem_u32(&bars[i]); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t sK = base, sV = base + kTileBytes, sQdO = base + 2 * kTileBytes;
    const int kv_head = blockIdx.x;
    const int group = p.Hq / p.Hkv;
    BwdKvWorkCp w;
    if constexpr (kCP) {
        w = reinterpret_cast<const BwdKvWorkCp*>(p.work)[blockIdx.y];
    } else {
        const BwdKvWork w4 = reinterpret_cast<const BwdKvWork*>(p.work)[blockIdx.y];
        w.kv0 = w4.kv0; w.q_begin = w4.q_begin; w.n_q = w4.n_q; w.q_end = w4.q_end;
        w.q_begin2 = 0; w.n_q2 = 0; w.pad0 = 0; w.pad1 = 0;
    }
    const int n_iter = (w.n_q + w.n_q2) * group;
    // global first query row of 64-query sub-tile `sub`, and what to subtract from a global query row for its local row
    int q_shift1 = 0, q_shift2 = 0;
    if constexpr (kCP) {
        const int p1 = cp_piece(ca.cp, w.q_begin);
        q_shift1 = ca.cp.bound[p1] - ca.cp.loc[p1];
        if (w.n_q2 > 0) {
            const int p2 = cp_piece(ca.cp, w.q_begin2);
            q_shift2 = ca.cp.bound[p2] - ca.cp.loc[p2];
        }
    }
    auto q_row = [&](int sub) -> int { return sub < w.n_q ? w.q_begin + sub * 64 : w.q_begin2 + (sub - w.n_q) * 64; };
    auto q_shift = [&](int sub) -> int { return sub < w.n_q ? q_shift1 : q_shift2; };

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < kNumBars; ++i) {
            const bool many = (i >= kPReady && i < kAccDone);      // arrived on by every warp of one element-wise group
            mbar_init(bar(i), many ? kBwd2EwWarps : 1);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm0 = *tmem_slot;
    // S^T[b] at 128 b, dP^T[b] at 128 b + 64, dV at 256, dK at 384. P^T[b] is written over S^T[b] and dS^T[b] over
    // dP^T[b]: the 32 queries of column half h as 16 packed columns at offset 32 h, i.e. inside the columns the writing
    // thread has itself just read, so the two halves' warps need no order between them.
    const uint32_t tDV = tm0 + 256, tDK = tm0 + 384;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(bar(kKv), 2 * kTileBytes);
            const CUtensorMap* mapK = &tmK;
            const CUtensorMap* mapV = &tmV;
            int k_loc = w.kv0;
            if constexpr (kCP) {
                const int pk = cp_piece(ca.cpk, w.kv0);
                mapK = &ca.peers.k[ca.cpk.owner[pk]];
                mapV = &ca.peers.v[ca.cpk.owner[pk]];
                k_loc = w.kv0 - ca.cpk.bound[pk] + ca.cpk.loc[pk];
            }
            tma_load_2d(sK, mapK, bar(kKv), kv_head * kHd, k_loc);
            tma_load_2d(sK + 16384, mapK, bar(kKv), kv_head * kHd + 64, k_loc);
            tma_load_2d(sV, mapV, bar(kKv), kv_head * kHd, k_loc);
            tma_load_2d(sV + 16384, mapV, bar(kKv), kv_head * kHd + 64, k_loc);
            for (int it = 0; it < n_iter; ++it) {
                const int st = it % kBwdKv2Stages;
                if (!mbar_wait(bar(kQEmpty + st), ((it / kBwdKv2Stages) & 1) ^ 1u, abort_flag, p.status)) break;
                const int h = kv_head * group + it % group;
                const int qr = q_row(it / group) - q_shift(it / group);     // local row of the sub-tile's first query
                const uint32_t full = bar(kQFull + st);
                const uint32_t sQ = sQdO + st * 2 * kHalfTile, sdO = sQ + kHalfTile;
                mbar_expect_tx(full, 2 * kHalfTile);
                tma_load_2d(sQ, &tmQ, full, h * kHd, qr);
                tma_load_2d(sQ + 8192, &tmQ, full, h * kHd + 64, qr);
                tma_load_2d(sdO, &tmdO, full, h * kHd, qr);
                tma_load_2d(sdO + 8192, &tmdO, full, h * kHd + 64, qr);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_st = make_idesc_bf16(128, 64, 0, 0);   // [keys x q] = K Q^T, V dO^T
            constexpr uint32_t idesc_acc = make_idesc_bf16(128, 128, 0, 1); // [keys x hd] = P^T dO, dS^T Q
            bool ok = mbar_wait(bar(kKv), 0, abort_flag, p.status);
            auto issue_s = [&](int j) -> bool {
                const int b = j & 1, st = j % kBwdKv2Stages;
                const uint32_t sQ = sQdO + st * 2 * kHalfTile, sdO = sQ + kHalfTile;
                if (!mbar_wait(bar(kQFull + st), (j / kBwdKv2Stages) & 1, abort_flag, p.status)) return false;   // Q, dO of step j
                // S^T / dP^T[b] are free: their last readers are the dV / dK products of step j - 2, which this thread
                // issued before this point, and the tensor pipe runs one thread's products in order
                tc_fence_after();
                const uint32_t tS = tm0 + 128 * b, tDP = tS + 64;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t offa = (ks >> 2) * 16384 + (ks & 3) * 32;  // K / V: 128-row halves
                    const uint32_t offb = (ks >> 2) * 8192 + (ks & 3) * 32;   // Q / dO: 64-row halves
                    tc_mma_f16(tS, make_smem_desc(sK + offa, 16, 1024), make_smem_desc(sQ + offb, 16, 1024), idesc_st, ks != 0);
                }
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t offa = (ks >> 2) * 16384 + (ks & 3) * 32;
                    const uint32_t offb = (ks >> 2) * 8192 + (ks & 3) * 32;
                    tc_mma_f16(tDP, make_smem_desc(sV + offa, 16, 1024), make_smem_desc(sdO + offb, 16, 1024), idesc_st, ks != 0);
                }
                tc_commit(bar(kSFull + b));
                return true;
            };
            if (ok && n_iter > 0) ok = issue_s(0);
            for (int it = 0; ok && it < n_iter; ++it) {
                const int b = it & 1, st = it % kBwdKv2Stages;
                const uint32_t sQ = sQdO + st * 2 * kHalfTile, sdO = sQ + kHalfTile;
                if (it + 1 < n_iter && !issue_s(it + 1)) break;
                if (!mbar_wait(bar(kPReady + b), (it >> 1) & 1, abort_flag, p.status)) break;      // P^T[b] written
                tc_fence_after();
                const uint32_t tPT = tm0 + 128 * b, tDST = tPT + 64;
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)   // 16 queries = 8 packed columns per step; queries 32.. sit at column 32
                    tc_mma_f16_tmem_a(tDV, tPT + (ks >> 1) * 32 + (ks & 1) * 8,
                                      make_smem_desc(sdO + ks * 2048, 8192, 1024), idesc_acc, (it | ks) != 0);
                if (!mbar_wait(bar(kDsReady + b), (it >> 1) & 1, abort_flag, p.status)) break;     // dS^T[b] written
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    tc_mma_f16_tmem_a(tDK, tDST + (ks >> 1) * 32 + (ks & 1) * 8,
                                      make_smem_desc(sQ + ks * 2048, 8192, 1024), idesc_acc, (it | ks) != 0);
                tc_commit(bar(kQEmpty + st));
                if (it == n_iter - 1) tc_commit(bar(kAccDone));
            }
        }
    } else {
        const int g = (warp - 2) >> 3;                            // element-wise group: steps with it % 2 == g, copy g of everything
        const int quad = warp & 3, half = ((warp - 2) & 7) >> 2;
        const int ew_tid = (threadIdx.x - 64) & (kBwd2Ew - 1);    // index inside the group
        const int key = quad * 32 + lane;                         // this thread's key row of the tile
        const int c0 = half * 32;                                 // its first query column
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const float c = p.scale * kLog2e;
        const long long key_abs = (long long)w.kv0 + key;
        const uint32_t tS = tm0 + 128 * g + lane_base + c0, tDP = tS + 64;
        const uint32_t tPT = tm0 + 128 * g + lane_base + c0, tDST = tPT + 64;   // this thread's 16 packed columns of P^T / dS^T
        float* lse_g = s_lse + g * 64;
        float* delta_g = s_delta + g * 64;
        bool ok = true;
        // statistics of a step, fetched by the group's first 128 threads (64 lse, 64 delta) one of its steps ahead
        auto fetch_stat = [&](int it) -> float {
            if (ew_tid >= 128 || it >= n_iter) return 0.f;
            const int h = kv_head * group + it % group;
            const long long qa = (long long)q_row(it / group) + (ew_tid & 63);
            const bool in = qa < w.q_end;
            const long long ql = qa - q_shift(it / group);
            if (ew_tid < 64) return in ? p.lse[(long long)h * p.T + ql] * kLog2e : INFINITY;
            return in ? p.delta[(long long)h * p.T + ql] : 0.f;
        };
        float stat = fetch_stat(g);
        for (int it = g; it < n_iter; it += 2) {
            const int k = it >> 1;                                // this group's step count: parity of its barriers
            const int qr = q_row(it / group);
            // Every thread of the group meets at the two barriers below in every one of its steps, also after a wait has
            // given up (it then skips the step's work): nobody may leave the loop early and strand the others.
            ew_bar_sync(g);                                       // the previous step's readers of the statistics are done
            if (ew_tid < 64) lse_g[ew_tid] = stat;
            else if (ew_tid < 128) delta_g[ew_tid - 64] = stat;
            stat = fetch_stat(it + 2);                            // in flight during this step
            ew_bar_sync(g);
            if (!ok) continue;
            if (!mbar_wait(bar(kSFull + g), k & 1, abort_flag, p.status)) { ok = false; continue; }
            tc_fence_after();
            uint32_t sr[32], dr[32];
            tmem_ld_32x32(tS, sr);
            tmem_ld_32x32(tDP, dr);
            tmem_ld_wait();
            // Only the tiles on the diagonal need the causal mask; everywhere else the loop carries no compare at all.
            // Column i of this thread is query qr + c0 + i; it sees key `key_abs` when i >= lim.
            // With a window it sees it only while i < lim + window (the query is at most window - 1 rows after the key).
            const bool need_mask = (qr < w.kv0 + 128) || (kWin && qr + 63 - w.kv0 >= p.window);
            const int lim = (int)(key_abs - qr) - c0;
            const int hi = kWin ? lim + p.window : 0;
            float pv[32];
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float pe = fast_exp2(__uint_as_float(sr[i]) * c - lse_g[c0 + i]);
                    pv[i] = (i < lim || (kWin && i >= hi)) ? 0.f : pe;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) pv[i] = fast_exp2(__uint_as_float(sr[i]) * c - lse_g[c0 + i]);
            }
            // P^T[g]: this thread's 32 probabilities as 16 packed columns, over the score columns it has just read
            {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) pk[i] = pack_bf16(pv[2 * i], pv[2 * i + 1]);
                tmem_st_32x16(tPT, pk);
                tmem_st_wait();
            }
            tc_fence_before();
            warp_arrive(bar(kPReady + g), lane);
            // dS^T = P^T * (dP^T - delta) * scale
#pragma unroll
            for (int i = 0; i < 32; ++i) pv[i] = pv[i] * (__uint_as_float(dr[i]) - delta_g[c0 + i]) * p.scale;
            {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) pk[i] = pack_bf16(pv[2 * i], pv[2 * i + 1]);
                tmem_st_32x16(tDST, pk);
                tmem_st_wait();
            }
            tc_fence_before();
            warp_arrive(bar(kDsReady + g), lane);
        }
        // the accumulators: group 0 stores dK, group 1 stores dV (each thread one row, 64 of its 128 columns)
        if (ok && mbar_wait(bar(kAccDone), 0, abort_flag, p.status)) {
            tc_fence_after();
            bool live = key_abs < w.q_end;
            long long ld = g == 0 ? p.ld_dk : p.ld_dv;
            void* out_base = g == 0 ? p.dK : p.dV;
            long long out_row = key_abs;
            if constexpr (kCP) {
                const int pk = cp_piece(ca.cpk, w.kv0);
                if (ca.cpk.owner[pk] == ca.cpk.my_rank) {
                    out_row = key_abs - ca.cpk.bound[pk] + ca.cpk.loc[pk];
                } else {
                    out_base = g == 0 ? p.dK_stage : p.dV_stage;
                    ld = p.ld_stage;
                    out_row = key_abs - ca.cpk.bound[pk] + ca.cpk.stage[pk];
                    if (ca.cpk.stage[pk] < 0) {            // no staging was planned for this piece: record it, write nothing
                        live = false;
                        if (key == 0 && half == 0 && p.status) atomicCAS(p.status, kStatusOk, kStatusBounds);
                    }
                }
            }
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out_base) + out_row * ld + kv_head * kHd + half * 64;
            const uint32_t tAcc = (g == 0 ? tDK : tDV) + lane_base + half * 64;
#pragma unroll 1
            for (int cc = 0; cc < 64; cc += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tAcc + cc, r);
                tmem_ld_wait();
                if (live) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8)
                        *reinterpret_cast<uint4*>(dst + cc + i) = make_uint4(
                            pack_bf16(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                            pack_bf16(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])),
                            pack_bf16(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5])),
                            pack_bf16(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7])));
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tm0, 512);
    }
}

// Q, dO (32 KiB each), 5 stages of (K, V) 64 x 128 (16 KiB each); dS lives in tensor memory (see the dK/dV kernel)
constexpr int kBwdQ2Stages = 5;
constexpr int kBwdQ2Tiles = 2 * kTileBytes + kBwdQ2Stages * 2 * kHalfTile;   // 229,376
constexpr int kBwdQ2Smem = kBwdQ2Tiles + 512;

template <bool kCP, bool kWin = false>
__global__ void __launch_bounds__(kBwd2Threads, 1)
attn_bwd_dq2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const BwdParams p, const __grid_constant__ CpArgs<kCP> ca) {
    if (status_poisoned(p.status)) return;
    extern __shared__ __align__(1024) uint8_t smem_q2[];
    const uint32_t base = smem_u32(smem_q2);
    if (base & 1023u) {
        if (threadIdx.x == 0 && p.status) atomicCAS(p.status, kStatusOk, kStatusBadArgument);
        return;
    }
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_q2 + kBwdQ2Tiles);
    enum { kQ = 0, kKvFull = 1, kKvEmpty = 6, kSFull = 11, kDsReady = 13, kAccDone = 15, kNumBars = 16 };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + kNumBars + 1);
    auto bar = [&](int i) { return smem_u32(&bars[i]); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t sQ = base, sdO = base + kTileBytes, sKV = base + 2 * kTileBytes;
    const int head = blockIdx.x;
    const int kv_head = head / (p.Hq / p.Hkv);
    const BwdQWork w = reinterpret_cast<const BwdQWork*>(p.work)[blockIdx.y];
    int q_shift = 0;                    // global query row - q_shift = local row (queries, dO, statistics, dQ are local)
    if constexpr (kCP) {
        const int pq = cp_piece(ca.cp, w.q0);
        q_shift = ca.cp.bound[pq] - ca.cp.loc[pq];
    }

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < kNumBars; ++i) mbar_init(bar(i), (i >= kDsReady && i < kAccDone) ? kBwd2EwWarps : 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm0 = *tmem_slot;
    const uint32_t tDQ = tm0 + 256;     // S[b] at 128 b, dP[b] at 128 b + 64

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(bar(kQ), 2 * kTileBytes);
            const int q_loc = w.q0 - q_shift;
            tma_load_2d(sQ, &tmQ, bar(kQ), head * kHd, q_loc);
            tma_load_2d(sQ + 16384, &tmQ, bar(kQ), head * kHd + 64, q_loc);
            tma_load_2d(sdO, &tmdO, bar(kQ), head * kHd, q_loc);
            tma_load_2d(sdO + 16384, &tmdO, bar(kQ), head * kHd + 64, q_loc);
            for (int j = 0; j < w.n_kv; ++j) {
                const int st = j % kBwdQ2Stages;
                if (!mbar_wait(bar(kKvEmpty + st), ((j / kBwdQ2Stages) & 1) ^ 1u, abort_flag, p.status)) break;
                const uint32_t full = bar(kKvFull + st);
                const uint32_t sK = sKV + st * 2 * kHalfTile, sV = sK + kHalfTile;
                int kr = w.kv0 + j * 64;
                const CUtensorMap* mapK = &tmK;
                const CUtensorMap* mapV = &tmV;
                if constexpr (kCP) {                       // the sub-tile's owner and its row in that rank's published buffer
                    const int pk = cp_piece(ca.cpk, kr);
                    mapK = &ca.peers.k[ca.cpk.owner[pk]];
                    mapV = &ca.peers.v[ca.cpk.owner[pk]];
                    kr = kr - ca.cpk.bound[pk] + ca.cpk.loc[pk];
                }
                mbar_expect_tx(full, 2 * kHalfTile);
                tma_load_2d(sK, mapK, full, kv_head * kHd, kr);
                tma_load_2d(sK + 8192, mapK, full, kv_head * kHd + 64, kr);
                tma_load_2d(sV, mapV, full, kv_head * kHd, kr);
                tma_load_2d(sV + 8192, mapV, full, kv_head * kHd + 64, kr);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, 0, 0);     // [q x keys]
            constexpr uint32_t idesc_dq = make_idesc_bf16(128, 128, 0, 1);   // [q x hd] = dS K
            bool ok = mbar_wait(bar(kQ), 0, abort_flag, p.status);
            auto issue_s = [&](int j) -> bool {
                const int b = j & 1, st = j % kBwdQ2Stages;
                const uint32_t sK = sKV + st * 2 * kHalfTile, sV = sK + kHalfTile;
                if (!mbar_wait(bar(kKvFull + st), (j / kBwdQ2Stages) & 1, abort_flag, p.status)) return false;
                tc_fence_after();       // S / dP[b]: last read by the dQ product of step j - 2, issued before this point
                const uint32_t tS = tm0 + 128 * b, tDP = tS + 64;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t offa = (ks >> 2) * 16384 + (ks & 3) * 32;
                    const uint32_t offb = (ks >> 2) * 8192 + (ks & 3) * 32;
                    tc_mma_f16(tS, make_smem_desc(sQ + offa, 16, 1024), make_smem_desc(sK + offb, 16, 1024), idesc_s, ks != 0);
                }
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t offa = (ks >> 2) * 16384 + (ks & 3) * 32;
                    const uint32_t offb = (ks >> 2) * 8192 + (ks & 3) * 32;
                    tc_mma_f16(tDP, make_smem_desc(sdO + offa, 16, 1024), make_smem_desc(sV + offb, 16, 1024), idesc_s, ks != 0);
                }
                tc_commit(bar(kSFull + b));
                return true;
            };
            if (ok && w.n_kv > 0) ok = issue_s(0);
            for (int j = 0; ok && j < w.n_kv; ++j) {
                const int b = j & 1, st = j % kBwdQ2Stages;
                const uint32_t sK = sKV + st * 2 * kHalfTile;
                if (j + 1 < w.n_kv && !issue_s(j + 1)) break;
                if (!mbar_wait(bar(kDsReady + b), (j >> 1) & 1, abort_flag, p.status)) break;
                tc_fence_after();
                const uint32_t tDS = tm0 + 128 * b + 64;      // dS[b], written over dP[b]
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    tc_mma_f16_tmem_a(tDQ, tDS + (ks >> 1) * 32 + (ks & 1) * 8,
                                      make_smem_desc(sK + ks * 2048, 8192, 1024), idesc_dq, (j | ks) != 0);
                tc_commit(bar(kKvEmpty + st));
                if (j == w.n_kv - 1) tc_commit(bar(kAccDone));
            }
        }
    } else {
        const int g = (warp - 2) >> 3;
        const int quad = warp & 3, half = ((warp - 2) & 7) >> 2;
        const int row = quad * 32 + lane;
        const int c0 = half * 32;
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const float c = p.scale * kLog2e;
        const long long q_abs = (long long)w.q0 + row;
        const bool in = q_abs < w.q_end;
        const long long q_local = q_abs - q_shift;
        const float lse2 = in ? p.lse[(long long)head * p.T + q_local] * kLog2e : INFINITY;
        const float dl = in ? p.delta[(long long)head * p.T + q_local] : 0.f;
        const uint32_t tS = tm0 + 128 * g + lane_base + c0, tDP = tS + 64;
        bool ok = true;
        for (int j = g; j < w.n_kv; j += 2) {
            const int k = j >> 1;
            if (!mbar_wait(bar(kSFull + g), k & 1, abort_flag, p.status)) { ok = false; break; }
            tc_fence_after();
            uint32_t sr[32], dr[32];
            tmem_ld_32x32(tS, sr);
            tmem_ld_32x32(tDP, dr);
            tmem_ld_wait();
            // column i of this thread is key k0 + i; the row sees it when i <= lim. Off the diagonal no compare is made.
            const int k0 = w.kv0 + j * 64 + c0;
            const bool need_mask = (k0 + 32 > w.q0) || (kWin && k0 + p.window <= w.q0 + 127);
            const int lim = (int)(q_abs - k0);
            const int lo = kWin ? lim - p.window + 1 : 0;                         // first visible column under a window
            float pv[32];
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float pe = fast_exp2(__uint_as_float(sr[i]) * c - lse2);
                    pv[i] = (i > lim || (kWin && i < lo)) ? 0.f : pe * (__uint_as_float(dr[i]) - dl) * p.scale;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    pv[i] = fast_exp2(__uint_as_float(sr[i]) * c - lse2) * (__uint_as_float(dr[i]) - dl) * p.scale;
            }
            {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) pk[i] = pack_bf16(pv[2 * i], pv[2 * i + 1]);
                tmem_st_32x16(tDP, pk);         // this thread's 16 packed columns of dS[g], over the dP columns it has just read
                tmem_st_wait();
            }
            tc_fence_before();
            warp_arrive(bar(kDsReady + g), lane);
        }
        // the accumulator: every thread of group g stores 32 columns of its row (group, half -> which 32 of the 128)
        if (ok && mbar_wait(bar(kAccDone), 0, abort_flag, p.status)) {
            tc_fence_after();
            const int col = g * 64 + half * 32;
            __nv_bfloat16* dq = reinterpret_cast<__nv_bfloat16*>(p.dQ) + q_local * p.ld_dq + head * kHd + col;
            uint32_t r[32];
            tmem_ld_32x32(tDQ + lane_base + col, r);
            tmem_ld_wait();
            if (in) {
#pragma unroll
                for (int i = 0; i < 32; i += 8)
                    *reinterpret_cast<uint4*>(dq + i) = make_uint4(
                        pack_bf16(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                        pack_bf16(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])),
                        pack_bf16(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5])),
                        pack_bf16(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7])));
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tm0, 512);
    }
}

// ---------------------------------------------------------------------------------------------
// Forward, second form: 64-key tiles, the running output accumulates in TMEM and is rescaled
// only when a row maximum grows by more than 2^8 (so the exponentials stay bounded without a
// rescale on every tile), and the CTA is small enough (112 KiB of shared memory, 256 TMEM
// columns, <= 168 registers) for two CTAs to share an SM: while one CTA's softmax warps work on
// a score tile, the other CTA's MMAs run, which is what keeps the tensor cores busy.
// Work items are the {q0, kv0, n_kv (64-key tiles), q_end} records also used by the dQ kernel.
// ---------------------------------------------------------------------------------------------
// Q + 2 x (K, V) = 96 KiB. P has no buffer of its own: once S = Q K^T has completed, the K tile
// of the stage is dead, so P (same 16 KiB) is written over it and the stage is released after P V.
constexpr int kFwd2Tiles = kTileBytes + 2 * 2 * kHalfTile;
constexpr int kFwd2Smem = kFwd2Tiles + 256;                              // + barriers and scalars

// 160 registers: six warps of 160 x 32 registers fit twice into the 64K-register file (the
// allocation granularity makes 168 miss it)
// 128 registers: warps are allotted to the four register-file partitions in whole groups of four,
// so a 6-warp CTA is charged for 8; two CTAs per SM then need <= 65536 / (2 * 8 * 32) registers.
__global__ void __maxnreg__(128)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
    if (status_poisoned(p.status)) return;
    extern __shared__ __align__(1024) uint8_t smem2[];
    const uint32_t base = smem_u32(smem2);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem2 + kFwd2Tiles);
    // bars[0]=q, [1..2]=kv_full, [3..4]=kv_empty, [5]=s_full[0], [6]=p_ready, [7]=o_full, [8]=s_full[1]
    uint32_t* tmem_slot_p = reinterpret_cast<uint32_t*>(smem2 + kFwd2Tiles + 80);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem2 + kFwd2Tiles + 88);
    if (base & 1023u) {
        if (threadIdx.x == 0 && p.status) atomicCAS(p.status, kStatusOk, kStatusBadArgument);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t sQ = base, sKV = base + kTileBytes;
    const uint32_t bar_q = smem_u32(&bars[0]), bar_p_ready = smem_u32(&bars[6]), bar_o_full = smem_u32(&bars[7]);
    const uint32_t bar_s_full[2] = {smem_u32(&bars[5]), smem_u32(&bars[8])};
    const int head = blockIdx.x;
    const int kv_head = head / (p.Hq / p.Hkv);
    const FwdWork w = p.work[blockIdx.y];

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar_q, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&bars[1 + s]), 1);
            mbar_init(smem_u32(&bars[3 + s]), 1);
        }
        mbar_init(bar_s_full[0], 1);
        mbar_init(bar_s_full[1], 1);
        mbar_init(bar_p_ready, 4);            // one arrival per softmax warp
        mbar_init(bar_o_full, 1);
        mbar_fence_init();
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(tmem_slot_p), 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem0 = *tmem_slot_p;
    // two 64-column score buffers so the next tile's Q K^T runs while this tile's softmax does
    const uint32_t tS = tmem0, tO = tmem0 + 128;

    if (warp == 4) {
        if (lane == 0) {
            mbar_expect_tx(bar_q, kTileBytes);
            tma_load_2d(sQ, &tmQ, bar_q, head * kHd, w.q0);
            tma_load_2d(sQ + 16384, &tmQ, bar_q, head * kHd + 64, w.q0);
            for (int j = 0; j < w.n_kv; ++j) {
                const int st = j & 1;
                if (!mbar_wait(smem_u32(&bars[3 + st]), ((j >> 1) & 1) ^ 1u, abort_flag, p.status)) break;
                const uint32_t full = smem_u32(&bars[1 + st]);
                const uint32_t sK = sKV + st * 2 * kHalfTile, sV = sK + kHalfTile;
                const int kr = w.kv0 + j * 64;
                mbar_expect_tx(full, 2 * kHalfTile);
                tma_load_2d(sK, &tmK, full, kv_head * kHd, kr);
                tma_load_2d(sK + 8192, &tmK, full, kv_head * kHd + 64, kr);
                tma_load_2d(sV, &tmV, full, kv_head * kHd, kr);
                tma_load_2d(sV + 8192, &tmV, full, kv_head * kHd + 64, kr);
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, 0, 0);
            constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, 0, 1);
            bool ok = mbar_wait(bar_q, 0, abort_flag, p.status);
            auto issue_s = [&](int j) -> bool {
                const int st = j & 1;
                const uint32_t sK = sKV + st * 2 * kHalfTile;
                if (!mbar_wait(smem_u32(&bars[1 + st]), (j >> 1) & 1, abort_flag, p.status)) return false;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t offa = (ks >> 2) * 16384 + (ks & 3) * 32;
                    const uint32_t offb = (ks >> 2) * 8192 + (ks & 3) * 32;
                    tc_mma_f16(tS + st * 64, make_smem_desc(sQ + offa, 16, 1024),
                               make_smem_desc(sK + offb, 16, 1024), idesc_s, ks != 0);
                }
                tc_commit(bar_s_full[st]);
                return true;
            };
            if (ok && w.n_kv > 0) ok = issue_s(0);
            for (int j = 0; ok && j < w.n_kv; ++j) {
                const int st = j & 1;
                const uint32_t sK = sKV + st * 2 * kHalfTile, sV = sK + kHalfTile;
                if (j + 1 < w.n_kv && !issue_s(j + 1)) break;
                if (!mbar_wait(bar_p_ready, j & 1, abort_flag, p.status)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    // P sits where this stage's K tile was
                    tc_mma_f16(tO, make_smem_desc(sK + ks * 32, 16, 1024),
                               make_smem_desc(sV + ks * 2048, 8192, 1024), idesc_o, (j | ks) != 0);
                }
                tc_commit(bar_o_full);
                tc_commit(smem_u32(&bars[3 + st]));
            }
        }
    } else {
        const int row = warp * 32 + lane;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const float c = p.scale * kLog2e;
        const long long q_abs = (long long)w.q0 + row;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < w.n_kv; ++j) {
            if (!mbar_wait(bar_s_full[j & 1], (j >> 1) & 1, abort_flag, p.status)) { ok = false; break; }
            tc_fence_after();
            const uint32_t tSj = tS + (j & 1) * 64;
            const int k0 = w.kv0 + j * 64;
            const bool need_mask = (k0 + 63 > w.q0);
            const uint32_t sP = sKV + (j & 1) * 2 * kHalfTile;
            // key column i of a half-tile is visible to this row when i <= lim - 32 * half; only diagonal tiles compare
            const int lim = (int)(q_abs - k0);
            float mx = m_ref;
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                uint32_t r[32];
                tmem_ld_32x32(tSj + lane_base + half * 32, r);
                tmem_ld_wait();
                if (need_mask) {
                    const int lh = lim - half * 32;
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, i <= lh ? __uint_as_float(r[i]) : -INFINITY);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
                }
            }
            // the previous P V product must be done before P is overwritten or O is rescaled
            if (j > 0 && !mbar_wait(bar_o_full, (j - 1) & 1, abort_flag, p.status)) { ok = false; break; }
            const bool grow = (mx - m_ref) * c > 8.f;   // also true on the first tile (m_ref = -inf)
            if (__any_sync(0xffffffffu, grow)) {
                const float alpha = fast_exp2((m_ref - mx) * c);
                if (j > 0) {
                    tc_fence_after();
#pragma unroll 1
                    for (int cc = 0; cc < 128; cc += 32) {
                        uint32_t r[32];
                        tmem_ld_32x32(tO + lane_base + cc, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tmem_st_32x32(tO + lane_base + cc, r);
                    }
                    tmem_st_wait();
                }
                l *= alpha;
                m_ref = mx;
            }
            const float mc = m_ref * c;
            float rs = 0.f;
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                uint32_t r[32];
                tmem_ld_32x32(tSj + lane_base + half * 32, r);   // second read of the tile: cheaper than 64 live registers
                tmem_ld_wait();
                uint32_t pk[16];
                // the row sum is taken from the fp32 probabilities (their bf16 roundings, which the P V product reads,
                // differ from them by unbiased noise of relative size 2^-9 that averages out over a row)
                if (need_mask) {
                    const int lh = lim - half * 32;
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float e0 = fast_exp2(__uint_as_float(r[i]) * c - mc);
                        const float e1 = fast_exp2(__uint_as_float(r[i + 1]) * c - mc);
                        const float p0 = i <= lh ? e0 : 0.f, p1 = i + 1 <= lh ? e1 : 0.f;
                        pk[i >> 1] = pack_bf16(p0, p1);
                        rs += p0 + p1;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = fast_exp2(__uint_as_float(r[i]) * c - mc);
                        const float p1 = fast_exp2(__uint_as_float(r[i + 1]) * c - mc);
                        pk[i >> 1] = pack_bf16(p0, p1);
                        rs += p0 + p1;
                    }
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint32_t a = sP + swz_off(row, half * 32 + q * 8);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(pk[4 * q]),
                                 "r"(pk[4 * q + 1]), "r"(pk[4 * q + 2]), "r"(pk[4 * q + 3])
                                 : "memory");
                }
            }
            l += rs;
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p_ready);
        }
        if (ok && mbar_wait(bar_o_full, (w.n_kv - 1) & 1, abort_flag, p.status)) {
            tc_fence_after();
            const bool live = q_abs < w.q_end;
            l = add_sink(l, m_ref * p.scale, p.sinks, head);
            const float inv = 1.f / l;
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.O) + q_abs * p.ldo + head * kHd;
#pragma unroll 1
            for (int cc = 0; cc < 128; cc += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tO + lane_base + cc, r);
                tmem_ld_wait();
                if (live) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8)
                        *reinterpret_cast<uint4*>(out + cc + i) = make_uint4(
                            pack_bf16(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv),
                            pack_bf16(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv),
                            pack_bf16(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv),
                            pack_bf16(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv));
                }
            }
            if (live) p.lse[(long long)head * p.T + q_abs] = m_ref * p.scale + logf(l);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem0, 256);
    }
}


// Forward, third form: as the second, but the probabilities never touch shared memory. Each softmax thread writes
// its row of P (bf16 pairs) with tcgen05.st into the tensor-memory columns its scores came from, and the P V product
// takes its A operand from tensor memory. Shared memory then carries only Q, K and V: a third less traffic per step on
// the resource that limits this kernel (operand fetches of the products and the K/V loads share one 128-byte-per-clock
// port), and the proxy fence between the softmax's stores and the product disappears.
template <bool kCP, bool kWin = false>
__global__ void __maxnreg__(128)
attn_fwd3_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnParams p, const __grid_constant__ CpArgs<kCP> ca) {
    if (status_poisoned(p.status)) return;
    extern __shared__ __align__(1024) uint8_t smem3[];
    const uint32_t base = smem_u32(smem3);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem3 + kFwd2Tiles);
    // bars[0]=q, [1..2]=kv_full, [3..4]=kv_empty, [5]=s_full[0], [6]=p_ready, [7]=o_full, [8]=s_full[1]
    uint32_t* tmem_slot_p = reinterpret_cast<uint32_t*>(smem3 + kFwd2Tiles + 80);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem3 + kFwd2Tiles + 88);
    if (base & 1023u) {
        if (threadIdx.x == 0 && p.status) atomicCAS(p.status, kStatusOk, kStatusBadArgument);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t sQ = base, sKV = base + kTileBytes;
    const uint32_t bar_q = smem_u32(&bars[0]), bar_p_ready = smem_u32(&bars[6]), bar_o_full = smem_u32(&bars[7]);
    const uint32_t bar_s_full[2] = {smem_u32(&bars[5]), smem_u32(&bars[8])};
    const int head = blockIdx.x;
    const int kv_head = head / (p.Hq / p.Hkv);
    const FwdWork w = p.work[blockIdx.y];
    int q_shift = 0;                    // global query row - q_shift = local row (queries, outputs, statistics are local)
    if constexpr (kCP) {
        const int pq = cp_piece(ca.cp, w.q0);
        q_shift = ca.cp.bound[pq] - ca.cp.loc[pq];
    }

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar_q, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&bars[1 + s]), 1);
            mbar_init(smem_u32(&bars[3 + s]), 1);
        }
        mbar_init(bar_s_full[0], 1);
        mbar_init(bar_s_full[1], 1);
        mbar_init(bar_p_ready, 4);            // one arrival per softmax warp
        mbar_init(bar_o_full, 1);
        mbar_fence_init();
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(tmem_slot_p), 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem0 = *tmem_slot_p;
    // two 64-column score buffers so the next tile's Q K^T runs while this tile's softmax does
    const uint32_t tS = tmem0, tO = tmem0 + 128;

    if (warp == 4) {
        if (lane == 0) {
            mbar_expect_tx(bar_q, kTileBytes);
            tma_load_2d(sQ, &tmQ, bar_q, head * kHd, w.q0 - q_shift);
            tma_load_2d(sQ + 16384, &tmQ, bar_q, head * kHd + 64, w.q0 - q_shift);
            for (int j = 0; j < w.n_kv; ++j) {
                const int st = j & 1;
                if (!mbar_wait(smem_u32(&bars[3 + st]), ((j >> 1) & 1) ^ 1u, abort_flag, p.status)) break;
                const uint32_t full = smem_u32(&bars[1 + st]);
                const uint32_t sK = sKV + st * 2 * kHalfTile, sV = sK + kHalfTile;
                int kr = w.kv0 + j * 64;
                const CUtensorMap* mapK = &tmK;
                const CUtensorMap* mapV = &tmV;
                if constexpr (kCP) {                       // the tile's owner and its row in that rank's published buffer
                    const int pk = cp_piece(ca.cpk, kr);
                    mapK = &ca.peers.k[ca.cpk.owner[pk]];
                    mapV = &ca.peers.v[ca.cpk.owner[pk]];
                    kr = kr - ca.cpk.bound[pk] + ca.cpk.loc[pk];
                }
                mbar_expect_tx(full, 2 * kHalfTile);
                tma_load_2d(sK, mapK, full, kv_head * kHd, kr);
                tma_load_2d(sK + 8192, mapK, full, kv_head * kHd + 64, kr);
                tma_load_2d(sV, mapV, full, kv_head * kHd, kr);
                tma_load_2d(sV + 8192, mapV, full, kv_head * kHd + 64, kr);
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, 0, 0);
            constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, 0, 1);
            bool ok = mbar_wait(bar_q, 0, abort_flag, p.status);
            auto issue_s = [&](int j) -> bool {
                const int st = j & 1;
                const uint32_t sK = sKV + st * 2 * kHalfTile;
                if (!mbar_wait(smem_u32(&bars[1 + st]), (j >> 1) & 1, abort_flag, p.status)) return false;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t offa = (ks >> 2) * 16384 + (ks & 3) * 32;
                    const uint32_t offb = (ks >> 2) * 8192 + (ks & 3) * 32;
                    tc_mma_f16(tS + st * 64, make_smem_desc(sQ + offa, 16, 1024),
                               make_smem_desc(sK + offb, 16, 1024), idesc_s, ks != 0);
                }
                tc_commit(bar_s_full[st]);
                return true;
            };
            if (ok && w.n_kv > 0) ok = issue_s(0);
            for (int j = 0; ok && j < w.n_kv; ++j) {
                const int st = j & 1;
                const uint32_t sK = sKV + st * 2 * kHalfTile, sV = sK + kHalfTile;
                if (j + 1 < w.n_kv && !issue_s(j + 1)) break;
                if (!mbar_wait(bar_p_ready, j & 1, abort_flag, p.status)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    // P: 16 keys = 8 packed columns per step, in the score buffer of this step
                    tc_mma_f16_tmem_a(tO, tS + st * 64 + ks * 8, make_smem_desc(sV + ks * 2048, 8192, 1024), idesc_o, (j | ks) != 0);
                }
                tc_commit(bar_o_full);
                tc_commit(smem_u32(&bars[3 + st]));
            }
        }
    } else {
        const int row = warp * 32 + lane;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const float c = p.scale * kLog2e;
        const long long q_abs = (long long)w.q0 + row;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < w.n_kv; ++j) {
            if (!mbar_wait(bar_s_full[j & 1], (j >> 1) & 1, abort_flag, p.status)) { ok = false; break; }
            tc_fence_after();
            const uint32_t tSj = tS + (j & 1) * 64;
            const int k0 = w.kv0 + j * 64;
            // key column i of a half-tile is visible to this row when lo - 32 * half <= i <= lim - 32 * half; only tiles on
            // the diagonal, or cut by the left edge of some row's window, compare at all
            const bool need_mask = (k0 + 63 > w.q0) || (kWin && k0 + p.window <= w.q0 + 127);
            const int lim = (int)(q_abs - k0);
            const int lo = kWin ? lim - p.window + 1 : 0;
            float mx = m_ref;
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                uint32_t r[32];
                tmem_ld_32x32(tSj + lane_base + half * 32, r);
                tmem_ld_wait();
                if (need_mask) {
                    const int lh = lim - half * 32, ll = lo - half * 32;
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, (i <= lh && (!kWin || i >= ll)) ? __uint_as_float(r[i]) : -INFINITY);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
                }
            }
            // the previous P V product must be done before P is overwritten or O is rescaled
            if (j > 0 && !mbar_wait(bar_o_full, (j - 1) & 1, abort_flag, p.status)) { ok = false; break; }
            const bool grow = (mx - m_ref) * c > 8.f;   // also true on the first tile (m_ref = -inf)
            if (__any_sync(0xffffffffu, grow)) {
                // a row whose keys so far all lie left of its window has seen nothing yet (both maxima are -inf):
                // it keeps its empty state instead of scaling by exp2(-inf + inf)
                const float alpha = (kWin && mx == -INFINITY) ? 1.f : fast_exp2((m_ref - mx) * c);
                if (j > 0) {
                    tc_fence_after();
#pragma unroll 1
                    for (int cc = 0; cc < 128; cc += 32) {
                        uint32_t r[32];
                        tmem_ld_32x32(tO + lane_base + cc, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tmem_st_32x32(tO + lane_base + cc, r);
                    }
                    tmem_st_wait();
                }
                l *= alpha;
                m_ref = mx;
            }
            const float mc = m_ref * c;
            float rs = 0.f;
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                uint32_t r[32];
                tmem_ld_32x32(tSj + lane_base + half * 32, r);   // second read of the tile: cheaper than 64 live registers
                tmem_ld_wait();
                uint32_t pk[16];
                // the row sum is taken from the fp32 probabilities (their bf16 roundings, which the P V product reads,
                // differ from them by unbiased noise of relative size 2^-9 that averages out over a row)
                if (need_mask) {
                    const int lh = lim - half * 32, ll = lo - half * 32;
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float e0 = fast_exp2(__uint_as_float(r[i]) * c - mc);
                        const float e1 = fast_exp2(__uint_as_float(r[i + 1]) * c - mc);
                        const float p0 = (i <= lh && (!kWin || i >= ll)) ? e0 : 0.f;
                        const float p1 = (i + 1 <= lh && (!kWin || i + 1 >= ll)) ? e1 : 0.f;
                        pk[i >> 1] = pack_bf16(p0, p1);
                        rs += p0 + p1;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = fast_exp2(__uint_as_float(r[i]) * c - mc);
                        const float p1 = fast_exp2(__uint_as_float(r[i + 1]) * c - mc);
                        pk[i >> 1] = pack_bf16(p0, p1);
                        rs += p0 + p1;
                    }
                }
                tmem_st_32x16(tSj + lane_base + half * 16, pk);      // P over the first 32 columns of this score buffer
            }
            tmem_st_wait();
            l += rs;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p_ready);
        }
        if (ok && mbar_wait(bar_o_full, (w.n_kv - 1) & 1, abort_flag, p.status)) {
            tc_fence_after();
            const bool live = q_abs < w.q_end;
            l = add_sink(l, m_ref * p.scale, p.sinks, head);
            const float inv = 1.f / l;
            const long long q_local = q_abs - q_shift;
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.O) + q_local * p.ldo + head * kHd;
#pragma unroll 1
            for (int cc = 0; cc < 128; cc += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tO + lane_base + cc, r);
                tmem_ld_wait();
                if (live) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8)
                        *reinterpret_cast<uint4*>(out + cc + i) = make_uint4(
                            pack_bf16(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv),
                            pack_bf16(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv),
                            pack_bf16(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv),
                            pack_bf16(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv));
                }
            }
            if (live) p.lse[(long long)head * p.T + q_local] = m_ref * p.scale + logf(l);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem0, 256);
    }
}



static int set_smem(const void* fn, int bytes) {
    return cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess ? 0 : -10;
}

// what the kernels get when context parallelism is off (never read)
static CpArgs<false> g_no_cp_args{};

// Tensor maps over every rank's published key / value buffer (box of `box_rows` rows) and the piece table.
static int fill_peer_maps(PeerMaps* peers, void* const* kv_ptrs, int n_bufs, long long kv_rows, long long kv_ld, int v_col,
                          int Hkv, int box_rows) {
    memset(peers, 0, sizeof(*peers));
    if (n_bufs < 1 || n_bufs > 8) return -1;
    for (int r = 0; r < 8; ++r) {
        const int src = r < n_bufs ? r : 0;               // unused slots repeat buffer 0's maps (valid, never selected)
        const char* base = reinterpret_cast<const char*>(kv_ptrs[src]);
        if (make_tmap_bf16(&peers->k[r], base, kv_rows, (long long)Hkv * kHd, kv_ld, box_rows)) return -1;
        if (make_tmap_bf16(&peers->v[r], base + (long long)v_col * 2, kv_rows, (long long)Hkv * kHd, kv_ld, box_rows)) return -1;
    }
    return 0;
}

// m: n_pieces, my rank (-1: owner of nothing), bound[17], owner[16], loc[16], stage[16]; owners index `n_bufs` buffers.
static int fill_cp_map(CpMap* cp, const int* m, int n_bufs) {
    cp->n_pieces = m[0];
    cp->my_rank = m[1];
    if (cp->n_pieces < 1 || cp->n_pieces > 16 || cp->my_rank < -1) return -2;
    for (int i = 0; i < 17; ++i) cp->bound[i] = m[2 + i];
    for (int i = 0; i < 16; ++i) {
        cp->owner[i] = m[19 + i];
        cp->loc[i] = m[35 + i];
        cp->stage[i] = m[51 + i];
        if (i < cp->n_pieces && (cp->owner[i] < 0 || cp->owner[i] >= n_bufs)) return -3;
    }
    return 0;
}

}  // namespace halo

using namespace halo;

template <bool kWin>
static int launch_fwd3_sinks(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p,
                             int n_tiles, cudaStream_t stream) {
    static bool cfg = false;
    if (!cfg) {
        if (set_smem((const void*)attn_fwd3_kernel<false, kWin>, kFwd2Smem)) return -10;
        cudaFuncSetAttribute((const void*)attn_fwd3_kernel<false, kWin>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        cfg = true;
    }
    attn_fwd3_kernel<false, kWin><<<dim3(p.Hq, n_tiles), kFwdThreads, kFwd2Smem, stream>>>(tq, tk, tv, p, g_no_cp_args);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" {

// q: [T, Hq*128] (row stride ldq), k / v: [T, Hkv*128] (ldk / ldv), o: [T, Hq*128] (ldo)
// work: device array of n_tiles {q0, kv0, n_kv, q_end}; lse: [Hq, T] fp32
int halo_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const void* work,
                  int n_tiles, long long T, int Hq, int Hkv, int head_dim, long long ldq,
                  long long ldk, long long ldv, long long ldo, float scale, int* status, void* stream) {
    if (head_dim != kHd || Hq % Hkv) return -1;
    if (n_tiles == 0) return 0;
    CUtensorMap tq, tk, tv;
    if (make_tmap_bf16(&tq, q, T, (long long)Hq * kHd, ldq, 128)) return -2;
    if (make_tmap_bf16(&tk, k, T, (long long)Hkv * kHd, ldk, 128)) return -3;
    if (make_tmap_bf16(&tv, v, T, (long long)Hkv * kHd, ldv, 128)) return -4;
    static bool cfg = false;
    if (!cfg) {
        if (set_smem((const void*)attn_fwd_kernel, kFwdSmem)) return -10;
        cfg = true;
    }
    AttnParams p{reinterpret_cast<const FwdWork*>(work), o, lse, ldo, T, Hq, Hkv, scale, status};
    attn_fwd_kernel<<<dim3(Hq, n_tiles), kFwdThreads, kFwdSmem, (cudaStream_t)stream>>>(tq, tk, tv, p);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Second form of the forward (64-key tiles, two CTAs per SM). work: n_tiles {q0, kv0, n_kv64, q_end}.
int halo_attn_fwd2(const void* q, const void* k, const void* v, void* o, float* lse, const void* work,
                   int n_tiles, long long T, int Hq, int Hkv, int head_dim, long long ldq,
                   long long ldk, long long ldv, long long ldo, float scale, int* status, void* stream) {
    if (head_dim != kHd || Hq % Hkv) return -1;
    if (n_tiles == 0) return 0;
    CUtensorMap tq, tk, tv;
    if (make_tmap_bf16(&tq, q, T, (long long)Hq * kHd, ldq, 128)) return -2;
    if (make_tmap_bf16(&tk, k, T, (long long)Hkv * kHd, ldk, 64)) return -3;
    if (make_tmap_bf16(&tv, v, T, (long long)Hkv * kHd, ldv, 64)) return -4;
    static bool cfg = false;
    if (!cfg) {
        if (set_smem((const void*)attn_fwd2_kernel, kFwd2Smem)) return -10;
        // two CTAs per SM need the largest shared-memory carve-out
        cudaFuncSetAttribute((const void*)attn_fwd2_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        cfg = true;
    }
    AttnParams p{reinterpret_cast<const FwdWork*>(work), o, lse, ldo, T, Hq, Hkv, scale, status};
    attn_fwd2_kernel<<<dim3(Hq, n_tiles), kFwdThreads, kFwd2Smem, (cudaStream_t)stream>>>(tq, tk, tv, p);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Third form of the forward (as the second, P kept in tensor memory). Same arguments and work list as halo_attn_fwd2.
int halo_attn_fwd3(const void* q, const void* k, const void* v, void* o, float* lse, const void* work,
                   int n_tiles, long long T, int Hq, int Hkv, int head_dim, long long ldq,
                   long long ldk, long long ldv, long long ldo, float scale, int* status, void* stream) {
    if (head_dim != kHd || Hq % Hkv) return -1;
    if (n_tiles == 0) return 0;
    CUtensorMap tq, tk, tv;
    if (make_tmap_bf16(&tq, q, T, (long long)Hq * kHd, ldq, 128)) return -2;
    if (make_tmap_bf16(&tk, k, T, (long long)Hkv * kHd, ldk, 64)) return -3;
    if (make_tmap_bf16(&tv, v, T, (long long)Hkv * kHd, ldv, 64)) return -4;
    static bool cfg = false;
    if (!cfg) {
        if (set_smem((const void*)attn_fwd3_kernel<false>, kFwd2Smem)) return -10;
        cudaFuncSetAttribute((const void*)attn_fwd3_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        cfg = true;
    }
    AttnParams p{reinterpret_cast<const FwdWork*>(work), o, lse, ldo, T, Hq, Hkv, scale, status};
    attn_fwd3_kernel<false><<<dim3(Hq, n_tiles), kFwdThreads, kFwd2Smem, (cudaStream_t)stream>>>(tq, tk, tv, p, g_no_cp_args);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Sliding-window forward (third form only): a query sees the last `window` keys up to itself. The work list's kv0 is the
// first key tile a query tile needs (aligned to 64 rows from its document's start), not the document's start.
int halo_attn_fwd3_window(const void* q, const void* k, const void* v, void* o, float* lse, const void* work,
                          int n_tiles, long long T, int Hq, int Hkv, int head_dim, long long ldq, long long ldk,
                          long long ldv, long long ldo, float scale, int window, int* status, void* stream) {
    if (head_dim != kHd || Hq % Hkv || window <= 0) return -1;
    if (n_tiles == 0) return 0;
    CUtensorMap tq, tk, tv;
    if (make_tmap_bf16(&tq, q, T, (long long)Hq * kHd, ldq, 128)) return -2;
    if (make_tmap_bf16(&tk, k, T, (long long)Hkv * kHd, ldk, 64)) return -3;
    if (make_tmap_bf16(&tv, v, T, (long long)Hkv * kHd, ldv, 64)) return -4;
    static bool cfg = false;
    if (!cfg) {
        if (set_smem((const void*)attn_fwd3_kernel<false, true>, kFwd2Smem)) return -10;
        cudaFuncSetAttribute((const void*)attn_fwd3_kernel<false, true>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        cfg = true;
    }
    AttnParams p{reinterpret_cast<const FwdWork*>(work), o, lse, ldo, T, Hq, Hkv, scale, status, window};
    attn_fwd3_kernel<false, true><<<dim3(Hq, n_tiles), kFwdThreads, kFwd2Smem, (cudaStream_t)stream>>>(tq, tk, tv, p, g_no_cp_args);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Forward with attention sinks (third form), with or without a sliding window: `sinks` holds one fp32 logit per query
// head. The logit enters the denominator in the kernel's last step, so the stored log-sum-exp and the normalised output are
// those of the softmax over keys plus sink; the backward kernels then need no change (the sink's value vector is zero).
int halo_attn_fwd3_sinks(const void* q, const void* k, const void* v, void* o, float* lse, const void* work,
                         int n_tiles, long long T, int Hq, int Hkv, int head_dim, long long ldq, long long ldk,
                         long long ldv, long long ldo, float scale, int window, const float* sinks, int* status,
                         void* stream) {
    if (head_dim != kHd || Hq % Hkv || window < 0 || !sinks) return -1;
    if (n_tiles == 0) return 0;
    CUtensorMap tq, tk, tv;
    if (make_tmap_bf16(&tq, q, T, (long long)Hq * kHd, ldq, 128)) return -2;
    if (make_tmap_bf16(&tk, k, T, (long long)Hkv * kHd, ldk, 64)) return -3;
    if (make_tmap_bf16(&tv, v, T, (long long)Hkv * kHd, ldv, 64)) return -4;
    AttnParams p{reinterpret_cast<const FwdWork*>(work), o, lse, ldo, T, Hq, Hkv, scale, status, window, sinks};
    return window > 0 ? launch_fwd3_sinks<true>(tq, tk, tv, p, n_tiles, (cudaStream_t)stream)
                      : launch_fwd3_sinks<false>(tq, tk, tv, p, n_tiles, (cudaStream_t)stream);
}

// Sliding-window backward (double-buffered kernels only). Work lists as halo_attn_bwd's, cut to the window: a key tile's
// query range ends window - 1 rows after its last key, a query tile's key range starts at its first row's window.
int halo_attn_bwd_window(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                         float* delta, void* dq, void* dk, void* dv, const void* kv_work, int n_kv_tiles,
                         const void* q_work, int n_q_tiles, long long T, int Hq, int Hkv, int head_dim, long long ldq,
                         long long ldk, long long ldv, long long ldo, long long ld_do, long long ld_dq, long long ld_dk,
                         long long ld_dv, float scale, int window, int* status, void* stream) {
    if (head_dim != kHd || Hq % Hkv || window <= 0) return -1;
    if (T == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    attn_delta_kernel<<<(unsigned)((T * Hq + 7) / 8), 256, 0, s>>>(
        (const __nv_bfloat16*)d_o, (const __nv_bfloat16*)o, delta, T, Hq, ld_do, ldo);
    CUtensorMap tq, tk, tv, tdo, tq64, tk64, tv64, tdo64;
    if (make_tmap_bf16(&tq, q, T, (long long)Hq * kHd, ldq, 128)) return -2;
    if (make_tmap_bf16(&tk, k, T, (long long)Hkv * kHd, ldk, 128)) return -3;
    if (make_tmap_bf16(&tv, v, T, (long long)Hkv * kHd, ldv, 128)) return -4;
    if (make_tmap_bf16(&tdo, d_o, T, (long long)Hq * kHd, ld_do, 128)) return -5;
    if (make_tmap_bf16(&tq64, q, T, (long long)Hq * kHd, ldq, 64)) return -6;
    if (make_tmap_bf16(&tk64, k, T, (long long)Hkv * kHd, ldk, 64)) return -7;
    if (make_tmap_bf16(&tv64, v, T, (long long)Hkv * kHd, ldv, 64)) return -8;
    if (make_tmap_bf16(&tdo64, d_o, T, (long long)Hq * kHd, ld_do, 64)) return -9;
    static bool cfg = false;
    if (!cfg) {
        if (set_smem((const void*)attn_bwd_dkdv2_kernel<false, true>, kBwdKv2Smem)) return -10;
        if (set_smem((const void*)attn_bwd_dq2_kernel<false, true>, kBwdQ2Smem)) return -10;
        cfg = true;
    }
    BwdParams p{kv_work, lse, delta, dq, dk, dv, ld_dq, ld_dk, ld_dv, T, Hq, Hkv, scale, status, nullptr, nullptr, 0, window};
    if (n_kv_tiles > 0)
        attn_bwd_dkdv2_kernel<false, true><<<dim3(Hkv, n_kv_tiles), kBwd2Threads, kBwdKv2Smem, s>>>(tq64, tk, tv, tdo64, p, g_no_cp_args);
    p.work = q_work;
    if (n_q_tiles > 0)
        attn_bwd_dq2_kernel<false, true><<<dim3(Hq, n_q_tiles), kBwd2Threads, kBwdQ2Smem, s>>>(tq, tk64, tv64, tdo, p, g_no_cp_args);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Context-parallel forward: q, o, lse are this rank's local rows; kv_ptrs[r] is rank r's published [kv_rows, kv_ld] buffer
// (keys in columns [0, v_col), values from column v_col), possibly a peer GPU's memory. work: {q0, document start,
// 64-key sub-tiles, document end} in the row's global numbering; cp_map: n_pieces, my rank, bound[17], owner[16], loc[16],
// stage[16] (host ints) for the query rows; kv_map: the same table for the key rows (owners index kv_ptrs).
int halo_attn_cp_fwd(const void* q, void* const* kv_ptrs, int n_ranks, long long kv_rows, long long kv_ld, int v_col,
                     void* o, float* lse, const void* work, int n_tiles, long long T_local, int Hq, int Hkv,
                     int head_dim, long long ldq, long long ldo, float scale, const int* cp_map, const int* kv_map,
                     int* status, void* stream) {
    if (head_dim != kHd || Hq % Hkv || n_ranks < 1 || n_ranks > 8) return -1;
    if (n_tiles == 0) return 0;
    CUtensorMap tq;
    if (make_tmap_bf16(&tq, q, T_local, (long long)Hq * kHd, ldq, 128)) return -2;
    static CpArgs<true> ca;                  // 3 KB: kept off the stack; entry points are called from one thread per process
    if (fill_peer_maps(&ca.peers, kv_ptrs, n_ranks, kv_rows, kv_ld, v_col, Hkv, 64)) return -3;
    if (fill_cp_map(&ca.cp, cp_map, 8) || fill_cp_map(&ca.cpk, kv_map, n_ranks)) return -4;
    static bool cfg = false;
    if (!cfg) {
        if (set_smem((const void*)attn_fwd3_kernel<true>, kFwd2Smem)) return -10;
        cudaFuncSetAttribute((const void*)attn_fwd3_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        cfg = true;
    }
    AttnParams p{reinterpret_cast<const FwdWork*>(work), o, lse, ldo, T_local, Hq, Hkv, scale, status};
    attn_fwd3_kernel<true><<<dim3(Hq, n_tiles), kFwdThreads, kFwd2Smem, (cudaStream_t)stream>>>(tq, ca.peers.k[0], ca.peers.v[0], p, ca);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Resident CTAs per SM the second forward form achieves on the current device (diagnostic).
int halo_attn_fwd2_occupancy() {
    set_smem((const void*)attn_fwd2_kernel, kFwd2Smem);
    cudaFuncSetAttribute((const void*)attn_fwd2_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    int n = -1;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attn_fwd2_kernel, kFwdThreads, kFwd2Smem);
    cudaFuncAttributes a;
    cudaFuncGetAttributes(&a, (const void*)attn_fwd2_kernel);
    int n0 = -1, n64 = -1;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n0, attn_fwd2_kernel, kFwdThreads, 0);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n64, attn_fwd2_kernel, kFwdThreads, 65536);
    for (int bs = 64; bs <= 512; bs *= 2) {
        int o = -1;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o, attn_fwd2_kernel, bs, 0);
        fprintf(stderr, "fwd2 occ(block=%d, dyn=0)=%d\n", bs, o);
    }
    {
        int o = -1;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o, attn_delta_kernel, 256, 0);
        fprintf(stderr, "delta kernel occ(256)=%d\n", o);
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMaxBlocksPerMultiprocessor, dev);
        fprintf(stderr, "max blocks/SM=%d\n", v);
        cudaDeviceGetAttribute(&v, cudaDevAttrMaxRegistersPerMultiprocessor, dev);
        fprintf(stderr, "regs/SM=%d\n", v);
        cudaDeviceGetAttribute(&v, cudaDevAttrMaxRegistersPerBlock, dev);
        fprintf(stderr, "regs/block=%d\n", v);
    }
    fprintf(stderr, "fwd2: regs=%d static_smem=%zu local=%zu maxthreads=%d maxdyn=%d carveout=%d occ(dyn=0)=%d occ(64K)=%d occ(%d)=%d\n",
            a.numRegs, a.sharedSizeBytes, a.localSizeBytes, a.maxThreadsPerBlock, a.maxDynamicSharedSizeBytes,
            a.preferredShmemCarveout, n0, n64, kFwd2Smem, n);
    return n;
}

// delta: [Hq, T] fp32 scratch. kv_work: n_kv_tiles {kv0, q_begin, n_q(64-row sub-tiles), q_end};
// q_work: n_q_tiles {q0, kv0, n_kv(64-key sub-tiles), q_end}.
int halo_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                  const float* lse, float* delta, void* dq, void* dk, void* dv, const void* kv_work,
                  int n_kv_tiles, const void* q_work, int n_q_tiles, long long T, int Hq, int Hkv,
                  int head_dim, long long ldq, long long ldk, long long ldv, long long ldo,
                  long long ld_do, long long ld_dq, long long ld_dk, long long ld_dv, float scale,
                  int* status, void* stream) {
    if (head_dim != kHd || Hq % Hkv) return -1;
    if (T == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    attn_delta_kernel<<<(unsigned)((T * Hq + 7) / 8), 256, 0, s>>>(
        (const __nv_bfloat16*)d_o, (const __nv_bfloat16*)o, delta, T, Hq, ld_do, ldo);
    CUtensorMap tq, tk, tv, tdo, tq64, tk64, tv64, tdo64;
    if (make_tmap_bf16(&tq, q, T, (long long)Hq * kHd, ldq, 128)) return -2;
    if (make_tmap_bf16(&tk, k, T, (long long)Hkv * kHd, ldk, 128)) return -3;
    if (make_tmap_bf16(&tv, v, T, (long long)Hkv * kHd, ldv, 128)) return -4;
    if (make_tmap_bf16(&tdo, d_o, T, (long long)Hq * kHd, ld_do, 128)) return -5;
    if (make_tmap_bf16(&tq64, q, T, (long long)Hq * kHd, ldq, 64)) return -6;
    if (make_tmap_bf16(&tk64, k, T, (long long)Hkv * kHd, ldk, 64)) return -7;
    if (make_tmap_bf16(&tv64, v, T, (long long)Hkv * kHd, ldv, 64)) return -8;
    if (make_tmap_bf16(&tdo64, d_o, T, (long long)Hq * kHd, ld_do, 64)) return -9;
    static bool cfg = false;
    static int variant = 2;
    if (!cfg) {
        if (set_smem((const void*)attn_bwd_dkdv_kernel, kBwdKvSmem)) return -10;
        if (set_smem((const void*)attn_bwd_dq_kernel, kBwdQSmem)) return -10;
        if (set_smem((const void*)attn_bwd_dkdv2_kernel<false>, kBwdKv2Smem)) return -10;
        if (set_smem((const void*)attn_bwd_dq2_kernel<false>, kBwdQ2Smem)) return -10;
        const char* e = getenv("HALO_ATTN_BWD_VARIANT");      // 2 (default): double-buffered form; 1: the first form
        if (e && atoi(e) == 1) variant = 1;
        cfg = true;
    }
    BwdParams p{kv_work, lse, delta, dq, dk, dv, ld_dq, ld_dk, ld_dv, T, Hq, Hkv, scale, status};
    if (n_kv_tiles > 0) {
        if (variant == 2)
            attn_bwd_dkdv2_kernel<false><<<dim3(Hkv, n_kv_tiles), kBwd2Threads, kBwdKv2Smem, s>>>(tq64, tk, tv, tdo64, p, g_no_cp_args);
        else attn_bwd_dkdv_kernel<<<dim3(Hkv, n_kv_tiles), kBwdThreads, kBwdKvSmem, s>>>(tq64, tk, tv, tdo64, p);
    }
    p.work = q_work;
    if (n_q_tiles > 0) {
        if (variant == 2)
            attn_bwd_dq2_kernel<false><<<dim3(Hq, n_q_tiles), kBwd2Threads, kBwdQ2Smem, s>>>(tq, tk64, tv64, tdo, p, g_no_cp_args);
        else attn_bwd_dq_kernel<<<dim3(Hq, n_q_tiles), kBwdThreads, kBwdQSmem, s>>>(tq, tk64, tv64, tdo, p);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Context-parallel backward. q, o, d_o, lse, delta, dq, dk, dv: this rank's local rows; kv_ptrs as in the forward.
// dk_stage / dv_stage ([rows, ld_stage]): where dK / dV of key tiles another rank owns are written (that rank adds them).
// kv_work: {k0, q_begin, n_q, doc end, q_begin2, n_q2, 0, 0} (8 ints); q_work: as the forward's work list.
int halo_attn_cp_bwd(const void* q, void* const* kv_ptrs, int n_ranks, long long kv_rows, long long kv_ld, int v_col,
                     const void* o, const void* d_o, const float* lse, float* delta, void* dq, void* dk, void* dv,
                     void* dk_stage, void* dv_stage, long long ld_stage, const void* kv_work, int n_kv_tiles,
                     const void* q_work, int n_q_tiles, long long T_local, int Hq, int Hkv, int head_dim, long long ldq,
                     long long ldo, long long ld_do, long long ld_dq, long long ld_dk, long long ld_dv, float scale,
                     const int* cp_map, const int* kv_map, int* status, void* stream) {
    if (head_dim != kHd || Hq % Hkv || n_ranks < 1 || n_ranks > 8) return -1;
    if (T_local == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    attn_delta_kernel<<<(unsigned)((T_local * Hq + 7) / 8), 256, 0, s>>>(
        (const __nv_bfloat16*)d_o, (const __nv_bfloat16*)o, delta, T_local, Hq, ld_do, ldo);
    CUtensorMap tq, tdo, tq64, tdo64;
    if (make_tmap_bf16(&tq, q, T_local, (long long)Hq * kHd, ldq, 128)) return -2;
    if (make_tmap_bf16(&tdo, d_o, T_local, (long long)Hq * kHd, ld_do, 128)) return -5;
    if (make_tmap_bf16(&tq64, q, T_local, (long long)Hq * kHd, ldq, 64)) return -6;
    if (make_tmap_bf16(&tdo64, d_o, T_local, (long long)Hq * kHd, ld_do, 64)) return -9;
    static CpArgs<true> ca128, ca64;         // key / value tensor maps with 128- and 64-row boxes
    if (fill_peer_maps(&ca128.peers, kv_ptrs, n_ranks, kv_rows, kv_ld, v_col, Hkv, 128)) return -3;
    if (fill_peer_maps(&ca64.peers, kv_ptrs, n_ranks, kv_rows, kv_ld, v_col, Hkv, 64)) return -4;
    if (fill_cp_map(&ca128.cp, cp_map, 8) || fill_cp_map(&ca128.cpk, kv_map, n_ranks)) return -12;
    ca64.cp = ca128.cp;
    ca64.cpk = ca128.cpk;
    static bool cfg = false;
    if (!cfg) {
        if (set_smem((const void*)attn_bwd_dkdv2_kernel<true>, kBwdKv2Smem)) return -10;
        if (set_smem((const void*)attn_bwd_dq2_kernel<true>, kBwdQ2Smem)) return -10;
        cfg = true;
    }
    BwdParams p{kv_work, lse, delta, dq, dk, dv, ld_dq, ld_dk, ld_dv, T_local, Hq, Hkv, scale, status, dk_stage, dv_stage, ld_stage};
    if (n_kv_tiles > 0)
        attn_bwd_dkdv2_kernel<true><<<dim3(Hkv, n_kv_tiles), kBwd2Threads, kBwdKv2Smem, s>>>(tq64, ca128.peers.k[0], ca128.peers.v[0],
                                                                                             tdo64, p, ca128);
    p.work = q_work;
    if (n_q_tiles > 0)
        attn_bwd_dq2_kernel<true><<<dim3(Hq, n_q_tiles), kBwd2Threads, kBwdQ2Smem, s>>>(tq, ca64.peers.k[0], ca64.peers.v[0], tdo, p,
                                                                                        ca64);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
