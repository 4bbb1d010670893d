// Pieces of the tcgen05 bf16 GEMM shared by the dense / grouped kernels and by the expert-parallel kernels that
// fuse token movement over peer memory into them: tile geometry, the work item, the kernel parameters, the dense
// tile walk and the epilogues (TMEM -> registers -> global memory).
#pragma once

#include "sm100_common.cuh"

namespace halo {

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockK = 64;
constexpr int kStages = 4;
constexpr int kATileBytes = kBlockM * kBlockK * 2;  // 16 KiB
constexpr int kBTileBytes = kBlockN * kBlockK * 2;  // 32 KiB
constexpr int kStageBytes = kATileBytes + kBTileBytes;
constexpr int kGemmThreads = 192;
constexpr int kTmemCols = 512;

enum : int {
    kEpiStoreBf16 = 0,
    kEpiStoreF32 = 1,
    kEpiAccumBf16 = 2,
    kEpiAccumF32 = 3,
    kEpiSwiglu = 4,  // columns [0,128) are gate, [128,256) are up: C = silu(gate) * up
    // as kEpiSwiglu, for experts with bias vectors around a clamped GLU: the tile's B coordinates index the bias bank
    // (one bias per row of B), pre = acc + bias, gate = min(pre_gate, limit), up = clamp(pre_up, -limit, limit),
    // C = (up + 1) * gate * sigmoid(glu_alpha * gate); aux receives the biased pre-activations
    kEpiClampedGlu = 5,
};

__host__ __device__ __forceinline__ bool epi_is_glu(int epi) { return epi == kEpiSwiglu || epi == kEpiClampedGlu; }

struct GemmWork {
    int a_mn;     // A coordinate along M of the tile's first row
    int a_k;      // A coordinate along the reduction index of the tile's first k-block
    int b_mn;     // B coordinate along N of columns [0,128) of the tile
    int b_mn2;    // B coordinate along N of columns [128,256) of the tile
    int b_k;      // B coordinate along the reduction index
    int k_iters;  // number of 64-wide k-blocks; 0 writes zeros
    int c_row;    // first row of C
    int c_col;    // first column of C (for the SwiGLU epilogue: of the activation output)
    int m_valid;  // rows of this tile that exist in C
    int n_valid;  // columns of this tile that exist in C
    int pad0, pad1;
};

struct GemmParams {
    void* C;
    void* aux;  // SwiGLU epilogue: optional [rows, 2F] copy of the pre-activation (gate | up)
    long long ldc;
    long long ld_aux;
    int epi;
    float alpha;
    int M, N, K;  // dense mode
    int tiles_m, tiles_n;
    int swiglu_f;            // SwiGLU: F (width of gate and of up); 0 otherwise
    const GemmWork* list;    // list mode when non-null
    const int* list_count;   // device count of list entries
    int* status;
    // Reduce-scatter epilogue (dense bf16 store only): rows [d * rs_rows, (d + 1) * rs_rows) of the product belong
    // to rank d, and a tile of those rows is stored straight into rank d's staging buffer c_peers[d] (that GPU's
    // memory mapped into this process) at row rs_rank * rs_rows + (row - d * rs_rows): slot rs_rank of the owner's
    // [rs_ranks][rs_rows][N] staging area. Tiles of other owners are visited first, the rank's own last, so the
    // NVLink stores of the early tiles drain while the later tiles are still being multiplied.
    void* c_peers[8];
    int rs_ranks, rs_rank, rs_rows;
    // kEpiClampedGlu: bias bank as one bf16 vector indexed like the rows of B, the clamp and the gate's slope
    const void* glu_bias;
    float glu_limit, glu_alpha;
};

__device__ __forceinline__ bool fetch_work(const GemmParams& p, int idx, int total, GemmWork& w) {
    if (idx >= total) return false;
    if (p.list) {
        w = p.list[idx];
        return true;
    }
    // dense: walk groups of 8 tile-rows, column-first inside a group, so CTAs running together
    // share A row-blocks and B column-blocks through L2
    const int group_m = 8;
    int tiles_m = p.tiles_m, tm_base = 0;
    w.pad0 = 0;
    if (p.rs_ranks > 1) {
        // owner-major order starting after this rank: every owner's row block is a dense sub-problem
        const int tm_per_owner = p.rs_rows / kBlockM;
        const int per_owner = tm_per_owner * p.tiles_n;
        const int o_seq = idx / per_owner;
        const int owner = (p.rs_rank + 1 + o_seq) % p.rs_ranks;
        idx -= o_seq * per_owner;
        tiles_m = tm_per_owner;
        tm_base = owner * tm_per_owner;
        w.pad0 = owner;
    }
    int per_group = group_m * p.tiles_n;
    int g = idx / per_group;
    int first_m = g * group_m;
    int gsz = min(tiles_m - first_m, group_m);
    int in_g = idx - g * per_group;
    int tm = tm_base + first_m + in_g % gsz;
    int tn = in_g / gsz;
    w.a_mn = tm * kBlockM;
    w.a_k = 0;
    w.b_k = 0;
    w.k_iters = (p.K + kBlockK - 1) / kBlockK;
    w.c_row = tm * kBlockM;
    if (p.rs_ranks > 1) w.c_row = p.rs_rank * p.rs_rows + (tm * kBlockM - w.pad0 * p.rs_rows);
    w.m_valid = min(kBlockM, p.M - tm * kBlockM);
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

// One epilogue warp's share of a finished tile: its 32 TMEM lanes (rows row_in_tile of the tile) x the tile's
// columns, read with tcgen05.ld and stored according to p.epi. Warp-collective: every lane must call it.
// `stage`: shared-memory address of this warp's 8 KB transposition buffer.
constexpr int kEpiStageBytesPerWarp = 32 * 256;   // 32 rows x 128 bf16 columns

__device__ __forceinline__ void epilogue_tile(const GemmParams& p, const GemmWork& w, uint32_t t_row, int row_in_tile,
                                              uint32_t stage) {
    const bool row_ok = row_in_tile < w.m_valid;
    const long long grow = (long long)w.c_row + row_in_tile;
    const bool zero = (w.k_iters == 0);
    if (p.epi == kEpiStoreBf16 && p.rs_ranks > 1) {
        // Reduce-scatter epilogue: the tile goes into the owner rank's staging area over NVLink. A thread owns one
        // accumulator row, so storing straight from registers would put 16-byte pieces 2*ldc bytes apart on the link;
        // instead the warp transposes 128 columns at a time through shared memory (16-byte units, XOR-swizzled by row)
        // and writes two 256-byte row segments per instruction. (For local stores L2 merges the pieces and the direct
        // path below measured faster.)
        const int lane = threadIdx.x & 31;
        const int warp_row0 = row_in_tile - lane;                 // first tile row of this warp
        __nv_bfloat16* cbase = reinterpret_cast<__nv_bfloat16*>(p.rs_ranks > 1 ? p.c_peers[w.pad0] : p.C);
#pragma unroll 1
        for (int c0 = 0; c0 < kBlockN; c0 += 128) {
            if (c0 >= w.n_valid) break;                           // uniform across the warp
#pragma unroll 1
            for (int cc = 0; cc < 128; cc += 32) {
                uint32_t r[32];
                tmem_ld_32x32(t_row + c0 + cc, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    uint32_t o[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float a = zero ? 0.f : __uint_as_float(r[j + 2 * q]) * p.alpha;
                        const float b = zero ? 0.f : __uint_as_float(r[j + 2 * q + 1]) * p.alpha;
                        o[q] = pack_bf16(a, b);
                    }
                    const int unit = (cc + j) >> 3;                // 16-byte unit within the 256-byte row
                    const uint32_t a = stage + lane * 256 + ((unit ^ (lane & 15)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                                 : "memory");
                }
            }
            __syncwarp();
            const int unit = lane & 15;
            const int col = c0 + unit * 8;
#pragma unroll 4
            for (int k = 0; k < 16; ++k) {
                const int rr = 2 * k + (lane >> 4);                // row within the warp's 32
                uint32_t v0, v1, v2, v3;
                const uint32_t a = stage + rr * 256 + ((unit ^ (rr & 15)) << 4);
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(a));
                if (warp_row0 + rr < w.m_valid && col + 8 <= w.n_valid)
                    *reinterpret_cast<uint4*>(cbase + ((long long)w.c_row + warp_row0 + rr) * p.ldc + w.c_col + col) =
                        make_uint4(v0, v1, v2, v3);
            }
            __syncwarp();
        }
        return;
    }
    if (epi_is_glu(p.epi)) {
        const bool clamped = (p.epi == kEpiClampedGlu);
#pragma unroll 1
        for (int c = 0; c < 128; c += 32) {
            uint32_t g[32], u[32];
            tmem_ld_32x32(t_row + c, g);
            tmem_ld_32x32(t_row + 128 + c, u);
            tmem_ld_wait();
            if (row_ok) {
                __nv_bfloat16* out =
                    reinterpret_cast<__nv_bfloat16*>(p.C) + grow * p.ldc + w.c_col + c;
                __nv_bfloat16* aux =
                    p.aux ? reinterpret_cast<__nv_bfloat16*>(p.aux) + grow * p.ld_aux +
                                w.c_col + c
                          : nullptr;
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    if (c + j + 8 <= w.n_valid) {
                        uint32_t o[4], pg[4], pu[4];
                        // the expert's bias for these eight gate and eight up columns: indexed like the rows of B
                        uint4 bias_g4 = make_uint4(0, 0, 0, 0), bias_u4 = make_uint4(0, 0, 0, 0);
                        if (clamped) {
                            const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(p.glu_bias);
                            bias_g4 = *reinterpret_cast<const uint4*>(bias + w.b_mn + c + j);
                            bias_u4 = *reinterpret_cast<const uint4*>(bias + w.b_mn2 + c + j);
                        }
                        const __nv_bfloat162* bias_g = reinterpret_cast<const __nv_bfloat162*>(&bias_g4);
                        const __nv_bfloat162* bias_u = reinterpret_cast<const __nv_bfloat162*>(&bias_u4);
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            // round the pre-activations to bf16 first so a later
                            // recomputation from the saved copy sees the same values
                            float g0 = zero ? 0.f : __uint_as_float(g[j + 2 * q]) * p.alpha;
                            float g1 = zero ? 0.f : __uint_as_float(g[j + 2 * q + 1]) * p.alpha;
                            float u0 = zero ? 0.f : __uint_as_float(u[j + 2 * q]) * p.alpha;
                            float u1 = zero ? 0.f : __uint_as_float(u[j + 2 * q + 1]) * p.alpha;
                            if (clamped) {
                                const float2 bgf = __bfloat1622float2(bias_g[q]), buf = __bfloat1622float2(bias_u[q]);
                                g0 += bgf.x; g1 += bgf.y; u0 += buf.x; u1 += buf.y;
                            }
                            pg[q] = pack_bf16(g0, g1);
                            pu[q] = pack_bf16(u0, u1);
                            __nv_bfloat162 gb = *reinterpret_cast<__nv_bfloat162*>(&pg[q]);
                            __nv_bfloat162 ub = *reinterpret_cast<__nv_bfloat162*>(&pu[q]);
                            float2 gf = __bfloat1622float2(gb), uf = __bfloat1622float2(ub);
                            float a0, a1;
                            if (clamped) {
                                const float gx = fminf(gf.x, p.glu_limit), gy = fminf(gf.y, p.glu_limit);
                                const float ux = fminf(fmaxf(uf.x, -p.glu_limit), p.glu_limit);
                                const float uy = fminf(fmaxf(uf.y, -p.glu_limit), p.glu_limit);
                                a0 = (ux + 1.f) * gx * sigmoid_fast(p.glu_alpha * gx);
                                a1 = (uy + 1.f) * gy * sigmoid_fast(p.glu_alpha * gy);
                            } else {
                                a0 = gf.x * sigmoid_fast(gf.x) * uf.x;
                                a1 = gf.y * sigmoid_fast(gf.y) * uf.y;
                            }
                            o[q] = pack_bf16(a0, a1);
                        }
                        *reinterpret_cast<uint4*>(out + j) = make_uint4(o[0], o[1], o[2], o[3]);
                        if (aux) {
                            *reinterpret_cast<uint4*>(aux + j) =
                                make_uint4(pg[0], pg[1], pg[2], pg[3]);
                            *reinterpret_cast<uint4*>(aux + p.swiglu_f + j) =
                                make_uint4(pu[0], pu[1], pu[2], pu[3]);
                        }
                    }
                }
            }
        }
    } else {
#pragma unroll 1
        for (int c = 0; c < kBlockN; c += 32) {
            if (c >= w.n_valid) break;  // uniform across the warp
            uint32_t r[32];
            tmem_ld_32x32(t_row + c, r);
            tmem_ld_wait();
            if (!row_ok) continue;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = zero ? 0.f : __uint_as_float(r[j]) * p.alpha;
            if (p.epi == kEpiStoreBf16 || p.epi == kEpiAccumBf16) {
                void* cbase = p.rs_ranks > 1 ? p.c_peers[w.pad0] : p.C;   // owner's staging area or C
                __nv_bfloat16* out =
                    reinterpret_cast<__nv_bfloat16*>(cbase) + grow * p.ldc + w.c_col + c;
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    if (c + j + 8 <= w.n_valid) {
                        if (p.epi == kEpiAccumBf16) {
                            uint4 old = *reinterpret_cast<const uint4*>(out + j);
                            const __nv_bfloat162* ob =
                                reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                float2 f = __bfloat1622float2(ob[q]);
                                v[j + 2 * q] += f.x;
                                v[j + 2 * q + 1] += f.y;
                            }
                        }
                        *reinterpret_cast<uint4*>(out + j) =
                            make_uint4(pack_bf16(v[j], v[j + 1]), pack_bf16(v[j + 2], v[j + 3]),
                                       pack_bf16(v[j + 4], v[j + 5]),
                                       pack_bf16(v[j + 6], v[j + 7]));
                    }
                }
            } else {
                float* out = reinterpret_cast<float*>(p.C) + grow * p.ldc + w.c_col + c;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    if (c + j + 4 <= w.n_valid) {
                        float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                        if (p.epi == kEpiAccumF32) {
                            float4 old = *reinterpret_cast<const float4*>(out + j);
                            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                        }
                        *reinterpret_cast<float4*>(out + j) = o;
                    }
                }
            }
        }
    }
}

}  // namespace halo
