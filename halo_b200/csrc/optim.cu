// AdamW on bf16 parameters with bf16 moments (6 bytes of state per parameter), fp32 arithmetic,
// stochastic rounding of the weight and of the second moment, nearest rounding of the first
// moment; one launch steps every tensor of a parameter group. Also the multi-tensor squared-norm
// used for global-norm clipping: the clip coefficient is not applied in a pass of its own, it is
// read from device memory inside the step, as is the skip flag a non-finite step raises.
//
// Rounding noise is Philox-4x32-10 keyed by (optimizer key, step, hash of the parameter name) and
// counted by the element's offset inside its tensor, so it does not depend on how tensors are
// batched into launches and a resumed run rounds exactly like the uninterrupted one.
//
// This file is compiled with -fmad=false: the arithmetic below is the definition the CPU twin in
// halo_b200/optim/adamw_bf16.py reproduces bit for bit.
//
// Counterpart of the reference's fused Triton step (halo/optimizers/adamw_bf16.py:99-187) and its
// rounding helper (halo/optimizers/stochastic_rounding.py:30-63).
#include "sm100_common.cuh"

namespace halo {

struct Philox {
    uint32_t c[4];
};

__device__ __forceinline__ Philox philox4x32_10(uint32_t k0, uint32_t k1, uint32_t c0, uint32_t c1) {
    uint32_t c[4] = {c0, c1, 0u, 0u};
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
        const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    Philox o;
    o.c[0] = c[0]; o.c[1] = c[1]; o.c[2] = c[2]; o.c[3] = c[3];
    return o;
}

__host__ __device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__device__ __forceinline__ __nv_bfloat16 sr_to_bf16(float x, uint32_t noise16) {
    uint32_t bits = __float_as_uint(x) + noise16;
    return __ushort_as_bfloat16((unsigned short)(bits >> 16));
}

struct AdamTable {
    void* const* p;          // bf16 parameters
    const void* const* g;    // gradients (bf16 or fp32, one dtype per launch)
    void* const* m;          // bf16 first moments
    void* const* v;          // bf16 second moments
    const long long* numel;
    const unsigned long long* name_hash;
    const int* block_start;  // [n_tensors + 1] prefix of blocks per tensor
    int n_tensors;
};

// One tensor described by value in the kernel parameters (no device-side table to upload).
struct AdamSingle {
    void* p;
    const void* g;
    void* m;
    void* v;
    long long numel;
    unsigned long long name_hash;
};

constexpr int kAdamThreads = 256;
constexpr int kAdamElemsPerBlock = kAdamThreads * 4 * 16;

template <bool GRAD_F32>
__global__ void __launch_bounds__(kAdamThreads)
adamw_bf16_kernel(AdamTable tab, AdamSingle one, float beta1, float beta2, float one_minus_beta1,
                  float one_minus_beta2, float step_size, float bc2_sqrt, float eps, float wd_factor,
                  unsigned long long key_step, const float* __restrict__ grad_scale,
                  const int* __restrict__ skip) {
    if (skip && *skip) return;
    // which tensor does this block belong to
    const bool single = tab.n_tensors == 0;
    int lo = 0, hi = tab.n_tensors;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (tab.block_start[mid] <= (int)blockIdx.x) lo = mid; else hi = mid;
    }
    const int ti = lo;
    const long long n = single ? one.numel : tab.numel[ti];
    const long long chunk0 =
        (long long)(blockIdx.x - (single ? 0 : tab.block_start[ti])) * kAdamElemsPerBlock;
    __nv_bfloat16* p = (__nv_bfloat16*)(single ? one.p : tab.p[ti]);
    __nv_bfloat16* m = (__nv_bfloat16*)(single ? one.m : tab.m[ti]);
    __nv_bfloat16* v = (__nv_bfloat16*)(single ? one.v : tab.v[ti]);
    const void* gptr = single ? one.g : tab.g[ti];
    const uint64_t mixed = splitmix64(splitmix64(key_step) ^ (single ? one.name_hash : tab.name_hash[ti]));
    const uint32_t k0 = (uint32_t)mixed, k1 = (uint32_t)(mixed >> 32);
    float scale = 1.f;
    const bool has_scale = grad_scale != nullptr;
    if (has_scale) {
        scale = *grad_scale;
        if (!GRAD_F32) scale = __bfloat162float(__float2bfloat16_rn(scale));
    }
#pragma unroll 1
    for (int it = 0; it < 16; ++it) {
        const long long quad = (chunk0 >> 2) + (long long)it * kAdamThreads + threadIdx.x;
        const long long e0 = quad * 4;
        if (e0 >= n) break;
        const Philox rnd = philox4x32_10(k0, k1, (uint32_t)quad, (uint32_t)((unsigned long long)quad >> 32));
        const bool full = (e0 + 4 <= n) && ((((uintptr_t)(p + e0)) & 7u) == 0) &&
                          ((((uintptr_t)(m + e0)) & 7u) == 0) && ((((uintptr_t)(v + e0)) & 7u) == 0);
        float pf[4], mf[4], vf[4], gf[4];
        const int cnt = (int)min((long long)4, n - e0);
        if (full) {
            const uint2 pu = *reinterpret_cast<const uint2*>(p + e0);
            const uint2 mu = *reinterpret_cast<const uint2*>(m + e0);
            const uint2 vu = *reinterpret_cast<const uint2*>(v + e0);
            const __nv_bfloat162* ph = reinterpret_cast<const __nv_bfloat162*>(&pu);
            const __nv_bfloat162* mh = reinterpret_cast<const __nv_bfloat162*>(&mu);
            const __nv_bfloat162* vh = reinterpret_cast<const __nv_bfloat162*>(&vu);
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                float2 a = __bfloat1622float2(ph[q]); pf[2 * q] = a.x; pf[2 * q + 1] = a.y;
                a = __bfloat1622float2(mh[q]); mf[2 * q] = a.x; mf[2 * q + 1] = a.y;
                a = __bfloat1622float2(vh[q]); vf[2 * q] = a.x; vf[2 * q + 1] = a.y;
            }
        } else {
            for (int j = 0; j < 4; ++j) {
                const bool ok = j < cnt;
                pf[j] = ok ? __bfloat162float(p[e0 + j]) : 0.f;
                mf[j] = ok ? __bfloat162float(m[e0 + j]) : 0.f;
                vf[j] = ok ? __bfloat162float(v[e0 + j]) : 0.f;
            }
        }
        if (GRAD_F32) {
            const float* g = (const float*)gptr;
            for (int j = 0; j < 4; ++j) gf[j] = j < cnt ? g[e0 + j] : 0.f;
        } else {
            const __nv_bfloat16* g = (const __nv_bfloat16*)gptr;
            for (int j = 0; j < 4; ++j) gf[j] = j < cnt ? __bfloat162float(g[e0 + j]) : 0.f;
        }
        __nv_bfloat16 po[4], mo[4], vo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float g = gf[j];
            if (has_scale) {
                g = g * scale;
                if (!GRAD_F32) g = __bfloat162float(__float2bfloat16_rn(g));
            }
            const float mn = mf[j] * beta1 + g * one_minus_beta1;
            const float vn = vf[j] * beta2 + (g * g) * one_minus_beta2;
            const float denom = sqrtf(vn) / bc2_sqrt + eps;
            const float pn = pf[j] * wd_factor - (step_size * mn) / denom;
            mo[j] = __float2bfloat16_rn(mn);
            vo[j] = sr_to_bf16(vn, rnd.c[j] >> 16);
            po[j] = sr_to_bf16(pn, rnd.c[j] & 0xFFFFu);
        }
        if (full) {
            *reinterpret_cast<uint2*>(p + e0) = *reinterpret_cast<uint2*>(po);
            *reinterpret_cast<uint2*>(m + e0) = *reinterpret_cast<uint2*>(mo);
            *reinterpret_cast<uint2*>(v + e0) = *reinterpret_cast<uint2*>(vo);
        } else {
            for (int j = 0; j < cnt; ++j) {
                p[e0 + j] = po[j];
                m[e0 + j] = mo[j];
                v[e0 + j] = vo[j];
            }
        }
    }
}

// partial[b] = sum of squares of block b's elements; same block table as the step.
template <bool GRAD_F32>
__global__ void __launch_bounds__(kAdamThreads)
sq_norm_kernel(AdamTable tab, float* __restrict__ partial) {
    __shared__ float red[8];
    int lo = 0, hi = tab.n_tensors;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (tab.block_start[mid] <= (int)blockIdx.x) lo = mid; else hi = mid;
    }
    const int ti = lo;
    const long long n = tab.numel[ti];
    const long long chunk0 = (long long)(blockIdx.x - tab.block_start[ti]) * kAdamElemsPerBlock;
    float acc = 0.f;
    for (int it = 0; it < 16; ++it) {
        const long long e0 = chunk0 + ((long long)it * kAdamThreads + threadIdx.x) * 4;
        for (int j = 0; j < 4; ++j) {
            if (e0 + j < n) {
                const float g = GRAD_F32 ? ((const float*)tab.g[ti])[e0 + j]
                                         : __bfloat162float(((const __nv_bfloat16*)tab.g[ti])[e0 + j]);
                acc += g * g;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
        for (int i = 0; i < 8; ++i) s += red[i];
        partial[blockIdx.x] = s;
    }
}

// out[0] (+)= sum(partial[0..n))   (single block, fixed order)
__global__ void __launch_bounds__(1024)
sum_partials_kernel(const float* __restrict__ partial, int n, float* __restrict__ out, int accumulate) {
    __shared__ double red[32];
    double acc = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) acc += (double)partial[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double s = 0.0;
        for (int i = 0; i < 32; ++i) s += red[i];
        out[0] = accumulate ? out[0] + (float)s : (float)s;
    }
}

// coef = min(1, max_norm / (sqrt(total_sq) + 1e-6)); skip = !isfinite(total_sq); norm_out = sqrt
__global__ void clip_coef_kernel(const float* __restrict__ total_sq, float max_norm,
                                 float* __restrict__ coef, int* __restrict__ skip,
                                 float* __restrict__ norm_out) {
    const float sq = *total_sq;
    const float norm = sqrtf(sq);
    const bool finite = isfinite(norm);
    if (norm_out) *norm_out = norm;
    if (skip) *skip = finite ? 0 : 1;
    float c = 1.f;
    if (max_norm > 0.f && finite) c = fminf(1.f, max_norm / (norm + 1e-6f));
    *coef = c;
}


// ---- AdamW with 8-bit moments and 24-bit weights (5 bytes of state per parameter) ------------------------------------
// The weight is the bf16 parameter plus a signed 8-bit correction in units of 1/256 of the parameter's own bf16 spacing:
// w = p + c * ulp(p) / 256, so the update accumulates in 16 significant bits although the model computes on bf16 p.
// The moments are stored per group of 256 elements as one fp32 scale and 8-bit codes on a square-root-spaced grid
// (fine steps near zero): m = sign(q) (|q| / 127)^2 * m_scale, sqrt(v) = (q / 255)^2 * v_scale. Codes and the weight
// correction are rounded stochastically (Philox noise keyed like the bf16 optimizer's) so that a slowly decaying moment is unbiased instead of
// sticking to its grid point; a positive second moment never rounds to code 0, which keeps the denominator away from
// eps alone. One warp owns one group (8 elements per lane), so the group maxima are warp shuffles.
constexpr int kQ8Group = 256;
constexpr int kQ8Threads = 256;
constexpr int kQ8ElemsPerBlock = 2048;

struct Q8Table {
    void* const* p;                    // bf16 parameters
    const void* const* g;              // gradients (bf16 or fp32)
    void* const* corr;                 // int8 weight corrections
    void* const* mq;                   // int8 first-moment codes
    void* const* vq;                   // uint8 second-moment codes
    void* const* m_scale;              // fp32 [groups]
    void* const* v_scale;              // fp32 [groups]
    const long long* numel;
    const unsigned long long* name_hash;
    const int* block_start;
    int n_tensors;
};

__device__ __forceinline__ float bf16_spacing_256th(float pf) {
    const uint32_t e = (__float_as_uint(pf) >> 23) & 0xFFu;
    return e > 15u ? __uint_as_float((e - 15u) << 23) : 0.f;
}
// 1 / bf16_spacing_256th(pf): the spacing is a power of two, so its reciprocal is exact and multiplying by it gives the
// same bits as dividing by the spacing (0 where the spacing is 0)
__device__ __forceinline__ float bf16_inv_spacing_256th(float pf) {
    const uint32_t e = (__float_as_uint(pf) >> 23) & 0xFFu;
    return e > 15u ? __uint_as_float((269u - e) << 23) : 0.f;
}
// groups whose largest moment is below this keep their scale and store zero codes: the reciprocal of a smaller scale
// would overflow
constexpr float kQ8MinScale = 1e-30f;

template <bool GRAD_F32>
__global__ void __launch_bounds__(kQ8Threads)
adamw_q8_kernel(const Q8Table tab, float beta1, float beta2, float omb1, float omb2, float step_size, float bc2_sqrt,
                float eps, float wd_factor, unsigned long long key_step, const float* __restrict__ grad_scale,
                const int* __restrict__ skip) {
    if (skip != nullptr && *skip != 0) return;
    // decode tables: (q / 127)^2 and (q / 255)^2, the same fp32 operations the per-element form did, once per block
    __shared__ float dec_m[128], dec_v[256];
    {
        const float rv = (float)threadIdx.x / 255.f;
        dec_v[threadIdx.x] = rv * rv;
        if (threadIdx.x < 128) {
            const float rm = (float)threadIdx.x / 127.f;
            dec_m[threadIdx.x] = rm * rm;
        }
    }
    __syncthreads();
    int lo = 0, hi = tab.n_tensors;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (tab.block_start[mid] <= (int)blockIdx.x) lo = mid; else hi = mid;
    }
    const int ti = lo;
    const long long n = tab.numel[ti];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long group = (long long)(blockIdx.x - tab.block_start[ti]) * (kQ8ElemsPerBlock / kQ8Group) + warp;
    const long long g0 = group * kQ8Group;
    if (g0 >= n) return;                                        // whole warp leaves together
    const long long e0 = g0 + lane * 8;
    __nv_bfloat16* p = (__nv_bfloat16*)tab.p[ti];
    signed char* corr = (signed char*)tab.corr[ti];
    signed char* mq = (signed char*)tab.mq[ti];
    unsigned char* vq = (unsigned char*)tab.vq[ti];
    float* m_scale = (float*)tab.m_scale[ti];
    float* v_scale = (float*)tab.v_scale[ti];
    const uint64_t mixed = splitmix64(splitmix64(key_step) ^ tab.name_hash[ti]);
    const uint32_t k0 = (uint32_t)mixed, k1 = (uint32_t)(mixed >> 32);
    float scale = 1.f;
    const bool has_scale = grad_scale != nullptr;
    if (has_scale) {
        scale = *grad_scale;
        if (!GRAD_F32) scale = __bfloat162float(__float2bfloat16_rn(scale));
    }
    const float ms = m_scale[group], vs = v_scale[group];
    const float inv_bc2 = 1.f / bc2_sqrt;
    float w[8], m[8], s[8];
    float m_max = 0.f, s_max = 0.f;
    // eight consecutive elements per lane: one 16-byte load of the parameters (and of bf16 gradients), 8-byte loads of
    // the three code arrays when the tensor's base addresses allow it
    const bool full = (e0 + 8 <= n) && ((((uintptr_t)(p + e0)) & 15u) == 0) && ((((uintptr_t)(corr + e0)) & 7u) == 0) &&
                      ((((uintptr_t)(mq + e0)) & 7u) == 0) && ((((uintptr_t)(vq + e0)) & 7u) == 0) &&
                      (GRAD_F32 || ((((uintptr_t)((const __nv_bfloat16*)tab.g[ti] + e0)) & 15u) == 0));
    float pin[8], gin[8];
    int cin[8], qmin[8], qvin[8];
    if (full) {
        const uint4 pu = *reinterpret_cast<const uint4*>(p + e0);
        const uint2 cu = *reinterpret_cast<const uint2*>(corr + e0);
        const uint2 mu = *reinterpret_cast<const uint2*>(mq + e0);
        const uint2 vu = *reinterpret_cast<const uint2*>(vq + e0);
        const __nv_bfloat16* ph = reinterpret_cast<const __nv_bfloat16*>(&pu);
        const signed char* cb = reinterpret_cast<const signed char*>(&cu);
        const signed char* mb = reinterpret_cast<const signed char*>(&mu);
        const unsigned char* vb = reinterpret_cast<const unsigned char*>(&vu);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            pin[j] = __bfloat162float(ph[j]);
            cin[j] = cb[j]; qmin[j] = mb[j]; qvin[j] = vb[j];
        }
        if (GRAD_F32) {
            const float4 ga = *reinterpret_cast<const float4*>((const float*)tab.g[ti] + e0);
            const float4 gb = *reinterpret_cast<const float4*>((const float*)tab.g[ti] + e0 + 4);
            gin[0] = ga.x; gin[1] = ga.y; gin[2] = ga.z; gin[3] = ga.w; gin[4] = gb.x; gin[5] = gb.y; gin[6] = gb.z; gin[7] = gb.w;
        } else {
            const uint4 gu = *reinterpret_cast<const uint4*>((const __nv_bfloat16*)tab.g[ti] + e0);
            const __nv_bfloat16* gh = reinterpret_cast<const __nv_bfloat16*>(&gu);
#pragma unroll
            for (int j = 0; j < 8; ++j) gin[j] = __bfloat162float(gh[j]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const long long e = e0 + j;
            const bool ok = e < n;
            pin[j] = ok ? __bfloat162float(p[e]) : 0.f;
            cin[j] = ok ? (int)corr[e] : 0;
            qmin[j] = ok ? (int)mq[e] : 0;
            qvin[j] = ok ? (int)vq[e] : 0;
            if (GRAD_F32) gin[j] = ok ? ((const float*)tab.g[ti])[e] : 0.f;
            else gin[j] = ok ? __bfloat162float(((const __nv_bfloat16*)tab.g[ti])[e]) : 0.f;
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const bool ok = e0 + j < n;
        const float pf = pin[j];
        const int c = cin[j], qm = qmin[j], qv = qvin[j];
        float g = gin[j];
        if (has_scale) {
            g = g * scale;
            if (!GRAD_F32) g = __bfloat162float(__float2bfloat16_rn(g));
        }
        const float wf = pf + (float)c * bf16_spacing_256th(pf);
        float mf = dec_m[qm < 0 ? -qm : qm] * ms;
        if (qm < 0) mf = -mf;
        const float sf = dec_v[qv] * vs;
        const float mn = mf * beta1 + g * omb1;
        const float vn = (sf * sf) * beta2 + (g * g) * omb2;
        const float sn = sqrtf(vn);
        const float denom = sn * inv_bc2 + eps;
        w[j] = wf * wd_factor - (step_size * mn) / denom;
        m[j] = ok ? mn : 0.f;
        s[j] = ok ? sn : 0.f;
        m_max = fmaxf(m_max, fabsf(m[j]));
        s_max = fmaxf(s_max, s[j]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        m_max = fmaxf(m_max, __shfl_xor_sync(0xffffffffu, m_max, off));
        s_max = fmaxf(s_max, __shfl_xor_sync(0xffffffffu, s_max, off));
    }
    if (lane == 0) {
        m_scale[group] = m_max;
        v_scale[group] = s_max;
    }
    // one reciprocal per group instead of a division per element
    const float inv_m = m_max > kQ8MinScale ? 1.f / m_max : 0.f;
    const float inv_s = s_max > kQ8MinScale ? 1.f / s_max : 0.f;
    const long long quad = e0 >> 2;
    const Philox r0 = philox4x32_10(k0, k1, (uint32_t)quad, (uint32_t)((unsigned long long)quad >> 32));
    const Philox r1 = philox4x32_10(k0, k1, (uint32_t)(quad + 1), (uint32_t)((unsigned long long)(quad + 1) >> 32));
    __align__(16) __nv_bfloat16 pout[8];
    __align__(8) signed char cout[8];
    __align__(8) signed char mout[8];
    __align__(8) unsigned char vout[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t word = j < 4 ? r0.c[j] : r1.c[j - 4];
        // one 32-bit word per element: 11 bits of rounding noise for each moment code, 10 for the weight correction
        const float um = (float)(word & 0x7FFu) / 2048.f;
        const float uv = (float)((word >> 11) & 0x7FFu) / 2048.f;
        const float uc = (float)(word >> 22) / 1024.f;
        int qm = 0;
        if (inv_m > 0.f) {
            const float r = sqrtf(fabsf(m[j]) * inv_m) * 127.f;
            qm = (int)floorf(r + um);
            qm = qm > 127 ? 127 : qm;
            if (m[j] < 0.f) qm = -qm;
        }
        int qv = 0;
        if (inv_s > 0.f && s[j] > 0.f) {
            const float r = sqrtf(s[j] * inv_s) * 255.f;
            qv = (int)floorf(r + uv);
            qv = qv > 255 ? 255 : (qv < 1 ? 1 : qv);
        }
        const __nv_bfloat16 pn = __float2bfloat16_rn(w[j]);
        const float pnf = __bfloat162float(pn);
        const float inv_st = bf16_inv_spacing_256th(pnf);
        int c = 0;
        if (inv_st > 0.f) {
            // stochastic: an update below 1/256 of the spacing still moves the weight in expectation
            c = (int)floorf((w[j] - pnf) * inv_st + uc);
            c = c > 127 ? 127 : (c < -128 ? -128 : c);
        }
        pout[j] = pn;
        cout[j] = (signed char)c;
        mout[j] = (signed char)qm;
        vout[j] = (unsigned char)qv;
    }
    if (full) {
        *reinterpret_cast<uint4*>(p + e0) = *reinterpret_cast<const uint4*>(pout);
        *reinterpret_cast<uint2*>(corr + e0) = *reinterpret_cast<const uint2*>(cout);
        *reinterpret_cast<uint2*>(mq + e0) = *reinterpret_cast<const uint2*>(mout);
        *reinterpret_cast<uint2*>(vq + e0) = *reinterpret_cast<const uint2*>(vout);
    } else {
        for (int j = 0; j < 8 && e0 + j < n; ++j) {
            p[e0 + j] = pout[j];
            corr[e0 + j] = cout[j];
            mq[e0 + j] = mout[j];
            vq[e0 + j] = vout[j];
        }
    }
}

}  // namespace halo

using namespace halo;

extern "C" {

int halo_adam_elems_per_block() { return kAdamElemsPerBlock; }

// All table pointers are device arrays prepared once by the optimizer (they only change when the
// parameter set does). total_blocks = block_start[n_tensors].
int halo_adamw_bf16_step(void* const* p, const void* const* g, void* const* m, void* const* v,
                         const long long* numel, const unsigned long long* name_hash,
                         const int* block_start, int n_tensors, int total_blocks, int grad_is_f32,
                         float beta1, float beta2, float step_size, float bc2_sqrt, float eps,
                         float wd_factor, unsigned long long key, unsigned long long step,
                         const float* grad_scale, const int* skip, void* stream) {
    if (n_tensors <= 0 || total_blocks <= 0) return 0;
    AdamTable t{p, g, m, v, numel, name_hash, block_start, n_tensors};
    AdamSingle one{};
    const float omb1 = (float)(1.0 - (double)beta1), omb2 = (float)(1.0 - (double)beta2);
    cudaStream_t s = (cudaStream_t)stream;
    if (grad_is_f32)
        adamw_bf16_kernel<true><<<total_blocks, kAdamThreads, 0, s>>>(
            t, one, beta1, beta2, omb1, omb2, step_size, bc2_sqrt, eps, wd_factor, key ^ step, grad_scale, skip);
    else
        adamw_bf16_kernel<false><<<total_blocks, kAdamThreads, 0, s>>>(
            t, one, beta1, beta2, omb1, omb2, step_size, bc2_sqrt, eps, wd_factor, key ^ step, grad_scale, skip);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// One tensor, every pointer passed by value: the form the host-state optimizer streams buckets with.
int halo_adamw_bf16_step_single(void* p, const void* g, void* m, void* v, long long numel,
                                unsigned long long name_hash, int grad_is_f32, float beta1, float beta2,
                                float step_size, float bc2_sqrt, float eps, float wd_factor,
                                unsigned long long key, unsigned long long step, const float* grad_scale,
                                const int* skip, void* stream) {
    if (numel <= 0) return 0;
    AdamTable t{};
    AdamSingle one{p, g, m, v, numel, name_hash};
    const float omb1 = (float)(1.0 - (double)beta1), omb2 = (float)(1.0 - (double)beta2);
    const long long blocks = (numel + kAdamElemsPerBlock - 1) / kAdamElemsPerBlock;
    cudaStream_t s = (cudaStream_t)stream;
    if (grad_is_f32)
        adamw_bf16_kernel<true><<<(unsigned)blocks, kAdamThreads, 0, s>>>(
            t, one, beta1, beta2, omb1, omb2, step_size, bc2_sqrt, eps, wd_factor, key ^ step, grad_scale, skip);
    else
        adamw_bf16_kernel<false><<<(unsigned)blocks, kAdamThreads, 0, s>>>(
            t, one, beta1, beta2, omb1, omb2, step_size, bc2_sqrt, eps, wd_factor, key ^ step, grad_scale, skip);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}


int halo_adam_q8_elems_per_block() { return kQ8ElemsPerBlock; }
int halo_adam_q8_group() { return kQ8Group; }

// table: device array of int64 [9, n_tensors] rows p, g, corr, mq, vq, m_scale, v_scale, numel, name_hash.
int halo_adamw_q8_step(const long long* table, const int* block_start, int n_tensors, int total_blocks, int grad_is_f32,
                       float beta1, float beta2, float step_size, float bc2_sqrt, float eps, float wd_factor,
                       unsigned long long key, unsigned long long step, const float* grad_scale, const int* skip,
                       void* stream) {
    if (n_tensors <= 0 || total_blocks <= 0) return 0;
    const long long* row = table;
    Q8Table t{(void* const*)(row), (const void* const*)(row + n_tensors), (void* const*)(row + 2 * n_tensors),
              (void* const*)(row + 3 * n_tensors), (void* const*)(row + 4 * n_tensors), (void* const*)(row + 5 * n_tensors),
              (void* const*)(row + 6 * n_tensors), row + 7 * n_tensors, (const unsigned long long*)(row + 8 * n_tensors),
              block_start, n_tensors};
    const float omb1 = (float)(1.0 - (double)beta1), omb2 = (float)(1.0 - (double)beta2);
    cudaStream_t s = (cudaStream_t)stream;
    if (grad_is_f32)
        adamw_q8_kernel<true><<<total_blocks, kQ8Threads, 0, s>>>(t, beta1, beta2, omb1, omb2, step_size, bc2_sqrt, eps,
                                                                  wd_factor, key ^ step, grad_scale, skip);
    else
        adamw_q8_kernel<false><<<total_blocks, kQ8Threads, 0, s>>>(t, beta1, beta2, omb1, omb2, step_size, bc2_sqrt, eps,
                                                                   wd_factor, key ^ step, grad_scale, skip);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// partial: fp32 scratch [total_blocks]; out_sq: device scalar.
int halo_sq_norm(const void* const* g, const long long* numel, const int* block_start,
                 int n_tensors, int total_blocks, int grad_is_f32, float* partial, float* out_sq,
                 int accumulate, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (n_tensors > 0 && total_blocks > 0) {
        AdamTable t{nullptr, g, nullptr, nullptr, numel, nullptr, block_start, n_tensors};
        if (grad_is_f32) sq_norm_kernel<true><<<total_blocks, kAdamThreads, 0, s>>>(t, partial);
        else sq_norm_kernel<false><<<total_blocks, kAdamThreads, 0, s>>>(t, partial);
    }
    sum_partials_kernel<<<1, 1024, 0, s>>>(partial, total_blocks > 0 ? total_blocks : 0, out_sq, accumulate);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int halo_clip_coef(const float* total_sq, float max_norm, float* coef, int* skip, float* norm_out,
                   void* stream) {
    clip_coef_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(total_sq, max_norm, coef, skip, norm_out);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
