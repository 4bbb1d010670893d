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
