// Decode-step attention against a padded key/value cache: one query token per sequence, all query heads of a
// key/value head handled by one CTA so every cached key and value is read from HBM exactly once.
//
//   cache layout  k, v: [batch, max_len, kv_heads, head_dim] bf16 (one layer's slice)
//   q:                  [batch, heads * head_dim] bf16        cols[b]: index of the newest key of sequence b
//   out[b, h, :] = softmax_j<=cols[b](scale * <q[b, h], k[b, j, h / G]>) @ v[b, j, h / G]
//
// grid (batch, kv_heads), 4 warps. A warp owns keys j = warp, warp + 4, ...; its lanes split head_dim, so a key row
// is one coalesced 128- or 256-byte read, the G dot products are lane-partial sums folded by shuffles, and every
// warp keeps an online-softmax state (max, sum, accumulator) per query head in registers. The four states are merged
// through shared memory at the end. The step is memory-bound: the cache is streamed once, nothing is written but
// the output row. Sequence lengths are read on the device - the host never synchronises on them.
//
// Stands where the reference's rollout engines run their paged decode kernels; here the cache is the sampler's own
// (halo_b200/inference/generate.py).
#include "sm100_common.cuh"

#include <math.h>

namespace halo {
namespace decode {

constexpr int kWarps = 4;
constexpr int kMaxGroup = 16;      // query heads per key/value head

template <int DPL>
__device__ __forceinline__ void load_row(const __nv_bfloat16* p, float (&f)[DPL]);
template <>
__device__ __forceinline__ void load_row<4>(const __nv_bfloat16* p, float (&f)[4]) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
template <>
__device__ __forceinline__ void load_row<2>(const __nv_bfloat16* p, float (&f)[2]) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    f[0] = a.x; f[1] = a.y;
}

// DPL = head_dim / 32 (dims per lane): 4 for head_dim 128, 2 for head_dim 64
template <int DPL>
__global__ void __launch_bounds__(kWarps * 32)
decode_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                        const __nv_bfloat16* __restrict__ vc, const long long* __restrict__ cols,
                        __nv_bfloat16* __restrict__ out, int n_heads, int n_kv_heads, long long max_len, float scale) {
    constexpr int D = 32 * DPL;
    __shared__ float s_m[kWarps][kMaxGroup];
    __shared__ float s_l[kWarps][kMaxGroup];
    __shared__ float s_acc[kWarps][kMaxGroup][D];
    const int b = blockIdx.x, hk = blockIdx.y;
    const int G = n_heads / n_kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    long long n_keys = cols[b] + 1;
    if (n_keys > max_len) n_keys = max_len;          // never read past the cache, whatever the host passed
    if (n_keys < 1) n_keys = 1;
    const long long key_stride = (long long)n_kv_heads * D;
    const __nv_bfloat16* kb = kc + ((long long)b * max_len) * key_stride + (long long)hk * D + lane * DPL;
    const __nv_bfloat16* vb = vc + ((long long)b * max_len) * key_stride + (long long)hk * D + lane * DPL;

    float qf[kMaxGroup][DPL], acc[kMaxGroup][DPL], m[kMaxGroup], l[kMaxGroup];
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) {
            acc[g][d] = 0.f;
            qf[g][d] = 0.f;
        }
        if (g < G) load_row<DPL>(q + ((long long)b * n_heads + (long long)hk * G + g) * D + lane * DPL, qf[g]);
    }
    for (long long j = warp; j < n_keys; j += kWarps) {
        float kf[DPL], vf[DPL];
        load_row<DPL>(kb + j * key_stride, kf);
        load_row<DPL>(vb + j * key_stride, vf);
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
            if (g < G) {
                float s = 0.f;
#pragma unroll
                for (int d = 0; d < DPL; ++d) s += qf[g][d] * kf[d];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                s *= scale;
                const float m_new = fmaxf(m[g], s);
                const float corr = __expf(m[g] - m_new);       // exp(-inf) = 0 on the first key
                const float p = __expf(s - m_new);
                l[g] = l[g] * corr + p;
#pragma unroll
                for (int d = 0; d < DPL; ++d) acc[g][d] = acc[g][d] * corr + p * vf[d];
                m[g] = m_new;
            }
        }
    }
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) {
        if (g < G) {
            if (lane == 0) {
                s_m[warp][g] = m[g];
                s_l[warp][g] = l[g];
            }
#pragma unroll
            for (int d = 0; d < DPL; ++d) s_acc[warp][g][lane * DPL + d] = acc[g][d];
        }
    }
    __syncthreads();
    // merge the four partial states: warp w finishes query heads g = w, w + 4, ...
    for (int g = warp; g < G; g += kWarps) {
        float big = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) big = fmaxf(big, s_m[w][g]);
        float denom = 0.f, num[DPL];
#pragma unroll
        for (int d = 0; d < DPL; ++d) num[d] = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float f = __expf(s_m[w][g] - big);            // a warp that saw no key holds (-inf, 0, 0): weight 0
            denom += s_l[w][g] * f;
#pragma unroll
            for (int d = 0; d < DPL; ++d) num[d] += s_acc[w][g][lane * DPL + d] * f;
        }
        const float inv = 1.f / denom;
        __nv_bfloat16* o = out + ((long long)b * n_heads + (long long)hk * G + g) * D + lane * DPL;
#pragma unroll
        for (int d = 0; d < DPL; d += 2)
            *reinterpret_cast<uint32_t*>(o + d) = pack_bf16(num[d] * inv, num[d + 1] * inv);
    }
}

}  // namespace decode
}  // namespace halo

extern "C" {

// q, out: [batch, n_heads * head_dim] bf16 contiguous. kc, vc: one layer of the cache, [batch, max_len, n_kv_heads,
// head_dim] bf16 contiguous. cols: [batch] int64 on the device.
int halo_decode_attention(const void* q, const void* kc, const void* vc, const long long* cols, void* out, int batch,
                          int n_heads, int n_kv_heads, int head_dim, long long max_len, float scale, void* stream) {
    using namespace halo::decode;
    if (batch < 0 || n_kv_heads < 1 || n_heads % n_kv_heads || n_heads / n_kv_heads > kMaxGroup || max_len < 1) return -1;
    if (head_dim != 128 && head_dim != 64) return -1;
    if (batch == 0) return 0;
    dim3 grid((unsigned)batch, (unsigned)n_kv_heads);
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 128)
        decode_attention_kernel<4><<<grid, kWarps * 32, 0, s>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)kc,
                                                                (const __nv_bfloat16*)vc, cols, (__nv_bfloat16*)out, n_heads,
                                                                n_kv_heads, max_len, scale);
    else
        decode_attention_kernel<2><<<grid, kWarps * 32, 0, s>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)kc,
                                                                (const __nv_bfloat16*)vc, cols, (__nv_bfloat16*)out, n_heads,
                                                                n_kv_heads, max_len, scale);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
