// AdamWBF16 on the host CPU, bit-identical to the device kernel (adamw_bf16_kernel): same operation order with
// no fused multiply-add, the same Philox-4x32-10 stream per group of four elements (keyed by step and parameter
// name), round-to-nearest for the first moment and stochastic rounding for the second moment and the weight.
//
// Used when a tensor's moments live in host memory: instead of streaming both moments to the device and back
// (8 bytes per parameter over PCIe), the gradient goes to the host and the new weight comes back (4 bytes per
// parameter) and the update itself runs here, on all cores.
//
// Built with -ffp-contract=off so that the compiler never contracts a*b+c into an fma.
#include <cmath>
#include <cstdint>
#include <cstring>

#ifdef _OPENMP
#include <omp.h>
#endif
#ifdef __AVX2__
#include <immintrin.h>
#endif

namespace {

inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

inline uint32_t f32_bits(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return u;
}

// round to nearest even, NaN kept quiet (what __float2bfloat16_rn does)
inline uint16_t f32_to_bf16_rn(float f) {
    const uint32_t u = f32_bits(f);
    const uint32_t rounded = (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
    const bool is_nan = (u & 0x7FFFFFFFu) > 0x7F800000u;
    return (uint16_t)(is_nan ? 0x7FFFu : rounded);
}

inline uint16_t sr_to_bf16(float x, uint32_t noise16) { return (uint16_t)((f32_bits(x) + noise16) >> 16); }

constexpr int kBlockQuads = 256;   // quads handled together so that the random stream and the update vectorise

}  // namespace

extern "C" {

// p, g, m, v: n bf16 elements each in host memory. grad_scale is applied (and the product rounded to bf16, as the
// device does for bf16 gradients) when has_scale != 0. Returns 0.
int halo_host_adamw_bf16(uint16_t* p, const uint16_t* g, uint16_t* m, uint16_t* v, long long n,
                         unsigned long long name_hash, unsigned long long key, unsigned long long step, float beta1,
                         float beta2, float step_size, float bc2_sqrt, float eps, float wd_factor, float grad_scale,
                         int has_scale, int n_threads) {
    const uint64_t mixed = splitmix64(splitmix64(key ^ step) ^ name_hash);
    const uint32_t k0_base = (uint32_t)mixed, k1_base = (uint32_t)(mixed >> 32);
    const float one_minus_beta1 = 1.0f - beta1, one_minus_beta2 = 1.0f - beta2;
    float scale = grad_scale;
    if (has_scale) scale = bf16_to_f32(f32_to_bf16_rn(scale));
    const long long n_quads = (n + 3) / 4;
    const long long n_blocks = (n_quads + kBlockQuads - 1) / kBlockQuads;
#ifdef _OPENMP
    if (n_threads > 0) omp_set_num_threads(n_threads);
#endif
#pragma omp parallel for schedule(static)
    for (long long b = 0; b < n_blocks; ++b) {
        const long long q0 = b * kBlockQuads;
        const int nq = (int)((n_quads - q0) < kBlockQuads ? (n_quads - q0) : kBlockQuads);
        uint32_t c0[kBlockQuads], c1[kBlockQuads], c2[kBlockQuads], c3[kBlockQuads];
        for (int i = 0; i < ((nq + 7) & ~7); ++i) {
            const uint64_t quad = (uint64_t)(q0 + i);
            c0[i] = (uint32_t)quad;
            c1[i] = (uint32_t)(quad >> 32);
            c2[i] = 0u;
            c3[i] = 0u;
        }
        uint32_t k0 = k0_base, k1 = k1_base;
#ifdef __AVX2__
        // eight quads per step: 32x32 -> 64 bit products of the even and of the odd lanes, re-interleaved
        const __m256i M0 = _mm256_set1_epi32((int)0xD2511F53u), M1 = _mm256_set1_epi32((int)0xCD9E8D57u);
        const int nq8 = (nq + 7) & ~7;          // the arrays are kBlockQuads long: running past nq is harmless
        for (int r = 0; r < 10; ++r) {
            const __m256i K0 = _mm256_set1_epi32((int)k0), K1 = _mm256_set1_epi32((int)k1);
            for (int i = 0; i < nq8; i += 8) {
                const __m256i a0 = _mm256_loadu_si256((const __m256i*)(c0 + i)), a1 = _mm256_loadu_si256((const __m256i*)(c1 + i));
                const __m256i a2 = _mm256_loadu_si256((const __m256i*)(c2 + i)), a3 = _mm256_loadu_si256((const __m256i*)(c3 + i));
                const __m256i e0 = _mm256_mul_epu32(a0, M0), o0 = _mm256_mul_epu32(_mm256_srli_epi64(a0, 32), M0);
                const __m256i e1 = _mm256_mul_epu32(a2, M1), o1 = _mm256_mul_epu32(_mm256_srli_epi64(a2, 32), M1);
                const __m256i lo0 = _mm256_blend_epi32(e0, _mm256_slli_epi64(o0, 32), 0xAA);
                const __m256i hi0 = _mm256_blend_epi32(_mm256_srli_epi64(e0, 32), o0, 0xAA);
                const __m256i lo1 = _mm256_blend_epi32(e1, _mm256_slli_epi64(o1, 32), 0xAA);
                const __m256i hi1 = _mm256_blend_epi32(_mm256_srli_epi64(e1, 32), o1, 0xAA);
                _mm256_storeu_si256((__m256i*)(c0 + i), _mm256_xor_si256(_mm256_xor_si256(hi1, a1), K0));
                _mm256_storeu_si256((__m256i*)(c1 + i), lo1);
                _mm256_storeu_si256((__m256i*)(c2 + i), _mm256_xor_si256(_mm256_xor_si256(hi0, a3), K1));
                _mm256_storeu_si256((__m256i*)(c3 + i), lo0);
            }
            k0 += 0x9E3779B9u;
            k1 += 0xBB67AE85u;
        }
#else
        for (int r = 0; r < 10; ++r) {
            for (int i = 0; i < nq; ++i) {
                const uint64_t p0 = (uint64_t)0xD2511F53u * c0[i];
                const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2[i];
                const uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0;
                const uint32_t hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
                const uint32_t n0 = hi1 ^ c1[i] ^ k0, n2 = hi0 ^ c3[i] ^ k1;
                c0[i] = n0;
                c1[i] = lo1;
                c2[i] = n2;
                c3[i] = lo0;
            }
            k0 += 0x9E3779B9u;
            k1 += 0xBB67AE85u;
        }
#endif
        // interleave the four words of every quad: element e of the block takes noise[e]
        uint32_t noise[4 * kBlockQuads];
        for (int i = 0; i < nq; ++i) {
            noise[4 * i] = c0[i];
            noise[4 * i + 1] = c1[i];
            noise[4 * i + 2] = c2[i];
            noise[4 * i + 3] = c3[i];
        }
        const long long e_begin = q0 * 4;
        const long long e_end = (e_begin + 4ll * nq) < n ? (e_begin + 4ll * nq) : n;
        const int cnt = (int)(e_end - e_begin);
        uint16_t* __restrict__ pp = p + e_begin;
        uint16_t* __restrict__ mm = m + e_begin;
        uint16_t* __restrict__ vv = v + e_begin;
        const uint16_t* __restrict__ gg = g + e_begin;
        // branch-free element update (vectorises: shifts, multiplies, sqrt, divide, selects)
        for (int e = 0; e < cnt; ++e) {
            float gf = bf16_to_f32(gg[e]);
            if (has_scale) gf = bf16_to_f32(f32_to_bf16_rn(gf * scale));
            const float mn = bf16_to_f32(mm[e]) * beta1 + gf * one_minus_beta1;
            const float vn = bf16_to_f32(vv[e]) * beta2 + (gf * gf) * one_minus_beta2;
            const float denom = std::sqrt(vn) / bc2_sqrt + eps;
            const float pn = bf16_to_f32(pp[e]) * wd_factor - (step_size * mn) / denom;
            mm[e] = f32_to_bf16_rn(mn);
            vv[e] = sr_to_bf16(vn, noise[e] >> 16);
            pp[e] = sr_to_bf16(pn, noise[e] & 0xFFFFu);
        }
    }
    return 0;
}

int halo_host_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
