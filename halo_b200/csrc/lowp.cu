// Block-scaled fake quantisation (quantise then dequantise in one pass) for the OCP MX formats and NVFP4:
//   mxfp8: e4m3 elements, one e8m0 (power-of-two) scale per 32 elements of the contraction axis
//   mxfp4: e2m1 elements, one e8m0 scale per 32 elements
//   nvfp4: e2m1 elements, one e4m3 scale per 16 elements times one fp32 power-of-two scale per tensor
// The input is bf16 [rows, K] with K a multiple of the block; a lane owns one 16-byte vector (8 elements), so a
// block is 4 (or 2) adjacent lanes and its abs-max is two (one) shuffles. Memory-bound: one read, one write.
//
// The arithmetic is exact where it can be, so that the PyTorch statement of the same round trip gives identical
// bits: the power-of-two exponent comes from frexp (no log2 rounding), scaling by it from ldexp, e2m1 rounding is
// a count of passed midpoints with ties to the even code, e4m3 rounding is the hardware conversion
// (round-to-nearest-even, saturating).
//
// Behavioural counterpart: halo/kernels/lowp/fake_quant_triton.py:101-181 and quantization.py:148-215.
#include "sm100_common.cuh"

#include <cuda_fp8.h>

namespace halo {
namespace lowp {

constexpr int kMxfp8 = 0, kMxfp4 = 1, kNvfp4 = 2;
constexpr float kE4M3Max = 448.f, kE2M1Max = 6.f;
constexpr float kAmaxFloor = 1.17549435e-38f;   // smallest normal fp32: keeps an all-zero block's exponent finite

// smallest integer e with r <= 2^e, for r > 0 (exact: frexp gives r = m * 2^x with m in [0.5, 1))
__device__ __forceinline__ int ceil_log2(float r) {
    int x;
    const float m = frexpf(r, &x);
    return m == 0.5f ? x - 1 : x;
}
__device__ __forceinline__ float e4m3_round(float v) {
    const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
    return __half2float(__half(__nv_cvt_fp8_to_halfraw(q, __NV_E4M3)));
}
// e2m1 magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6: the code is the number of midpoints passed; a tie goes to the even code
__device__ __forceinline__ float e2m1_round(float v) {
    const float mag = fminf(fabsf(v), kE2M1Max);
    const int code = (mag > 0.25f) + (mag >= 0.75f) + (mag > 1.25f) + (mag >= 1.75f) + (mag > 2.5f) + (mag >= 3.5f) + (mag > 5.f);
    const float levels[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    return copysignf(levels[code], v);
}

template <int FMT>
__global__ void __launch_bounds__(256) fake_quant_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                                         long long n_vec, const float* __restrict__ tensor_amax) {
    constexpr int kLanesPerBlock = FMT == kNvfp4 ? 2 : 4;
    constexpr float kElemMax = FMT == kMxfp8 ? kE4M3Max : kE2M1Max;
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
    float global_scale = 1.f;
    if (FMT == kNvfp4) global_scale = ldexpf(1.f, ceil_log2(fmaxf(*tensor_amax, kAmaxFloor) / (kE4M3Max * kE2M1Max)));
    for (long long base = warp * 32; base < n_vec; base += n_warps * 32) {
        const long long i = base + lane;
        const bool live = i < n_vec;       // n_vec is a multiple of kLanesPerBlock and base of 32: a block is all live or all idle
        float f[8];
        if (live) {
            const uint4 u = reinterpret_cast<const uint4*>(x)[i];
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 t = __bfloat1622float2(h[j]);
                f[2 * j] = t.x;
                f[2 * j + 1] = t.y;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = 0.f;
        }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
#pragma unroll
        for (int o = kLanesPerBlock / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        float o8[8];
        if (FMT == kNvfp4) {
            const float scale = e4m3_round(fminf(amax / kE2M1Max / global_scale, kE4M3Max));
            const float unit = scale * global_scale;
            const float divisor = unit == 0.f ? 1.f : unit;
#pragma unroll
            for (int j = 0; j < 8; ++j) o8[j] = e2m1_round(f[j] / divisor) * unit;
        } else {
            int e = ceil_log2(fmaxf(amax, kAmaxFloor) / kElemMax);
            e = e < -127 ? -127 : (e > 127 ? 127 : e);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float scaled = fminf(fmaxf(ldexpf(f[j], -e), -kElemMax), kElemMax);
                const float q = FMT == kMxfp8 ? e4m3_round(scaled) : e2m1_round(scaled);
                o8[j] = ldexpf(q, e);
            }
        }
        if (live)
            reinterpret_cast<uint4*>(y)[i] = make_uint4(pack_bf16(o8[0], o8[1]), pack_bf16(o8[2], o8[3]), pack_bf16(o8[4], o8[5]),
                                                        pack_bf16(o8[6], o8[7]));
    }
}

}  // namespace lowp
}  // namespace halo

extern "C" {

// fmt: 0 = mxfp8, 1 = mxfp4, 2 = nvfp4 (tensor_amax: device pointer to max |x| over the tensor, nvfp4 only).
// numel must be a multiple of the format's block (32, 32, 16) and the blocks must lie along contiguous memory.
int halo_fake_quant_bf16(const void* x, void* y, long long numel, int fmt, const float* tensor_amax, void* stream) {
    using namespace halo::lowp;
    const int block = fmt == kNvfp4 ? 16 : 32;
    if (fmt < 0 || fmt > 2 || numel < 0 || numel % block) return -1;
    if (fmt == kNvfp4 && tensor_amax == nullptr) return -1;
    if (numel == 0) return 0;
    const long long n_vec = numel / 8;
    long long blocks = (n_vec + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    cudaStream_t s = (cudaStream_t)stream;
    if (fmt == kMxfp8)
        fake_quant_kernel<kMxfp8><<<(unsigned)blocks, 256, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n_vec, tensor_amax);
    else if (fmt == kMxfp4)
        fake_quant_kernel<kMxfp4><<<(unsigned)blocks, 256, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n_vec, tensor_amax);
    else
        fake_quant_kernel<kNvfp4><<<(unsigned)blocks, 256, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n_vec, tensor_amax);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
