// Dequantisation of 4-bit block-quantised weights (QLoRA base matrices) to bf16.
//   codes  : uint8 [n / 2], two 4-bit level indices per byte, the first value in the high nibble
//   maxima : fp32 [n / 64], the absolute maximum of each block of 64 values
//   levels : 16 fp32 levels in [-1, 1] (nf4: normal quantiles; fp4: the e2m1 grid / 6), passed by value
// A thread turns 8 bytes (16 values, one quarter of a block) into two 16-byte stores: the kernel reads 0.5 byte and
// writes 2 bytes per value, so its floor is the HBM write of the bf16 matrix.
// value = levels[code] * maxima[block], rounded to bf16 once (the same single rounding as the tensor-op statement).
//
// Behavioural counterpart: the bitsandbytes 4-bit dequantisation the reference reaches through load_in_4bit
// (halo/model_loading/dtype.py:114-119).
#include "sm100_common.cuh"

namespace halo {
namespace nf4 {

struct Levels {
    float v[16];
};

__global__ void __launch_bounds__(256) dequant_kernel(const uint2* __restrict__ codes, const float* __restrict__ maxima,
                                                      __nv_bfloat16* __restrict__ out, long long n_chunks, Levels levels) {
    __shared__ float table[16];
    if (threadIdx.x < 16) table[threadIdx.x] = levels.v[threadIdx.x];
    __syncthreads();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_chunks; i += stride) {
        const uint2 c = codes[i];                  // 8 bytes = 16 values; chunk i lies in block i / 4
        const float m = maxima[i >> 2];
        const unsigned words[2] = {c.x, c.y};
        __nv_bfloat162 o[8];
#pragma unroll
        for (int w = 0; w < 2; ++w) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const unsigned byte = (words[w] >> (8 * b)) & 0xFFu;      // little-endian: byte b of the word
                o[w * 4 + b] = __floats2bfloat162_rn(table[byte >> 4] * m, table[byte & 0xFu] * m);
            }
        }
        uint4* dst = reinterpret_cast<uint4*>(out + i * 16);
        dst[0] = *reinterpret_cast<const uint4*>(&o[0]);
        dst[1] = *reinterpret_cast<const uint4*>(&o[4]);
    }
}

}  // namespace nf4
}  // namespace halo

extern "C" {

// n: number of values, a multiple of 64; codes / out 16-byte aligned (8 for codes). levels: 16 floats on the host.
int halo_dequant_4bit_bf16(const void* codes, const float* maxima, void* out, long long n, const float* levels, void* stream) {
    if (n < 0 || n % 64 || levels == nullptr) return -1;
    if (n == 0) return 0;
    if ((reinterpret_cast<uintptr_t>(codes) & 7u) || (reinterpret_cast<uintptr_t>(out) & 15u)) return -2;
    halo::nf4::Levels lv;
    for (int i = 0; i < 16; ++i) lv.v[i] = levels[i];
    const long long n_chunks = n / 16;
    long long blocks = (n_chunks + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    halo::nf4::dequant_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
        (const uint2*)codes, maxima, (__nv_bfloat16*)out, n_chunks, lv);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
