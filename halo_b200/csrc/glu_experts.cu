// Element-wise half of routed experts with per-expert bias vectors and a clamped GLU (the gpt-oss expert form), on rows
// grouped by expert:
//
//   pre  = x W_gate_up^T + b_gate_up[e]                    (bias, clamp and activation run in the grouped GEMM's epilogue)
//   gate = min(pre[:F], limit);  up = clamp(pre[F:], -limit, limit)
//   act  = (up + 1) * gate * sigmoid(alpha * gate)
//   y    = act W_down^T + b_down[e]                        (bias added to the rows of the second grouped GEMM)
//
//   expert_glu_bwd        dpre (over pre) and w * act (over the incoming dact), per-row <dact, act> for the routing weights
//   expert_add_bias_rows  y_rows += b_down[e], or per-row <dy, b_down[e]> added to the routing-weight gradient
//   expert_colsum         per-expert column sums of a row buffer (optionally weighted per row): the bias gradients,
//                         one thread per (expert, column), rows in order, so the sums are reproducible
//
// Rows of expert e are seg_start[e] .. seg_start[e] + seg_rows[e] - 1; segments start on multiples of 128 rows and the
// rows between a segment's end and the next start are pads. A row's expert is found by bisection over seg_start.
// Pad rows get their expert's bias like any other row: nothing reads them back (the combine addresses real rows only,
// and the backward scales them by a routing weight of zero). The forward's bias + clamp + activation is the
// kEpiClampedGlu epilogue of the grouped GEMM (gemm_sm100.cuh); this file holds what has no product to ride on.
//
// Native form of the gpt-oss branch of halo/models/moe/experts.py and the bias / clamp epilogues of
// halo/kernels/fused_glu.py:118-205.
#include "sm100_common.cuh"

namespace halo {

__device__ __forceinline__ float wsum_glu(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// the expert whose segment holds (or precedes) row r: the last e with seg_start[e] <= r
__device__ __forceinline__ int expert_of_row(const int* __restrict__ seg_start, int n_local, long long r) {
    int lo = 0, hi = n_local - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (seg_start[mid] <= r) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// one warp per row; 8 bf16 per lane per step. dpre may be pre and act_w may be dact (in place): a thread reads the vectors it overwrites before it writes them
__global__ void __launch_bounds__(256)
expert_glu_bwd_kernel(const __nv_bfloat16* pre, const __nv_bfloat16* dact, const float* __restrict__ w,
                      __nv_bfloat16* dpre, __nv_bfloat16* act_w, float* __restrict__ dwrow,
                      const int* __restrict__ total_rows, int F, int cap_rows, float limit, float alpha) {
    const int lane = threadIdx.x & 31;
    const int rows = min(*total_rows, cap_rows);
    const int nvec = F / 8;
    for (long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); r < rows; r += (long long)gridDim.x * 8) {
        const float sc = w[r];
        const __nv_bfloat16* pg = pre + r * 2 * F;
        float dot = 0.f;
        for (int v = lane; v < nvec; v += 32) {
            const uint4 gu = *reinterpret_cast<const uint4*>(pg + v * 8);
            const uint4 uu = *reinterpret_cast<const uint4*>(pg + F + v * 8);
            const uint4 du = *reinterpret_cast<const uint4*>(dact + r * F + v * 8);
            const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gu);
            const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uu);
            const __nv_bfloat162* dh = reinterpret_cast<const __nv_bfloat162*>(&du);
            uint4 og, ou, oa;
            __nv_bfloat162* ogh = reinterpret_cast<__nv_bfloat162*>(&og);
            __nv_bfloat162* ouh = reinterpret_cast<__nv_bfloat162*>(&ou);
            __nv_bfloat162* oah = reinterpret_cast<__nv_bfloat162*>(&oa);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 g = __bfloat1622float2(gh[q]), u = __bfloat1622float2(uh[q]), d = __bfloat1622float2(dh[q]);
                float og2[2], ou2[2], oa2[2];
                const float gs[2] = {g.x, g.y}, us[2] = {u.x, u.y}, ds[2] = {d.x, d.y};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float gc = fminf(gs[h], limit);
                    const float uc = fminf(fmaxf(us[h], -limit), limit);
                    const float sg = sigmoid_fast(alpha * gc);
                    const float glu = gc * sg;
                    // the forward rounded act to bf16 before the down projection; use the same value here
                    const float a = __bfloat162float(__float2bfloat16_rn((uc + 1.f) * glu));
                    dot += ds[h] * a;
                    const float dx = ds[h] * sc;
                    // the clamps pass a gradient on their closed range, as tensor clamps do
                    ou2[h] = (us[h] >= -limit && us[h] <= limit) ? dx * glu : 0.f;
                    og2[h] = (gs[h] <= limit) ? dx * (uc + 1.f) * sg * (1.f + alpha * gc * (1.f - sg)) : 0.f;
                    oa2[h] = a * sc;
                }
                ogh[q] = __floats2bfloat162_rn(og2[0], og2[1]);
                ouh[q] = __floats2bfloat162_rn(ou2[0], ou2[1]);
                oah[q] = __floats2bfloat162_rn(oa2[0], oa2[1]);
            }
            *reinterpret_cast<uint4*>(dpre + r * 2 * F + v * 8) = og;
            *reinterpret_cast<uint4*>(dpre + r * 2 * F + F + v * 8) = ou;
            *reinterpret_cast<uint4*>(act_w + r * F + v * 8) = oa;
        }
        dot = wsum_glu(dot);
        if (lane == 0) dwrow[r] = dot;
    }
}

// mode 0: rows[r] += bias[e(r)]; mode 1: rowdot[r] += <rows[r], bias[e(r)]> (rows untouched)
template <int kMode>
__global__ void __launch_bounds__(256)
expert_bias_rows_kernel(__nv_bfloat16* rows_buf, const __nv_bfloat16* __restrict__ bias, float* __restrict__ rowdot,
                        const int* __restrict__ seg_start, int n_local, const int* __restrict__ total_rows, int H,
                        int cap_rows) {
    const int lane = threadIdx.x & 31;
    const int rows = min(*total_rows, cap_rows);
    const int nvec = H / 8;
    for (long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); r < rows; r += (long long)gridDim.x * 8) {
        const int e = expert_of_row(seg_start, n_local, r);
        __nv_bfloat16* pr = rows_buf + r * H;
        const __nv_bfloat16* pb = bias + (long long)e * H;
        float dot = 0.f;
        for (int v = lane; v < nvec; v += 32) {
            const uint4 xu = *reinterpret_cast<const uint4*>(pr + v * 8);
            const uint4 bu = *reinterpret_cast<const uint4*>(pb + v * 8);
            const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xu);
            const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&bu);
            uint4 o;
            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 x = __bfloat1622float2(xh[q]), b = __bfloat1622float2(bh[q]);
                if (kMode == 0) oh[q] = __floats2bfloat162_rn(x.x + b.x, x.y + b.y);
                else dot += x.x * b.x + x.y * b.y;
            }
            if (kMode == 0) *reinterpret_cast<uint4*>(pr + v * 8) = o;
        }
        if (kMode == 1) {
            dot = wsum_glu(dot);
            if (lane == 0) rowdot[r] += dot;
        }
    }
}

// out[e, c] = sum over the rows r of expert e of (w ? w[r] : 1) * src[r, c]; one thread per column, rows in order
__global__ void __launch_bounds__(256)
expert_colsum_kernel(const __nv_bfloat16* __restrict__ src, const float* __restrict__ w, float* __restrict__ out,
                     const int* __restrict__ seg_start, const int* __restrict__ seg_rows, int C, int cap_rows) {
    const int e = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const long long r0 = seg_start[e];
    const long long r1 = min((long long)cap_rows, r0 + seg_rows[e]);
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;     // four rows in flight; a fixed order of additions
    long long r = r0;
    for (; r + 3 < r1; r += 4) {
        const float w0 = w ? w[r] : 1.f, w1 = w ? w[r + 1] : 1.f, w2 = w ? w[r + 2] : 1.f, w3 = w ? w[r + 3] : 1.f;
        acc0 += w0 * __bfloat162float(src[r * C + c]);
        acc1 += w1 * __bfloat162float(src[(r + 1) * C + c]);
        acc2 += w2 * __bfloat162float(src[(r + 2) * C + c]);
        acc3 += w3 * __bfloat162float(src[(r + 3) * C + c]);
    }
    for (; r < r1; ++r) acc0 += (w ? w[r] : 1.f) * __bfloat162float(src[r * C + c]);
    out[(long long)e * C + c] = (acc0 + acc1) + (acc2 + acc3);
}

}  // namespace halo

#define HALO_LAUNCH_CHECK() (cudaGetLastError() == cudaSuccess ? 0 : -11)

extern "C" {
using namespace halo;

int halo_expert_glu_bwd(const void* pre, const void* dact, const float* w, void* dpre, void* act_w, float* dwrow,
                        const int* total_rows, int F, int cap_rows, float limit, float alpha, void* stream) {
    if (F % 8) return -1;
    expert_glu_bwd_kernel<<<2368, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)pre, (const __nv_bfloat16*)dact, w, (__nv_bfloat16*)dpre, (__nv_bfloat16*)act_w, dwrow,
        total_rows, F, cap_rows, limit, alpha);
    return HALO_LAUNCH_CHECK();
}

int halo_expert_add_bias_rows(void* rows, const void* bias, const int* seg_start, int n_local, const int* total_rows,
                              int H, int cap_rows, void* stream) {
    if (H % 8 || n_local <= 0) return -1;
    expert_bias_rows_kernel<0><<<2368, 256, 0, (cudaStream_t)stream>>>(
        (__nv_bfloat16*)rows, (const __nv_bfloat16*)bias, nullptr, seg_start, n_local, total_rows, H, cap_rows);
    return HALO_LAUNCH_CHECK();
}

int halo_expert_bias_rowdot(const void* rows, const void* bias, float* rowdot, const int* seg_start, int n_local,
                            const int* total_rows, int H, int cap_rows, void* stream) {
    if (H % 8 || n_local <= 0) return -1;
    expert_bias_rows_kernel<1><<<2368, 256, 0, (cudaStream_t)stream>>>(
        (__nv_bfloat16*)const_cast<void*>(rows), (const __nv_bfloat16*)bias, rowdot, seg_start, n_local, total_rows, H,
        cap_rows);
    return HALO_LAUNCH_CHECK();
}

int halo_expert_colsum(const void* src, const float* w, float* out, const int* seg_start, const int* seg_rows,
                       int n_local, int C, int cap_rows, void* stream) {
    if (n_local <= 0 || C <= 0) return -1;
    expert_colsum_kernel<<<dim3((C + 255) / 256, n_local), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)src, w, out, seg_start, seg_rows, C, cap_rows);
    return HALO_LAUNCH_CHECK();
}

}  // extern "C"
