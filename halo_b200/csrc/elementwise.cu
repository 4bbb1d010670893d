// Memory-bound kernels of the decoder layer: RMSNorm (with the residual add folded in), the
// per-head q/k RMSNorm + rotary embedding of Qwen3 attention, SwiGLU, and the row-wise
// cross-entropy that turns a logits chunk into its gradient in place. All math is fp32 on bf16
// storage with 16-byte accesses; each kernel touches every byte once.
//
// They stand where the reference swaps in Liger's Triton RMSNorm / RoPE / SwiGLU / cross-entropy
// or ATen's rms_norm (halo/model_loading/liger/dispatch.py:416, family_specs.py:34-36) and its
// own GLU kernel (halo/kernels/fused_glu.py:118-205).
#include "sm100_common.cuh"

#include <stdio.h>

#include "halo_noalloc.h"

namespace halo {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float bf16_round(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]),
                      pack_bf16(f[6], f[7]));
}

// ---------------------------------------------------------------------------------------------
// RMSNorm forward. L threads share a row (L = 32, 128 or 256), each owning VPT 8-element vectors:
// H = 8 * L * VPT. Optional residual: h = x + res (written to h_out), y = norm(h).
//   y = w * bf16(h * rstd)   (the rounding order of the Hugging Face Qwen3 module)
// ---------------------------------------------------------------------------------------------
template <int L>
__device__ __forceinline__ float row_sum(float v, float* scratch /* [256/32] floats */) {
    v = warp_sum(v);
    if (L == 32) return v;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int WPR = L / 32;  // warps per row
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float s = 0.f;
    const int first = (warp / WPR) * WPR;
#pragma unroll
    for (int i = 0; i < WPR; ++i) s += scratch[first + i];
    return s;
}

template <int VPT, int L>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, long long rows,
                   int H, float eps) {
    __shared__ float scratch[8];
    constexpr int RPB = 256 / L;
    const int tl = threadIdx.x % L;
    long long row = (long long)blockIdx.x * RPB + threadIdx.x / L;
    const bool live = row < rows;
    if (!live) row = rows - 1;  // keep every thread in the block-wide reduction
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
    const uint4* rr = res ? reinterpret_cast<const uint4*>(res + row * H) : nullptr;
    float v[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        unpack8(xr[tl + L * i], v[i]);
        if (rr) {
            float r[8];
            unpack8(rr[tl + L * i], r);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] = bf16_round(v[i][j] + r[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
    ss = row_sum<L>(ss, scratch);
    if (!live) return;
    const float rstd = rsqrtf(ss / (float)H + eps);
    if (tl == 0 && rstd_out) rstd_out[row] = rstd;
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    uint4* yr = reinterpret_cast<uint4*>(y + row * H);
    uint4* hr = h_out ? reinterpret_cast<uint4*>(h_out + row * H) : nullptr;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        if (hr) hr[tl + L * i] = pack8(v[i]);
        float wv[8], o[8];
        unpack8(wr[tl + L * i], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = wv[j] * bf16_round(v[i][j] * rstd);
        yr[tl + L * i] = pack8(o);
    }
}

// RMSNorm backward. dx = rstd * (g*w - xhat * mean(g*w*xhat)) (+ dres); per-block partial dw.
// A fixed grid walks the rows so the partial-sum buffer stays [gridDim.x, H].
template <int VPT, int L>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ h,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, long long rows, int H) {
    __shared__ float scratch[8];
    constexpr int RPB = 256 / L;
    const int tl = threadIdx.x % L, rg = threadIdx.x / L;
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    float wv[VPT][8], dwacc[VPT][8];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        unpack8(wr[tl + L * i], wv[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    }
    const long long n_iter = (rows + (long long)gridDim.x * RPB - 1) / ((long long)gridDim.x * RPB);
    for (long long it = 0; it < n_iter; ++it) {
        long long row = (it * gridDim.x + blockIdx.x) * RPB + rg;
        const bool live = row < rows;
        if (!live) row = rows - 1;
        const uint4* gr = reinterpret_cast<const uint4*>(g + row * H);
        const uint4* hr = reinterpret_cast<const uint4*>(h + row * H);
        const float rs = rstd[row];
        float gw[VPT][8], xh[VPT][8];
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            float gv[8], hv[8];
            unpack8(gr[tl + L * i], gv);
            unpack8(hr[tl + L * i], hv);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                xh[i][j] = hv[j] * rs;
                gw[i][j] = gv[j] * wv[i][j];
                dot += gw[i][j] * xh[i][j];
                if (live) dwacc[i][j] += gv[j] * xh[i][j];
            }
        }
        dot = row_sum<L>(dot, scratch) / (float)H;
        if (!live) continue;
        uint4* dxr = reinterpret_cast<uint4*>(dx + row * H);
        const uint4* dr = dres ? reinterpret_cast<const uint4*>(dres + row * H) : nullptr;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = rs * (gw[i][j] - xh[i][j] * dot);
            if (dr) {
                float r[8];
                unpack8(dr[tl + L * i], r);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] += r[j];
            }
            dxr[tl + L * i] = pack8(o);
        }
    }
    // fold the RPB row groups of this block, which own the same columns, then write the partial
    __shared__ float red[RPB > 1 ? RPB : 1][L * 8 + 1];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 8; ++j) red[rg][tl * 8 + j] = dwacc[i][j];
        __syncthreads();
        for (int c = threadIdx.x; c < L * 8; c += 256) {
            float s = 0.f;
#pragma unroll
            for (int q = 0; q < RPB; ++q) s += red[q][c];
            // column of element (vector tl' + L*i, lane j): (tl' + L*i)*8 + j with c = tl'*8 + j
            dw_partial[(long long)blockIdx.x * H + (long long)i * L * 8 + c] = s;
        }
    }
}

__global__ void reduce_partials_kernel(const float* __restrict__ partial, int n_partials, int H,
                                       float* __restrict__ out_f32,
                                       __nv_bfloat16* __restrict__ out_bf16, int accumulate) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= H) return;
    float s = 0.f;
    for (int i = 0; i < n_partials; ++i) s += partial[(long long)i * H + c];
    if (out_f32) out_f32[c] = accumulate ? out_f32[c] + s : s;
    if (out_bf16)
        out_bf16[c] = __float2bfloat16_rn(accumulate ? __bfloat162float(out_bf16[c]) + s : s);
}

// ---------------------------------------------------------------------------------------------
// Rotary table: cos/sin of pos * theta^(-2i/D), i < D/2, rounded to bf16 as the module does.
// ---------------------------------------------------------------------------------------------
__global__ void rope_table_kernel(const int* __restrict__ pos, long long T, int half, float theta,
                                  float2* __restrict__ table) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * half) return;
    const long long t = i / half;
    const int k = (int)(i % half);
    const float inv = powf(theta, -(float)(2 * k) / (float)(2 * half));
    float s, c;
    sincosf((float)pos[t] * inv, &s, &c);
    table[i] = make_float2(bf16_round(c), bf16_round(s));
}

// q/k RMSNorm over head_dim (=128) + rotate-half RoPE. One warp per (token, head); lane owns
// elements [4*lane, 4*lane+4), its rotation partner is lane ^ 16.
//   qkv: [T, (Hq + 2*Hkv) * 128] raw projections;  q_out: [T, Hq*128];  k_out: [T, Hkv*128]
__global__ void __launch_bounds__(256)
qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ wq,
                       const __nv_bfloat16* __restrict__ wk, const float2* __restrict__ table,
                       __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out,
                       float* __restrict__ rstd_out, long long T, int Hq, int Hkv, float eps,
                       int use_norm) {
    const int lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int heads = Hq + Hkv;
    if (wid >= T * heads) return;
    const long long t = wid / heads;
    const int hd = (int)(wid % heads);
    const long long in_ld = (long long)(Hq + 2 * Hkv) * 128;
    const __nv_bfloat16* src = qkv + t * in_ld + (long long)hd * 128 + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float2 a = __bfloat1622float2(rh[0]), b = __bfloat1622float2(rh[1]);
    float v[4] = {a.x, a.y, b.x, b.y};
    float rstd = 1.f;
    if (use_norm) {
        float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
        rstd = rsqrtf(ss / 128.f + eps);
        if (lane == 0) rstd_out[wid] = rstd;
        const __nv_bfloat16* w = (hd < Hq ? wq : wk) + lane * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = bf16_round(__bfloat162float(w[j]) * bf16_round(v[j] * rstd));
    }
    float o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float partner = __shfl_xor_sync(0xffffffffu, v[j], 16);
        const float2 cs = table[t * 64 + ((lane & 15) * 4 + j)];
        // first half: x*cos - partner*sin ; second half: x*cos + partner*sin
        const float rot = (lane < 16) ? -partner : partner;
        o[j] = bf16_round(v[j] * cs.x) + bf16_round(rot * cs.y);
    }
    __nv_bfloat16* dst = (hd < Hq) ? q_out + t * (long long)Hq * 128 + (long long)hd * 128 + lane * 4
                                   : k_out + t * (long long)Hkv * 128 + (long long)(hd - Hq) * 128 + lane * 4;
    *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
}

// Backward: undo the rotation on the incoming gradient, then RMSNorm backward per head.
//   dq: [T, Hq*128], dk: [T, Hkv*128] -> dqkv[:, : (Hq+Hkv)*128]; per-block partial dwq / dwk.
__global__ void __launch_bounds__(256)
qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk,
                       const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ wq,
                       const __nv_bfloat16* __restrict__ wk, const float2* __restrict__ table,
                       const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dqkv,
                       float* __restrict__ dw_partial, long long T, int Hq, int Hkv, int use_norm) {
    __shared__ float red[8][2][128];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int heads = Hq + Hkv;
    const long long in_ld = (long long)(Hq + 2 * Hkv) * 128;
    float dwq_acc[4] = {0, 0, 0, 0}, dwk_acc[4] = {0, 0, 0, 0};
    float wqv[4], wkv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        wqv[j] = use_norm ? __bfloat162float(wq[lane * 4 + j]) : 1.f;
        wkv[j] = use_norm ? __bfloat162float(wk[lane * 4 + j]) : 1.f;
    }
    const long long total = T * heads;
    for (long long wid = (long long)blockIdx.x * 8 + warp; wid < total; wid += (long long)gridDim.x * 8) {
        const long long t = wid / heads;
        const int hd = (int)(wid % heads);
        const bool is_q = hd < Hq;
        const __nv_bfloat16* gsrc = is_q ? dq + t * (long long)Hq * 128 + (long long)hd * 128 + lane * 4
                                         : dk + t * (long long)Hkv * 128 + (long long)(hd - Hq) * 128 + lane * 4;
        const uint2 graw = *reinterpret_cast<const uint2*>(gsrc);
        const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&graw);
        float2 ga = __bfloat1622float2(gh[0]), gb = __bfloat1622float2(gh[1]);
        float go[4] = {ga.x, ga.y, gb.x, gb.y};
        float gn[4];  // gradient w.r.t. the normalised, weighted vector
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float partner = __shfl_xor_sync(0xffffffffu, go[j], 16);
            const float2 cs = table[t * 64 + ((lane & 15) * 4 + j)];
            // transpose of the rotation: first half gets +partner*sin, second half -partner*sin
            gn[j] = go[j] * cs.x + ((lane < 16) ? partner : -partner) * cs.y;
        }
        float out[4];
        if (use_norm) {
            const __nv_bfloat16* src = qkv + t * in_ld + (long long)hd * 128 + lane * 4;
            const uint2 raw = *reinterpret_cast<const uint2*>(src);
            const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&raw);
            float2 a = __bfloat1622float2(rh[0]), b = __bfloat1622float2(rh[1]);
            const float x[4] = {a.x, a.y, b.x, b.y};
            const float rs = rstd_in[wid];
            float dot = 0.f, xh[4], gw[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                xh[j] = x[j] * rs;
                gw[j] = gn[j] * (is_q ? wqv[j] : wkv[j]);
                dot += gw[j] * xh[j];
                if (is_q) dwq_acc[j] += gn[j] * xh[j];
                else dwk_acc[j] += gn[j] * xh[j];
            }
            dot = warp_sum(dot) / 128.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) out[j] = rs * (gw[j] - xh[j] * dot);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) out[j] = gn[j];
        }
        __nv_bfloat16* dst = dqkv + t * in_ld + (long long)hd * 128 + lane * 4;
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(out[0], out[1]), pack_bf16(out[2], out[3]));
    }
    if (use_norm && dw_partial) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            red[warp][0][lane * 4 + j] = dwq_acc[j];
            red[warp][1][lane * 4 + j] = dwk_acc[j];
        }
        __syncthreads();
        const int which = threadIdx.x >> 7, c = threadIdx.x & 127;
        float s = 0.f;
#pragma unroll
        for (int wq_ = 0; wq_ < 8; ++wq_) s += red[wq_][which][c];
        dw_partial[(long long)blockIdx.x * 256 + which * 128 + c] = s;
    }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU on a packed [rows, 2F] pre-activation (gate | up).
// ---------------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ pre, __nv_bfloat16* __restrict__ act,
                                  long long rows, int F) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int vec_per_row = F / 8;
    if (i >= rows * vec_per_row) return;
    const long long r = i / vec_per_row;
    const int c = (int)(i % vec_per_row) * 8;
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(pre + r * 2 * F + c), g);
    unpack8(*reinterpret_cast<const uint4*>(pre + r * 2 * F + F + c), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    *reinterpret_cast<uint4*>(act + r * F + c) = pack8(o);
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ pre, const __nv_bfloat16* __restrict__ dact,
                                  __nv_bfloat16* __restrict__ dpre, long long rows, int F) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int vec_per_row = F / 8;
    if (i >= rows * vec_per_row) return;
    const long long r = i / vec_per_row;
    const int c = (int)(i % vec_per_row) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const uint4*>(pre + r * 2 * F + c), g);
    unpack8(*reinterpret_cast<const uint4*>(pre + r * 2 * F + F + c), u);
    unpack8(*reinterpret_cast<const uint4*>(dact + r * F + c), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float s = 1.f / (1.f + __expf(-g[j]));
        du[j] = d[j] * g[j] * s;
        dg[j] = d[j] * u[j] * s * (1.f + g[j] * (1.f - s));
    }
    *reinterpret_cast<uint4*>(dpre + r * 2 * F + c) = pack8(dg);
    *reinterpret_cast<uint4*>(dpre + r * 2 * F + F + c) = pack8(du);
}

// ---------------------------------------------------------------------------------------------
// Cross-entropy over one logits chunk [rows, V] (bf16), in place: on return the chunk holds
// grad_scale * row_scale[row] * (softmax - onehot) and loss_rows / lse carry the forward results.
// One block per row.
// Rows whose label is ignore_index get a zero gradient.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512)
cross_entropy_inplace_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                             const float* __restrict__ grad_scale, const float* __restrict__ row_scale,
                             float* __restrict__ loss_rows,
                             float* __restrict__ lse_out, long long ld, int V, long long ignore_index) {
    __shared__ float sm[16], ss[16];
    __shared__ float row_lse;
    const long long row = blockIdx.x;
    __nv_bfloat16* lr = logits + row * ld;
    const long long label = labels[row];
    const int nvec = V / 8;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // online max / sum
    float m = -INFINITY, s = 0.f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(lr + i * 8), f);
        float lm = f[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
        const float nm = fmaxf(m, lm);
        float add = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) add += __expf(f[j] - nm);
        s = s * __expf(m - nm) + add;
        m = nm;
    }
    for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) {
        const float f = __bfloat162float(lr[i]);
        const float nm = fmaxf(m, f);
        s = s * __expf(m - nm) + __expf(f - nm);
        m = nm;
    }
    const float wm = warp_max(m);
    s = warp_sum(m == -INFINITY ? 0.f : s * __expf(m - wm));  // a thread (or a whole warp) may own no column
    if (lane == 0) { sm[warp] = wm; ss[warp] = s; }
    __syncthreads();
    if (warp == 0) {
        float mm = lane < (int)(blockDim.x >> 5) ? sm[lane] : -INFINITY;
        float sv = lane < (int)(blockDim.x >> 5) ? ss[lane] : 0.f;
        const float gm = warp_max(mm);
        sv = warp_sum(mm == -INFINITY ? 0.f : sv * __expf(mm - gm));
        if (lane == 0) row_lse = gm + logf(sv);
    }
    __syncthreads();
    const float lse = row_lse;
    const bool ignored = (label == ignore_index);
    if (threadIdx.x == 0) {
        if (lse_out) lse_out[row] = lse;
        loss_rows[row] = ignored ? 0.f : lse - __bfloat162float(lr[label]);
    }
    __syncthreads();  // the label logit is read before it is overwritten
    const float gs = ignored ? 0.f : (grad_scale ? *grad_scale : 1.f) * (row_scale ? row_scale[row] : 1.f);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(lr + i * 8), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float p = __expf(f[j] - lse);
            if ((long long)(i * 8 + j) == label) p -= 1.f;
            f[j] = p * gs;
        }
        *reinterpret_cast<uint4*>(lr + i * 8) = pack8(f);
    }
    for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) {
        float p = __expf(__bfloat162float(lr[i]) - lse);
        if ((long long)i == label) p -= 1.f;
        lr[i] = __float2bfloat16_rn(p * gs);
    }
}

// Token log-probabilities and entropy from a logits chunk, no gradient (scoring passes of RL).
__global__ void __launch_bounds__(512)
logprob_entropy_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                       float* __restrict__ logp, float* __restrict__ entropy, long long ld, int V,
                       long long ignore_index) {
    __shared__ float sm[16], ss[16], st[16];
    const long long row = blockIdx.x;
    const __nv_bfloat16* lr = logits + row * ld;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float m = -INFINITY, s = 0.f, tsum = 0.f;  // tsum = sum exp(f-m) * f
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float f = __bfloat162float(lr[i]);
        const float nm = fmaxf(m, f);
        const float sc = __expf(m - nm), e = __expf(f - nm);
        s = s * sc + e;
        tsum = tsum * sc + e * f;
        m = nm;
    }
    const float wm = warp_max(m);
    const float sc = (m == -INFINITY) ? 0.f : __expf(m - wm);  // a thread may own no column
    s = warp_sum(s * sc);
    tsum = warp_sum(tsum * sc);
    if (lane == 0) { sm[warp] = wm; ss[warp] = s; st[warp] = tsum; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        float mm = lane < nw ? sm[lane] : -INFINITY;
        float sv = lane < nw ? ss[lane] : 0.f;
        float tv = lane < nw ? st[lane] : 0.f;
        const float gm = warp_max(mm);
        const float c2 = (mm == -INFINITY) ? 0.f : __expf(mm - gm);
        sv = warp_sum(sv * c2);
        tv = warp_sum(tv * c2);
        if (lane == 0) {
            const float lse = gm + logf(sv);
            const long long label = labels[row];
            logp[row] = (label == ignore_index) ? 0.f : __bfloat162float(lr[label]) - lse;
            if (entropy) entropy[row] = lse - tv / sv;
        }
    }
}

}  // namespace halo

using namespace halo;

extern "C" {

#define HALO_LAUNCH_CHECK() (cudaGetLastError() == cudaSuccess ? 0 : -11)

// Pick the threads-per-row L (32, 128, 256) and vectors-per-thread so that H = 8 * L * VPT, VPT <= 4.
static bool rms_shape(int H, int* L, int* vpt) {
    const int cands[3] = {32, 128, 256};
    for (int i = 0; i < 3; ++i) {
        const int l = cands[i];
        if (H % (8 * l) == 0 && H / (8 * l) <= 4) {
            *L = l;
            *vpt = H / (8 * l);
            return true;
        }
    }
    return false;
}

#define RMS_DISPATCH(KERNEL, ...)                                                                \
    if (L == 32) {                                                                               \
        switch (vpt) {                                                                           \
            case 1: KERNEL<1, 32><<<grid, 256, 0, s>>>(__VA_ARGS__); break;                      \
            case 2: KERNEL<2, 32><<<grid, 256, 0, s>>>(__VA_ARGS__); break;                      \
            case 3: KERNEL<3, 32><<<grid, 256, 0, s>>>(__VA_ARGS__); break;                      \
            default: KERNEL<4, 32><<<grid, 256, 0, s>>>(__VA_ARGS__); break;                     \
        }                                                                                        \
    } else if (L == 128) {                                                                       \
        switch (vpt) {                                                                           \
            case 1: KERNEL<1, 128><<<grid, 256, 0, s>>>(__VA_ARGS__); break;                     \
            case 2: KERNEL<2, 128><<<grid, 256, 0, s>>>(__VA_ARGS__); break;                     \
            case 3: KERNEL<3, 128><<<grid, 256, 0, s>>>(__VA_ARGS__); break;                     \
            default: KERNEL<4, 128><<<grid, 256, 0, s>>>(__VA_ARGS__); break;                    \
        }                                                                                        \
    } else {                                                                                     \
        switch (vpt) {                                                                           \
            case 1: KERNEL<1, 256><<<grid, 256, 0, s>>>(__VA_ARGS__); break;                     \
            case 2: KERNEL<2, 256><<<grid, 256, 0, s>>>(__VA_ARGS__); break;                     \
            case 3: KERNEL<3, 256><<<grid, 256, 0, s>>>(__VA_ARGS__); break;                     \
            default: KERNEL<4, 256><<<grid, 256, 0, s>>>(__VA_ARGS__); break;                    \
        }                                                                                        \
    }

int halo_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out,
                     float* rstd, long long rows, int H, float eps, void* stream) {
    int L, vpt;
    if (!rms_shape(H, &L, &vpt)) return -1;
    if (rows == 0) return 0;
    const int rpb = 256 / L;
    dim3 grid((unsigned)((rows + rpb - 1) / rpb));
    cudaStream_t s = (cudaStream_t)stream;
    RMS_DISPATCH(rmsnorm_fwd_kernel, (const __nv_bfloat16*)x, (const __nv_bfloat16*)res,
                 (const __nv_bfloat16*)w, (__nv_bfloat16*)y, (__nv_bfloat16*)h_out, rstd, rows, H, eps)
    return HALO_LAUNCH_CHECK();
}

int halo_rmsnorm_supported(int H) {
    int L, vpt;
    return rms_shape(H, &L, &vpt) ? 1 : 0;
}

int halo_rmsnorm_bwd_blocks(long long rows, int H) {
    int L = 32, vpt = 1;
    rms_shape(H, &L, &vpt);
    const int rpb = 256 / L;
    long long b = (rows + rpb - 1) / rpb;
    static_assert(HALO_NOALLOC_MAX_BLOCKS >= 592, "the built-in scratch must cover the largest grid");
    return (int)(b < 592 ? b : 592);
}

// dw_partial: fp32 scratch of halo_rmsnorm_bwd_blocks(rows, H) * H elements.
int halo_rmsnorm_bwd(const void* g, const void* h, const void* w, const float* rstd,
                     const void* dres, void* dx, float* dw_partial, float* dw_f32, void* dw_bf16,
                     int accumulate, long long rows, int H, void* stream) {
    int L, vpt;
    if (!rms_shape(H, &L, &vpt)) return -1;
    if (rows == 0) return 0;
    const int blocks = halo_rmsnorm_bwd_blocks(rows, H);
    dim3 grid(blocks);
    cudaStream_t s = (cudaStream_t)stream;
    RMS_DISPATCH(rmsnorm_bwd_kernel, (const __nv_bfloat16*)g, (const __nv_bfloat16*)h,
                 (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx,
                 dw_partial, rows, H)
    reduce_partials_kernel<<<(H + 255) / 256, 256, 0, s>>>(dw_partial, blocks, H, dw_f32,
                                                          (__nv_bfloat16*)dw_bf16, accumulate);
    return HALO_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Allocation-free RMSNorm backward (see halo_noalloc.h). The per-block partial sums live in a
// file-scope device array instead of a caller-provided buffer.
// ---------------------------------------------------------------------------------------------
}  // extern "C"

static __device__ __align__(256) float g_noalloc_scratch[HALO_NOALLOC_MAX_BLOCKS * HALO_NOALLOC_MAX_HIDDEN];

// In host code `g_noalloc_scratch` is only a handle for the runtime, not a device address: the
// address a kernel can use comes from cudaGetSymbolAddress, once per device.
static float* noalloc_scratch_for_current_device() {
    constexpr int kMaxDevices = 64;
    static float* cached[kMaxDevices] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (cached[dev] == nullptr) {
        float* ptr = nullptr;
        if (cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch) != cudaSuccess) return nullptr;
        cached[dev] = ptr;
    }
    return cached[dev];
}

extern "C" {

int halo_rmsnorm_bwd_noalloc(const void* g, const void* h, const void* w, const float* rstd,
                             const void* dres, void* dx, float* dw_f32, void* dw_bf16,
                             int accumulate, long long rows, int H, void* stream) {
    int L, vpt;
    if (!rms_shape(H, &L, &vpt)) return -1;
    if (H > HALO_NOALLOC_MAX_HIDDEN) {
        fprintf(stderr, "halo_rmsnorm_bwd_noalloc: hidden size %d exceeds the built-in scratch (max %d); "
                        "use halo_rmsnorm_bwd with a caller-provided buffer\n", H, HALO_NOALLOC_MAX_HIDDEN);
        return -3;
    }
    if (rows == 0) return 0;
    float* scratch = noalloc_scratch_for_current_device();
    if (scratch == nullptr) return -4;
    // halo_rmsnorm_bwd never launches more than HALO_NOALLOC_MAX_BLOCKS blocks and each block
    // writes H floats, so blocks * H <= the array's size
    return halo_rmsnorm_bwd(g, h, w, rstd, dres, dx, scratch, dw_f32, dw_bf16, accumulate, rows, H, stream);
}

int halo_rope_table(const int* pos, long long T, int head_dim, float theta, void* table,
                    void* stream) {
    const int half = head_dim / 2;
    const long long n = T * half;
    rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        pos, T, half, theta, (float2*)table);
    return HALO_LAUNCH_CHECK();
}

int halo_qknorm_rope_fwd(const void* qkv, const void* wq, const void* wk, const void* table,
                         void* q_out, void* k_out, float* rstd, long long T, int Hq, int Hkv,
                         int head_dim, float eps, int use_norm, void* stream) {
    if (head_dim != 128) return -1;
    const long long warps = T * (Hq + Hkv);
    qknorm_rope_fwd_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk,
        (const float2*)table, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out, rstd, T, Hq, Hkv, eps,
        use_norm);
    return HALO_LAUNCH_CHECK();
}

int halo_qknorm_rope_bwd_blocks(long long T, int heads) {
    long long b = (T * heads + 7) / 8;
    return (int)(b < 1184 ? b : 1184);
}

// dw_partial: fp32 scratch of halo_qknorm_rope_bwd_blocks(...) * 256; dwq/dwk: fp32 [128] outputs.
int halo_qknorm_rope_bwd(const void* dq, const void* dk, const void* qkv, const void* wq,
                         const void* wk, const void* table, const float* rstd, void* dqkv,
                         float* dw_partial, float* dwq, float* dwk, int accumulate, long long T,
                         int Hq, int Hkv, int head_dim, int use_norm, void* stream) {
    if (head_dim != 128) return -1;
    const int blocks = halo_qknorm_rope_bwd_blocks(T, Hq + Hkv);
    cudaStream_t s = (cudaStream_t)stream;
    qknorm_rope_bwd_kernel<<<blocks, 256, 0, s>>>(
        (const __nv_bfloat16*)dq, (const __nv_bfloat16*)dk, (const __nv_bfloat16*)qkv,
        (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk, (const float2*)table, rstd,
        (__nv_bfloat16*)dqkv, dw_partial, T, Hq, Hkv, use_norm);
    if (use_norm) {
        // partial layout per block: [dwq(128) | dwk(128)]
        reduce_partials_kernel<<<1, 256, 0, s>>>(dw_partial, blocks, 256, dwq, nullptr, accumulate);
        (void)dwk;  // dwq points at a [256] buffer: first 128 = q weight grad, last 128 = k weight grad
    }
    return HALO_LAUNCH_CHECK();
}

int halo_swiglu_fwd(const void* pre, void* act, long long rows, int F, void* stream) {
    if (F % 8) return -1;
    const long long n = rows * (F / 8);
    swiglu_fwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)pre, (__nv_bfloat16*)act, rows, F);
    return HALO_LAUNCH_CHECK();
}

int halo_swiglu_bwd(const void* pre, const void* dact, void* dpre, long long rows, int F,
                    void* stream) {
    if (F % 8) return -1;
    const long long n = rows * (F / 8);
    swiglu_bwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)pre, (const __nv_bfloat16*)dact, (__nv_bfloat16*)dpre, rows, F);
    return HALO_LAUNCH_CHECK();
}

int halo_cross_entropy_inplace(void* logits, const long long* labels, const float* grad_scale,
                               const float* row_scale, float* loss_rows, float* lse, long long rows, long long ld, int V,
                               long long ignore_index, void* stream) {
    if (rows == 0) return 0;
    if (ld % 8) return -1;
    cross_entropy_inplace_kernel<<<(unsigned)rows, 512, 0, (cudaStream_t)stream>>>(
        (__nv_bfloat16*)logits, labels, grad_scale, row_scale, loss_rows, lse, ld, V, ignore_index);
    return HALO_LAUNCH_CHECK();
}

int halo_logprob_entropy(const void* logits, const long long* labels, float* logp, float* entropy,
                         long long rows, long long ld, int V, long long ignore_index, void* stream) {
    if (rows == 0) return 0;
    logprob_entropy_kernel<<<(unsigned)rows, 512, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)logits, labels, logp, entropy, ld, V, ignore_index);
    return HALO_LAUNCH_CHECK();
}

}  // extern "C"
