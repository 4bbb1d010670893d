// Residual-stream kernels of the hyper-connected and gated-residual decoder families: the collapse / mix / inject
// of N parallel residual streams [T, N, H], the Sinkhorn-Knopp projection of the [T, N, N] mixing matrices, the
// per-stream RMSNorm with (1 + w) scaling and the sigmoid-gated stream mean. All of it is memory-bound: every
// kernel reads each stream element once with 16-byte accesses, computes in fp32 and rounds once at the store.
//
// Work split: one warp owns one token (or one norm group). Its lanes walk the hidden dimension in 8-element
// vectors, so the per-token reductions (the gradients of the [T, N] and [T, N, N] weights) are warp shuffles with
// a fixed order - no atomics, runs are repeatable. N is a template parameter (1..8): the per-token weights sit in
// registers.
//
// Behavioural counterparts: halo/kernels/hyper_connection.py:60-630 and halo/kernels/gated_residual.py:30-200.
#include "sm100_common.cuh"

namespace halo {
namespace streams {

constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ void unpack(const uint4& u, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}
__device__ __forceinline__ float dot8(const float (&a)[8], const float (&b)[8]) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) s += a[j] * b[j];
    return s;
}
// token of this warp, or -1 past the end (no block-wide barrier follows, so such a warp may leave)
__device__ __forceinline__ long long warp_token(long long T) {
    const long long t = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    return t < T ? t : -1;
}

// ---- collapse: out[t, h] = sum_n w[t, n] * x[t, n, h] -----------------------------------------------------------
template <int N>
__global__ void __launch_bounds__(256) collapse_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                                           __nv_bfloat16* __restrict__ out, long long T, int H) {
    const long long t = warp_token(T);
    if (t < 0) return;
    const int lane = threadIdx.x & 31, V = H / 8;
    float wn[N];
#pragma unroll
    for (int n = 0; n < N; ++n) wn[n] = w[t * N + n];
    const uint4* xr = reinterpret_cast<const uint4*>(x + t * N * (long long)H);
    uint4* orow = reinterpret_cast<uint4*>(out + t * (long long)H);
    for (int v = lane; v < V; v += 32) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int n = 0; n < N; ++n) {
            float f[8];
            unpack(xr[n * V + v], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += wn[n] * f[j];
        }
        orow[v] = pack(acc);
    }
}

// dx[t, n, h] = w[t, n] * g[t, h];  dw[t, n] = sum_h g[t, h] * x[t, n, h]
template <int N>
__global__ void __launch_bounds__(256) collapse_bwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ x,
                                                           const float* __restrict__ w, __nv_bfloat16* __restrict__ dx,
                                                           float* __restrict__ dw, long long T, int H) {
    const long long t = warp_token(T);
    if (t < 0) return;
    const int lane = threadIdx.x & 31, V = H / 8;
    float wn[N], dwn[N];
#pragma unroll
    for (int n = 0; n < N; ++n) {
        wn[n] = w[t * N + n];
        dwn[n] = 0.f;
    }
    const uint4* gr = reinterpret_cast<const uint4*>(g + t * (long long)H);
    const uint4* xr = reinterpret_cast<const uint4*>(x + t * N * (long long)H);
    uint4* dxr = reinterpret_cast<uint4*>(dx + t * N * (long long)H);
    for (int v = lane; v < V; v += 32) {
        float gf[8];
        unpack(gr[v], gf);
#pragma unroll
        for (int n = 0; n < N; ++n) {
            float f[8], o[8];
            unpack(xr[n * V + v], f);
            dwn[n] += dot8(gf, f);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = wn[n] * gf[j];
            dxr[n * V + v] = pack(o);
        }
    }
#pragma unroll
    for (int n = 0; n < N; ++n) {
        const float s = wsum(dwn[n]);
        if (lane == 0) dw[t * N + n] = s;
    }
}

// ---- mix: out[t, m, h] = post[t, m] * block[t, h] + sum_n comb[t, n, m] * res[t, n, h] -----------------------------
template <int N>
__global__ void __launch_bounds__(256) mix_fwd_kernel(const __nv_bfloat16* __restrict__ block, const __nv_bfloat16* __restrict__ res,
                                                      const float* __restrict__ post, const float* __restrict__ comb,
                                                      __nv_bfloat16* __restrict__ out, long long T, int H) {
    __shared__ float s_comb[kWarpsPerBlock][N * N];
    __shared__ float s_post[kWarpsPerBlock][N];
    const long long t = warp_token(T);
    if (t < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, V = H / 8;
    for (int i = lane; i < N * N; i += 32) s_comb[warp][i] = comb[t * N * N + i];
    if (lane < N) s_post[warp][lane] = post[t * N + lane];
    __syncwarp();
    const uint4* br = reinterpret_cast<const uint4*>(block + t * (long long)H);
    const uint4* rr = reinterpret_cast<const uint4*>(res + t * N * (long long)H);
    uint4* orow = reinterpret_cast<uint4*>(out + t * N * (long long)H);
    for (int v = lane; v < V; v += 32) {
        float bf[8], rf[N][8];
        unpack(br[v], bf);
#pragma unroll
        for (int n = 0; n < N; ++n) unpack(rr[n * V + v], rf[n]);
#pragma unroll
        for (int m = 0; m < N; ++m) {
            float o[8];
            const float pm = s_post[warp][m];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = pm * bf[j];
#pragma unroll
            for (int n = 0; n < N; ++n) {
                const float c = s_comb[warp][n * N + m];
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] += c * rf[n][j];
            }
            orow[m * V + v] = pack(o);
        }
    }
}

// dblock[t, h] = sum_m post[m] g[m, h];  dpost[t, m] = sum_h block[h] g[m, h];
// dres[t, n, h] = sum_m comb[n, m] g[m, h];  dcomb[t, n, m] = sum_h res[n, h] g[m, h]
template <int N>
__global__ void __launch_bounds__(256) mix_bwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ block,
                                                      const __nv_bfloat16* __restrict__ res, const float* __restrict__ post,
                                                      const float* __restrict__ comb, __nv_bfloat16* __restrict__ dblock,
                                                      __nv_bfloat16* __restrict__ dres, float* __restrict__ dpost,
                                                      float* __restrict__ dcomb, long long T, int H) {
    __shared__ float s_comb[kWarpsPerBlock][N * N];
    __shared__ float s_post[kWarpsPerBlock][N];
    const long long t = warp_token(T);
    if (t < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, V = H / 8;
    for (int i = lane; i < N * N; i += 32) s_comb[warp][i] = comb[t * N * N + i];
    if (lane < N) s_post[warp][lane] = post[t * N + lane];
    __syncwarp();
    float dp[N], dc[N * N];
#pragma unroll
    for (int m = 0; m < N; ++m) dp[m] = 0.f;
#pragma unroll
    for (int i = 0; i < N * N; ++i) dc[i] = 0.f;
    const uint4* gr = reinterpret_cast<const uint4*>(g + t * N * (long long)H);
    const uint4* br = reinterpret_cast<const uint4*>(block + t * (long long)H);
    const uint4* rr = reinterpret_cast<const uint4*>(res + t * N * (long long)H);
    uint4* dbr = reinterpret_cast<uint4*>(dblock + t * (long long)H);
    uint4* drr = reinterpret_cast<uint4*>(dres + t * N * (long long)H);
    for (int v = lane; v < V; v += 32) {
        float gf[N][8], bf[8], db[8];
#pragma unroll
        for (int m = 0; m < N; ++m) unpack(gr[m * V + v], gf[m]);
        unpack(br[v], bf);
#pragma unroll
        for (int j = 0; j < 8; ++j) db[j] = 0.f;
#pragma unroll
        for (int m = 0; m < N; ++m) {
            const float pm = s_post[warp][m];
#pragma unroll
            for (int j = 0; j < 8; ++j) db[j] += pm * gf[m][j];
            dp[m] += dot8(bf, gf[m]);
        }
        dbr[v] = pack(db);
#pragma unroll
        for (int n = 0; n < N; ++n) {
            float rf[8], dr[8];
            unpack(rr[n * V + v], rf);
#pragma unroll
            for (int j = 0; j < 8; ++j) dr[j] = 0.f;
#pragma unroll
            for (int m = 0; m < N; ++m) {
                const float c = s_comb[warp][n * N + m];
#pragma unroll
                for (int j = 0; j < 8; ++j) dr[j] += c * gf[m][j];
                dc[n * N + m] += dot8(rf, gf[m]);
            }
            drr[n * V + v] = pack(dr);
        }
    }
#pragma unroll
    for (int m = 0; m < N; ++m) {
        const float s = wsum(dp[m]);
        if (lane == 0) dpost[t * N + m] = s;
    }
#pragma unroll
    for (int i = 0; i < N * N; ++i) {
        const float s = wsum(dc[i]);
        if (lane == 0) dcomb[t * N * N + i] = s;
    }
}

// ---- inject: out[t, n, h] = res[t, n, h] + gate[t, n] * block[t, h] ------------------------------------------------
template <int N>
__global__ void __launch_bounds__(256) inject_fwd_kernel(const __nv_bfloat16* __restrict__ block, const __nv_bfloat16* __restrict__ res,
                                                         const float* __restrict__ gate, __nv_bfloat16* __restrict__ out,
                                                         long long T, int H) {
    const long long t = warp_token(T);
    if (t < 0) return;
    const int lane = threadIdx.x & 31, V = H / 8;
    float gn[N];
#pragma unroll
    for (int n = 0; n < N; ++n) gn[n] = gate[t * N + n];
    const uint4* br = reinterpret_cast<const uint4*>(block + t * (long long)H);
    const uint4* rr = reinterpret_cast<const uint4*>(res + t * N * (long long)H);
    uint4* orow = reinterpret_cast<uint4*>(out + t * N * (long long)H);
    for (int v = lane; v < V; v += 32) {
        float bf[8];
        unpack(br[v], bf);
#pragma unroll
        for (int n = 0; n < N; ++n) {
            float rf[8], o[8];
            unpack(rr[n * V + v], rf);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = rf[j] + gn[n] * bf[j];
            orow[n * V + v] = pack(o);
        }
    }
}

// dblock[t, h] = sum_n gate[n] g[n, h];  dgate[t, n] = sum_h block[h] g[n, h]   (dres is g itself)
template <int N>
__global__ void __launch_bounds__(256) inject_bwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ block,
                                                         const float* __restrict__ gate, __nv_bfloat16* __restrict__ dblock,
                                                         float* __restrict__ dgate, long long T, int H) {
    const long long t = warp_token(T);
    if (t < 0) return;
    const int lane = threadIdx.x & 31, V = H / 8;
    float gn[N], dg[N];
#pragma unroll
    for (int n = 0; n < N; ++n) {
        gn[n] = gate[t * N + n];
        dg[n] = 0.f;
    }
    const uint4* gr = reinterpret_cast<const uint4*>(g + t * N * (long long)H);
    const uint4* br = reinterpret_cast<const uint4*>(block + t * (long long)H);
    uint4* dbr = reinterpret_cast<uint4*>(dblock + t * (long long)H);
    for (int v = lane; v < V; v += 32) {
        float bf[8], db[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        unpack(br[v], bf);
#pragma unroll
        for (int n = 0; n < N; ++n) {
            float gf[8];
            unpack(gr[n * V + v], gf);
            dg[n] += dot8(bf, gf);
#pragma unroll
            for (int j = 0; j < 8; ++j) db[j] += gn[n] * gf[j];
        }
        dbr[v] = pack(db);
    }
#pragma unroll
    for (int n = 0; n < N; ++n) {
        const float s = wsum(dg[n]);
        if (lane == 0) dgate[t * N + n] = s;
    }
}

// ---- Sinkhorn-Knopp on [T, N, N] fp32: columns, then (rows, columns) x loops; one thread per token ------------------
// scales: [T, 2 * loops + 1, N] (the divisor of every step, kept for the reverse pass) or null.
template <int N>
__global__ void sinkhorn_fwd_kernel(const float* __restrict__ comb, float* __restrict__ out, float* __restrict__ scales,
                                    long long T, int loops, float eps) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const int steps = 2 * loops + 1;
    float m[N * N];
#pragma unroll
    for (int i = 0; i < N * N; ++i) m[i] = comb[t * N * N + i];
    float* sc = scales ? scales + t * steps * N : nullptr;
    auto columns = [&](int step) {
#pragma unroll
        for (int j = 0; j < N; ++j) {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < N; ++i) s += m[i * N + j];
            s += eps;
            if (sc) sc[step * N + j] = s;
#pragma unroll
            for (int i = 0; i < N; ++i) m[i * N + j] /= s;
        }
    };
    auto rows = [&](int step) {
#pragma unroll
        for (int i = 0; i < N; ++i) {
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < N; ++j) s += m[i * N + j];
            s += eps;
            if (sc) sc[step * N + i] = s;
#pragma unroll
            for (int j = 0; j < N; ++j) m[i * N + j] /= s;
        }
    };
    columns(0);
    for (int l = 0; l < loops; ++l) {
        rows(2 * l + 1);
        columns(2 * l + 2);
    }
#pragma unroll
    for (int i = 0; i < N * N; ++i) out[t * N * N + i] = m[i];
}

// Reverse of y = x / s, s = sum(x, axis) + eps:  dx = (dy - sum(dy * y, axis)) / s  and  x = y * s.
template <int N>
__global__ void sinkhorn_bwd_kernel(const float* __restrict__ grad, const float* __restrict__ out, const float* __restrict__ scales,
                                    float* __restrict__ dcomb, long long T, int loops) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const int steps = 2 * loops + 1;
    float y[N * N], g[N * N];
#pragma unroll
    for (int i = 0; i < N * N; ++i) {
        y[i] = out[t * N * N + i];
        g[i] = grad[t * N * N + i];
    }
    const float* sc = scales + t * steps * N;
    auto columns = [&](int step) {
#pragma unroll
        for (int j = 0; j < N; ++j) {
            const float s = sc[step * N + j];
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < N; ++i) d += g[i * N + j] * y[i * N + j];
#pragma unroll
            for (int i = 0; i < N; ++i) {
                g[i * N + j] = (g[i * N + j] - d) / s;
                y[i * N + j] *= s;
            }
        }
    };
    auto rows = [&](int step) {
#pragma unroll
        for (int i = 0; i < N; ++i) {
            const float s = sc[step * N + i];
            float d = 0.f;
#pragma unroll
            for (int j = 0; j < N; ++j) d += g[i * N + j] * y[i * N + j];
#pragma unroll
            for (int j = 0; j < N; ++j) {
                g[i * N + j] = (g[i * N + j] - d) / s;
                y[i * N + j] *= s;
            }
        }
    };
    for (int l = 0; l < loops; ++l) {
        const int step = steps - 1 - 2 * l;
        columns(step);
        rows(step - 1);
    }
    columns(0);
#pragma unroll
    for (int i = 0; i < N * N; ++i) dcomb[t * N * N + i] = g[i];
}

// ---- per-stream RMSNorm with (1 + w): y = x * rsqrt(mean_group(x^2) + eps) * (1 + w) ------------------------------
// x: [rows, S * H]; w: [S * H] fp32; one warp per (row, stream) group of H features; rstd: [rows * S].
__global__ void __launch_bounds__(256) grouped_rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                                                  __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                                                  long long groups, int S, int H, float eps) {
    const long long gi = warp_token(groups);
    if (gi < 0) return;
    const int lane = threadIdx.x & 31, V = H / 8;
    const int s = (int)(gi % S);
    const uint4* xr = reinterpret_cast<const uint4*>(x + gi * (long long)H);
    const float4* wr = reinterpret_cast<const float4*>(w + (long long)s * H);
    uint4* yr = reinterpret_cast<uint4*>(y + gi * (long long)H);
    float ss = 0.f;
    for (int v = lane; v < V; v += 32) {
        float f[8];
        unpack(xr[v], f);
        ss += dot8(f, f);
    }
    ss = wsum(ss);
    const float r = rsqrtf(ss / (float)H + eps);
    if (lane == 0) rstd[gi] = r;
    for (int v = lane; v < V; v += 32) {
        float f[8], o[8];
        unpack(xr[v], f);
        const float4 w0 = wr[2 * v], w1 = wr[2 * v + 1];
        const float wf[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = f[j] * r * (1.f + wf[j]);
        yr[v] = pack(o);
    }
}

// dx = r * (dy * (1 + w)) - x * r^3 * mean(dy * (1 + w) * x)
__global__ void __launch_bounds__(256) grouped_rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                                  const float* __restrict__ w, const float* __restrict__ rstd,
                                                                  __nv_bfloat16* __restrict__ dx, long long groups, int S, int H) {
    const long long gi = warp_token(groups);
    if (gi < 0) return;
    const int lane = threadIdx.x & 31, V = H / 8;
    const int s = (int)(gi % S);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + gi * (long long)H);
    const uint4* xr = reinterpret_cast<const uint4*>(x + gi * (long long)H);
    const float4* wr = reinterpret_cast<const float4*>(w + (long long)s * H);
    uint4* dxr = reinterpret_cast<uint4*>(dx + gi * (long long)H);
    const float r = rstd[gi];
    float dot = 0.f;
    for (int v = lane; v < V; v += 32) {
        float gf[8], f[8];
        unpack(gr[v], gf);
        unpack(xr[v], f);
        const float4 w0 = wr[2 * v], w1 = wr[2 * v + 1];
        const float wf[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) dot += gf[j] * (1.f + wf[j]) * f[j];
    }
    dot = wsum(dot);
    const float c = r * r * r * dot / (float)H;
    for (int v = lane; v < V; v += 32) {
        float gf[8], f[8], o[8];
        unpack(gr[v], gf);
        unpack(xr[v], f);
        const float4 w0 = wr[2 * v], w1 = wr[2 * v + 1];
        const float wf[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r * gf[j] * (1.f + wf[j]) - f[j] * c;
        dxr[v] = pack(o);
    }
}

// Column sums of dy * x * rstd over rows (the norm weight's gradient), two stages, fixed order.
// Stage 1: block (cx, slab) sums rows slab, slab + n_slabs, ... of 256 columns into partial[slab, col].
__global__ void __launch_bounds__(256) norm_weight_grad_partial_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                                      const float* __restrict__ rstd, float* __restrict__ partial,
                                                                      long long rows, int S, int H, int n_slabs) {
    __shared__ float s_acc[kWarpsPerBlock][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int W = S * H;
    const int col = blockIdx.x * 256 + lane * 8;
    const int slab = blockIdx.y;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (col < W) {
        const int s = col / H;          // a vector of 8 never straddles streams: H is a multiple of 8
        for (long long r = (long long)slab * kWarpsPerBlock + warp; r < rows; r += (long long)n_slabs * kWarpsPerBlock) {
            float gf[8], f[8];
            unpack(*reinterpret_cast<const uint4*>(dy + r * W + col), gf);
            unpack(*reinterpret_cast<const uint4*>(x + r * W + col), f);
            const float rs = rstd[r * S + s];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += gf[j] * f[j] * rs;
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s_acc[warp][lane * 8 + j] = acc[j];
    __syncthreads();
    const int c = threadIdx.x;
    float sum = 0.f;
#pragma unroll
    for (int wi = 0; wi < kWarpsPerBlock; ++wi) sum += s_acc[wi][c];
    const int out_col = blockIdx.x * 256 + c;
    if (out_col < W) partial[(long long)slab * W + out_col] = sum;
}

__global__ void norm_weight_grad_final_kernel(const float* __restrict__ partial, float* __restrict__ dw, int W, int n_slabs) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    float s = 0.f;
    for (int i = 0; i < n_slabs; ++i) s += partial[(long long)i * W + c];
    dw[c] = s;
}

// ---- gated stream mean: out[r, h] = bf16(mean_s bf16(bf16(sigmoid(up[r, s, h])) * normed[r, s, h])) ----------------
// (the roundings are those of the elementwise expression evaluated in bf16). One warp per row.
template <int S>
__global__ void __launch_bounds__(256) gate_mix_fwd_kernel(const __nv_bfloat16* __restrict__ up, const __nv_bfloat16* __restrict__ normed,
                                                           __nv_bfloat16* __restrict__ out, long long rows, int H) {
    const long long r = warp_token(rows);
    if (r < 0) return;
    const int lane = threadIdx.x & 31, V = H / 8;
    const uint4* ur = reinterpret_cast<const uint4*>(up + r * S * (long long)H);
    const uint4* nr = reinterpret_cast<const uint4*>(normed + r * S * (long long)H);
    uint4* orow = reinterpret_cast<uint4*>(out + r * (long long)H);
    for (int v = lane; v < V; v += 32) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < S; ++s) {
            float uf[8], nf[8];
            unpack(ur[s * V + v], uf);
            unpack(nr[s * V + v], nf);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float sg = __bfloat162float(__float2bfloat16_rn(1.f / (1.f + __expf(-uf[j]))));
                acc[j] += __bfloat162float(__float2bfloat16_rn(sg * nf[j]));
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] *= (1.f / (float)S);
        orow[v] = pack(acc);
    }
}

// dnormed = (dout / S) * sg;  dup = (dout / S) * normed * sg * (1 - sg)
template <int S>
__global__ void __launch_bounds__(256) gate_mix_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ up,
                                                           const __nv_bfloat16* __restrict__ normed, __nv_bfloat16* __restrict__ dup,
                                                           __nv_bfloat16* __restrict__ dnormed, long long rows, int H) {
    const long long r = warp_token(rows);
    if (r < 0) return;
    const int lane = threadIdx.x & 31, V = H / 8;
    const uint4* gr = reinterpret_cast<const uint4*>(dout + r * (long long)H);
    const uint4* ur = reinterpret_cast<const uint4*>(up + r * S * (long long)H);
    const uint4* nr = reinterpret_cast<const uint4*>(normed + r * S * (long long)H);
    uint4* dur = reinterpret_cast<uint4*>(dup + r * S * (long long)H);
    uint4* dnr = reinterpret_cast<uint4*>(dnormed + r * S * (long long)H);
    for (int v = lane; v < V; v += 32) {
        float gf[8];
        unpack(gr[v], gf);
#pragma unroll
        for (int j = 0; j < 8; ++j) gf[j] *= (1.f / (float)S);
#pragma unroll
        for (int s = 0; s < S; ++s) {
            float uf[8], nf[8], du[8], dn[8];
            unpack(ur[s * V + v], uf);
            unpack(nr[s * V + v], nf);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float sg = 1.f / (1.f + __expf(-uf[j]));
                dn[j] = gf[j] * sg;
                du[j] = gf[j] * nf[j] * sg * (1.f - sg);
            }
            dur[s * V + v] = pack(du);
            dnr[s * V + v] = pack(dn);
        }
    }
}

// ---- sum of squares per row (the RMS of the flattened streams, for the stream projection) ------------------------
__global__ void __launch_bounds__(256) row_rstd_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ rstd, long long rows,
                                                       int W, float eps) {
    const long long r = warp_token(rows);
    if (r < 0) return;
    const int lane = threadIdx.x & 31, V = W / 8;
    const uint4* xr = reinterpret_cast<const uint4*>(x + r * (long long)W);
    float ss = 0.f;
    for (int v = lane; v < V; v += 32) {
        float f[8];
        unpack(xr[v], f);
        ss += dot8(f, f);
    }
    ss = wsum(ss);
    if (lane == 0) rstd[r] = rsqrtf(ss / (float)W + eps);
}

// ---- masked softmax backward (element-wise half of a masked-matmul attention backward) -------------------------
// probs = allowed ? exp(scores * scale - lse) : 0;  d_scores = probs * (upstream - delta) * scale
template <typename OutT>
__device__ __forceinline__ OutT to_out(float v);
template <>
__device__ __forceinline__ float to_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename OutT>
__global__ void masked_softmax_bwd_kernel(const float* __restrict__ scores, const unsigned char* __restrict__ allowed,
                                          const float* __restrict__ lse, const float* __restrict__ upstream,
                                          const float* __restrict__ delta, OutT* __restrict__ probs, OutT* __restrict__ d_scores,
                                          long long n_rows, int n_queries, int n_keys, long long stride_allowed, float scale) {
    const long long total = n_rows * (long long)n_keys;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / n_keys;
        const int key = (int)(i - row * n_keys);
        const bool ok = allowed[(row % n_queries) * stride_allowed + key] != 0;
        const float p = ok ? __expf(scores[i] * scale - lse[row]) : 0.f;
        if (probs) probs[i] = to_out<OutT>(p);
        if (d_scores) d_scores[i] = to_out<OutT>(p * (upstream[i] - delta[row]) * scale);
    }
}

}  // namespace streams
}  // namespace halo

using namespace halo::streams;

extern "C" {

#define STREAMS_CHECK() (cudaGetLastError() == cudaSuccess ? 0 : -11)
#define STREAMS_SWITCH_N(N, CALL)                \
    switch (N) {                                 \
        case 1: { constexpr int kN = 1; CALL; } break; \
        case 2: { constexpr int kN = 2; CALL; } break; \
        case 3: { constexpr int kN = 3; CALL; } break; \
        case 4: { constexpr int kN = 4; CALL; } break; \
        case 5: { constexpr int kN = 5; CALL; } break; \
        case 6: { constexpr int kN = 6; CALL; } break; \
        case 7: { constexpr int kN = 7; CALL; } break; \
        case 8: { constexpr int kN = 8; CALL; } break; \
        default: return -1;                      \
    }

static inline unsigned warp_grid(long long n) { return (unsigned)((n + kWarpsPerBlock - 1) / kWarpsPerBlock); }
static inline bool bad_shape(long long T, int N, int H) { return T < 0 || N < 1 || N > 8 || H <= 0 || (H % 8) != 0; }

int halo_stream_collapse_fwd(const void* x, const float* w, void* out, long long T, int N, int H, void* stream) {
    if (bad_shape(T, N, H)) return -1;
    if (T == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    STREAMS_SWITCH_N(N, (collapse_fwd_kernel<kN><<<warp_grid(T), 256, 0, s>>>((const __nv_bfloat16*)x, w, (__nv_bfloat16*)out, T, H)))
    return STREAMS_CHECK();
}

int halo_stream_collapse_bwd(const void* g, const void* x, const float* w, void* dx, float* dw, long long T, int N, int H,
                             void* stream) {
    if (bad_shape(T, N, H)) return -1;
    if (T == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    STREAMS_SWITCH_N(N, (collapse_bwd_kernel<kN><<<warp_grid(T), 256, 0, s>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)x, w,
                                                                              (__nv_bfloat16*)dx, dw, T, H)))
    return STREAMS_CHECK();
}

int halo_stream_mix_fwd(const void* block, const void* res, const float* post, const float* comb, void* out, long long T,
                        int N, int H, void* stream) {
    if (bad_shape(T, N, H)) return -1;
    if (T == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    STREAMS_SWITCH_N(N, (mix_fwd_kernel<kN><<<warp_grid(T), 256, 0, s>>>((const __nv_bfloat16*)block, (const __nv_bfloat16*)res, post,
                                                                         comb, (__nv_bfloat16*)out, T, H)))
    return STREAMS_CHECK();
}

int halo_stream_mix_bwd(const void* g, const void* block, const void* res, const float* post, const float* comb, void* dblock,
                        void* dres, float* dpost, float* dcomb, long long T, int N, int H, void* stream) {
    if (bad_shape(T, N, H)) return -1;
    if (T == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    STREAMS_SWITCH_N(N, (mix_bwd_kernel<kN><<<warp_grid(T), 256, 0, s>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)block,
                                                                         (const __nv_bfloat16*)res, post, comb, (__nv_bfloat16*)dblock,
                                                                         (__nv_bfloat16*)dres, dpost, dcomb, T, H)))
    return STREAMS_CHECK();
}

int halo_stream_inject_fwd(const void* block, const void* res, const float* gate, void* out, long long T, int N, int H,
                           void* stream) {
    if (bad_shape(T, N, H)) return -1;
    if (T == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    STREAMS_SWITCH_N(N, (inject_fwd_kernel<kN><<<warp_grid(T), 256, 0, s>>>((const __nv_bfloat16*)block, (const __nv_bfloat16*)res, gate,
                                                                            (__nv_bfloat16*)out, T, H)))
    return STREAMS_CHECK();
}

int halo_stream_inject_bwd(const void* g, const void* block, const float* gate, void* dblock, float* dgate, long long T, int N,
                           int H, void* stream) {
    if (bad_shape(T, N, H)) return -1;
    if (T == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    STREAMS_SWITCH_N(N, (inject_bwd_kernel<kN><<<warp_grid(T), 256, 0, s>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)block, gate,
                                                                            (__nv_bfloat16*)dblock, dgate, T, H)))
    return STREAMS_CHECK();
}

// scales may be null (nothing kept for a reverse pass)
int halo_sinkhorn_fwd(const float* comb, float* out, float* scales, long long T, int N, int iters, float eps, void* stream) {
    if (T < 0 || N < 1 || N > 8 || iters < 1) return -1;
    if (T == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned grid = (unsigned)((T + 127) / 128);
    STREAMS_SWITCH_N(N, (sinkhorn_fwd_kernel<kN><<<grid, 128, 0, s>>>(comb, out, scales, T, iters - 1, eps)))
    return STREAMS_CHECK();
}

int halo_sinkhorn_bwd(const float* grad, const float* out, const float* scales, float* dcomb, long long T, int N, int iters,
                      void* stream) {
    if (T < 0 || N < 1 || N > 8 || iters < 1 || scales == nullptr) return -1;
    if (T == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned grid = (unsigned)((T + 127) / 128);
    STREAMS_SWITCH_N(N, (sinkhorn_bwd_kernel<kN><<<grid, 128, 0, s>>>(grad, out, scales, dcomb, T, iters - 1)))
    return STREAMS_CHECK();
}

int halo_grouped_rmsnorm_fwd(const void* x, const float* w, void* y, float* rstd, long long rows, int S, int H, float eps,
                             void* stream) {
    if (rows < 0 || S < 1 || H <= 0 || (H % 8) != 0) return -1;
    if (rows == 0) return 0;
    grouped_rmsnorm_fwd_kernel<<<warp_grid(rows * S), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, w, (__nv_bfloat16*)y, rstd,
                                                                                     rows * S, S, H, eps);
    return STREAMS_CHECK();
}

int halo_grouped_rmsnorm_slabs(long long rows) {
    long long n = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    return (int)(n < 1 ? 1 : (n > 64 ? 64 : n));
}

// partial: fp32 scratch of halo_grouped_rmsnorm_slabs(rows) * S * H elements; dw: [S * H] fp32
int halo_grouped_rmsnorm_bwd(const void* dy, const void* x, const float* w, const float* rstd, void* dx, float* partial,
                             float* dw, long long rows, int S, int H, void* stream) {
    if (rows < 0 || S < 1 || H <= 0 || (H % 8) != 0) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const int W = S * H;
    const int slabs = halo_grouped_rmsnorm_slabs(rows);
    if (rows > 0)
        grouped_rmsnorm_bwd_kernel<<<warp_grid(rows * S), 256, 0, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, w, rstd,
                                                                       (__nv_bfloat16*)dx, rows * S, S, H);
    if (dw != nullptr) {
        dim3 grid((unsigned)((W + 255) / 256), (unsigned)slabs);
        norm_weight_grad_partial_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, rstd, partial, rows, S, H,
                                                             slabs);
        norm_weight_grad_final_kernel<<<(unsigned)((W + 255) / 256), 256, 0, s>>>(partial, dw, W, slabs);
    }
    return STREAMS_CHECK();
}

int halo_gate_mix_fwd(const void* up, const void* normed, void* out, long long rows, int S, int H, void* stream) {
    if (bad_shape(rows, S, H)) return -1;
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    STREAMS_SWITCH_N(S, (gate_mix_fwd_kernel<kN><<<warp_grid(rows), 256, 0, s>>>((const __nv_bfloat16*)up, (const __nv_bfloat16*)normed,
                                                                                 (__nv_bfloat16*)out, rows, H)))
    return STREAMS_CHECK();
}

int halo_gate_mix_bwd(const void* dout, const void* up, const void* normed, void* dup, void* dnormed, long long rows, int S,
                      int H, void* stream) {
    if (bad_shape(rows, S, H)) return -1;
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    STREAMS_SWITCH_N(S, (gate_mix_bwd_kernel<kN><<<warp_grid(rows), 256, 0, s>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)up,
                                                                                 (const __nv_bfloat16*)normed, (__nv_bfloat16*)dup,
                                                                                 (__nv_bfloat16*)dnormed, rows, H)))
    return STREAMS_CHECK();
}

int halo_row_rstd(const void* x, float* rstd, long long rows, int W, float eps, void* stream) {
    if (rows < 0 || W <= 0 || (W % 8) != 0) return -1;
    if (rows == 0) return 0;
    row_rstd_kernel<<<warp_grid(rows), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, rstd, rows, W, eps);
    return STREAMS_CHECK();
}

// out_bf16: 1 = bf16 outputs, 0 = fp32. probs / d_scores may be null (then upstream / delta are not read).
int halo_masked_softmax_bwd(const float* scores, const unsigned char* allowed, const float* lse, const float* upstream,
                            const float* delta, void* probs, void* d_scores, long long n_rows, int n_queries, int n_keys,
                            long long stride_allowed, float scale, int out_bf16, void* stream) {
    if (n_rows < 0 || n_queries < 1 || n_keys < 1) return -1;
    if (d_scores != nullptr && (upstream == nullptr || delta == nullptr)) return -1;
    if (n_rows == 0) return 0;
    const long long total = n_rows * (long long)n_keys;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_bf16)
        masked_softmax_bwd_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>(scores, allowed, lse, upstream, delta,
                                                                                  (__nv_bfloat16*)probs, (__nv_bfloat16*)d_scores, n_rows,
                                                                                  n_queries, n_keys, stride_allowed, scale);
    else
        masked_softmax_bwd_kernel<float><<<(unsigned)blocks, 256, 0, s>>>(scores, allowed, lse, upstream, delta, (float*)probs,
                                                                          (float*)d_scores, n_rows, n_queries, n_keys, stride_allowed, scale);
    return STREAMS_CHECK();
}

}  // extern "C"
