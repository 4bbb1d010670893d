// Mixture-of-experts routing and token movement.
//
//   router_topk          softmax over expert logits + top-k (+ renormalisation), fwd and bwd
//   route_hist/scan/place deterministic counting sort of the [T, k] routing by expert: each
//                        (token, k) slot gets a row in its expert's segment of the receive
//                        buffer of the rank that owns the expert
//   dispatch_rows        pushes every token row to its k destination rows, which may live in a
//                        peer GPU's memory (plain stores through NVLink peer pointers)
//   combine_rows         pulls the k expert outputs of a token back (peer loads), weights them
//                        and sums in fp32 in slot order, so the result is bitwise reproducible
//   scale_rows_dot       backward helper on the expert side: dy = w * dout, dw = <dout, y>
//
// Segments start on multiples of 128 rows so a GEMM tile never straddles two experts; the pad
// rows are zeroed so they contribute nothing to weight gradients.
//
// Replaces DeepEP dispatch/combine plus the reference's Triton sort / permute kernels
// (halo/kernels/moe_route_sort.py:40-125, halo/kernels/moe_permute.py:18-72,
// halo/distributed/expert_parallel/deepep/backends.py:360-393).
#include "sm100_common.cuh"

namespace halo {

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---------------------------------------------------------------------------------------------
// Router: one warp per token, E <= 256 experts (E % 32 == 0), k <= 16.
// Ties go to the lower expert index.
// ---------------------------------------------------------------------------------------------
template <int EPL>  // experts per lane
__global__ void __launch_bounds__(256)
router_topk_fwd_kernel(const float* __restrict__ logits, int* __restrict__ topk_idx,
                       float* __restrict__ topk_w, float* __restrict__ probs_out,
                       const float* __restrict__ sel_bias, long long T, int k, int renorm) {
    const int lane = threadIdx.x & 31;
    const long long t = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (t >= T) return;
    constexpr int E = EPL * 32;
    float p[EPL], b[EPL];   // b: per-expert selection bias (balancing); it ranks experts, it never weighs them
#pragma unroll
    for (int i = 0; i < EPL; ++i) b[i] = sel_bias ? sel_bias[i * 32 + lane] : 0.f;
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        p[i] = logits[t * E + i * 32 + lane];
        m = fmaxf(m, p[i]);
    }
    m = wmax(m);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        p[i] = __expf(p[i] - m);
        s += p[i];
    }
    s = wsum(s);
    const float inv = 1.f / s;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        p[i] *= inv;
        if (probs_out) probs_out[t * E + i * 32 + lane] = p[i];
    }
    float sel_sum = 0.f;
    float my_w = 0.f;
    int my_idx = 0;
    unsigned taken = 0;
    for (int r = 0; r < k; ++r) {
        float best = -INFINITY, best_p = 0.f;
        int best_e = E;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            if (!((taken >> i) & 1u) && p[i] + b[i] > best) {
                best = p[i] + b[i];
                best_p = p[i];
                best_e = i * 32 + lane;
            }
        }
        // warp arg-max, lower index wins ties
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const float op = __shfl_xor_sync(0xffffffffu, best_p, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) {
                best = ob;
                best_p = op;
                best_e = oe;
            }
        }
        if ((best_e & 31) == lane) taken |= 1u << (best_e >> 5);
        if (lane == r) {
            my_w = best_p;
            my_idx = best_e;
        }
        sel_sum += best_p;
    }
    if (lane < k) {
        topk_idx[t * k + lane] = my_idx;
        topk_w[t * k + lane] = renorm ? my_w / sel_sum : my_w;
    }
}

// d logits from d weights: through the renormalisation and the softmax.
template <int EPL>
__global__ void __launch_bounds__(256)
router_topk_bwd_kernel(const float* __restrict__ logits, const int* __restrict__ topk_idx,
                       const float* __restrict__ dw, float* __restrict__ dlogits, long long T, int k,
                       int renorm) {
    const int lane = threadIdx.x & 31;
    const long long t = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (t >= T) return;
    constexpr int E = EPL * 32;
    float p[EPL], dp[EPL];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        p[i] = logits[t * E + i * 32 + lane];
        m = fmaxf(m, p[i]);
        dp[i] = 0.f;
    }
    m = wmax(m);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        p[i] = __expf(p[i] - m);
        s += p[i];
    }
    s = wsum(s);
#pragma unroll
    for (int i = 0; i < EPL; ++i) p[i] /= s;
    // selected probabilities and their incoming gradients
    float sel_sum = 0.f, dot = 0.f;
    for (int r = 0; r < k; ++r) {
        const int e = topk_idx[t * k + r];
        const float g = dw[t * k + r];
        float pe = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i)
            if (i * 32 + lane == e) {
                pe = p[i];
                dp[i] = g;
            }
        pe = wsum(pe);
        sel_sum += pe;
        dot += g * pe;
    }
    if (renorm) {
        // w_j = p_j / S  =>  dL/dp_j = (g_j - sum_i g_i w_i) / S on the selected set
        const float mean = dot / sel_sum;
        for (int r = 0; r < k; ++r) {
            const int e = topk_idx[t * k + r];
#pragma unroll
            for (int i = 0; i < EPL; ++i)
                if (i * 32 + lane == e) dp[i] = (dp[i] - mean) / sel_sum;
        }
    }
    float pd = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) pd += p[i] * dp[i];
    pd = wsum(pd);
#pragma unroll
    for (int i = 0; i < EPL; ++i) dlogits[t * E + i * 32 + lane] = p[i] * (dp[i] - pd);
}

// ---------------------------------------------------------------------------------------------
// Counting sort of routing slots by expert (stable in slot order, no atomics on global memory).
// ---------------------------------------------------------------------------------------------
constexpr int kSlotsPerBlock = 4096;

// block_hist[b][e] = slots of block b routed to expert e
__global__ void __launch_bounds__(256)
route_hist_kernel(const int* __restrict__ topk_idx, long long n_slots, int E,
                  int* __restrict__ block_hist) {
    extern __shared__ int hist[];
    for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    const long long base = (long long)blockIdx.x * kSlotsPerBlock;
    for (int i = threadIdx.x; i < kSlotsPerBlock; i += blockDim.x) {
        const long long s = base + i;
        if (s < n_slots) {
            const int e = topk_idx[s];
            if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) block_hist[(long long)blockIdx.x * E + e] = hist[e];
}

// per expert: exclusive scan over blocks (in place) and the total count
__global__ void route_scan_kernel(int* __restrict__ block_hist, int n_blocks, int E,
                                  int* __restrict__ counts) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    int run = 0;
    for (int b = 0; b < n_blocks; ++b) {
        const int c = block_hist[(long long)b * E + e];
        block_hist[(long long)b * E + e] = run;
        run += c;
    }
    counts[e] = run;
}

// Layout of every rank's receive buffer from the all-gathered counts.
//   counts_all[src][e]: slots rank `src` routes to global expert e.
// Outputs for the calling rank `me`:
//   seg_start[le], seg_rows[le]  its own local experts' segments (start multiple of 128)
//   dst_base[e]                  first row, in the owner's buffer, of this rank's slots for e
//   total_rows[0]                padded rows this rank receives
__global__ void route_layout_kernel(const int* __restrict__ counts_all, int n_ranks, int E, int me,
                                    int* __restrict__ seg_start, int* __restrict__ seg_rows,
                                    int* __restrict__ dst_base, int* __restrict__ total_rows,
                                    int cap_rows, int* __restrict__ status) {
    const int e_loc = E / n_ranks;
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    for (int r = 0; r < n_ranks; ++r) {
        int row = 0;
        for (int le = 0; le < e_loc; ++le) {
            const int e = r * e_loc + le;
            int rows = 0, before_me = 0;
            for (int s = 0; s < n_ranks; ++s) {
                const int c = counts_all[s * E + e];
                if (s < me) before_me += c;
                rows += c;
            }
            dst_base[e] = row + before_me;
            if (r == me) {
                // a segment that would run past the provisioned buffer is truncated (and flagged):
                // its excess slots are dropped by the dispatch kernel's own bound check
                const int s0 = min(row, cap_rows / 128 * 128);
                const int fit = max(0, min(rows, cap_rows / 128 * 128 - s0));
                seg_start[le] = s0;
                seg_rows[le] = fit;
                if (fit != rows && status) atomicCAS(status, kStatusOk, kStatusBounds);
            }
            row += (rows + 127) / 128 * 128;
        }
        if (r == me) total_rows[0] = min(row, cap_rows);
    }
}

// slot_row[s] = destination row of slot s in the owner's buffer; slot order inside an expert is
// slot-index order.
__global__ void __launch_bounds__(1024)
route_place_kernel(const int* __restrict__ topk_idx, long long n_slots, int E,
                   const int* __restrict__ block_hist /* scanned */,
                   const int* __restrict__ dst_base, int* __restrict__ slot_row,
                   const int* __restrict__ my_prefix /* or null */, int* __restrict__ send_slot /* or null */) {
    extern __shared__ int sh[];
    int* base = sh;            // [E] running position of each expert inside this block
    int* warp_cnt = sh + E;    // [32][E]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int e = threadIdx.x; e < E; e += blockDim.x)
        base[e] = dst_base[e] + block_hist[(long long)blockIdx.x * E + e];
    const long long blk0 = (long long)blockIdx.x * kSlotsPerBlock;
    for (int round = 0; round < kSlotsPerBlock / 1024; ++round) {
        for (int i = threadIdx.x; i < 32 * E; i += blockDim.x) warp_cnt[i] = 0;
        __syncthreads();
        const long long s = blk0 + round * 1024 + threadIdx.x;
        int e = -1;
        if (s < n_slots) {
            e = topk_idx[s];
            if (e < 0 || e >= E) e = -1;
        }
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
        if (e >= 0 && rank_in_warp == 0) warp_cnt[warp * E + e] = __popc(peers);
        __syncthreads();
        for (int ee = threadIdx.x; ee < E; ee += blockDim.x) {
            int run = base[ee];
            for (int w = 0; w < 32; ++w) {
                const int c = warp_cnt[w * E + ee];
                warp_cnt[w * E + ee] = run;
                run += c;
            }
            base[ee] = run;
        }
        __syncthreads();
        if (e >= 0) {
            const int row = warp_cnt[warp * E + e] + rank_in_warp;
            slot_row[s] = row;
            // the same slots listed in destination order (expert by expert, rows ascending): what a sender walks
            if (send_slot) send_slot[my_prefix[e] + (row - dst_base[e])] = (int)s;
        } else if (s < n_slots) slot_row[s] = -1;
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// Token movement. `bufs.p[r]` is the base of rank r's buffer ([rows, H] bf16); for the local rank
// it is an ordinary device pointer, for a peer it is that GPU's memory mapped into this process.
// The table travels by value in the kernel parameters, so no device-side table is needed; it is
// declared __grid_constant__ so that indexing it by a run-time rank reads the parameter bank instead
// of first copying the whole table to each thread's stack.
// ---------------------------------------------------------------------------------------------
constexpr int kMaxPeers = 16;
struct PeerPtrs {
    void* p[kMaxPeers];
};
// One block per token: the row is read once and stored k times.
__global__ void __launch_bounds__(256)
dispatch_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ topk_idx,
                     const int* __restrict__ slot_row, const float* __restrict__ slot_w,
                     const __grid_constant__ PeerPtrs bufs, const __grid_constant__ PeerPtrs wbufs, int has_w,
                     long long T, int k, int H, int experts_per_rank, int cap_rows, int* status) {
    const int nvec = H / 8;
    // the grid may be smaller than T (a bounded footprint leaves room on every SM for a GEMM running beside it)
    for (long long t = blockIdx.x; t < T; t += gridDim.x) {
        const uint4* src = reinterpret_cast<const uint4*>(x + t * H);
        for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
            const uint4 val = src[v];
            for (int j = 0; j < k; ++j) {
                const int row = slot_row[t * k + j];
                if (row < 0) continue;
                if (row >= cap_rows) {
                    // the receive buffer was provisioned too small for this routing: never write past it
                    if (v == 0 && status) atomicCAS(status, kStatusOk, kStatusBounds);
                    continue;
                }
                const int r = topk_idx[t * k + j] / experts_per_rank;
                reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(bufs.p[r]) + (long long)row * H)[v] = val;
            }
        }
        if (has_w && threadIdx.x < k) {
            const int j = threadIdx.x;
            const int row = slot_row[t * k + j];
            if (row >= 0 && row < cap_rows)
                reinterpret_cast<float*>(wbufs.p[topk_idx[t * k + j] / experts_per_rank])[row] = slot_w[t * k + j];
        }
    }
}

// Zero the pad rows [seg_start+seg_rows, next multiple of 128) of the local buffer.
__global__ void __launch_bounds__(256)
zero_pad_rows_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ seg_start,
                     const int* __restrict__ seg_rows, int H, int cap_rows) {
    const int le = blockIdx.x;
    const int first = min(seg_start[le] + seg_rows[le], cap_rows);
    const int last = min((first + 127) / 128 * 128, cap_rows);
    const int nvec = H / 8;
    for (int r = first + blockIdx.y; r < last; r += gridDim.y) {
        uint4* dst = reinterpret_cast<uint4*>(buf + (long long)r * H);
        for (int v = threadIdx.x; v < nvec; v += blockDim.x) dst[v] = make_uint4(0, 0, 0, 0);
    }
}

// out[t] = sum_j w[t,j] * bufs[rank(t,j)][row(t,j)]   (+ addend[t]);  w == nullptr means 1.
__global__ void __launch_bounds__(256)
combine_rows_kernel(const __grid_constant__ PeerPtrs bufs, const int* __restrict__ topk_idx,
                    const int* __restrict__ slot_row, const float* __restrict__ w,
                    const __nv_bfloat16* __restrict__ addend, __nv_bfloat16* __restrict__ out,
                    long long T, int k, int H, int experts_per_rank, int cap_rows) {
    const int nvec = H / 8;
    constexpr int kChunk = 8;   // rows fetched together: all loads of a chunk are in flight before any is used
    for (long long t = blockIdx.x; t < T; t += gridDim.x) {
        for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int j0 = 0; j0 < k; j0 += kChunk) {
                uint4 u[kChunk];
                float wj[kChunk];
#pragma unroll
                for (int jj = 0; jj < kChunk; ++jj) {
                    const int j = j0 + jj;
                    u[jj] = make_uint4(0, 0, 0, 0);
                    wj[jj] = 0.f;
                    if (j < k) {
                        const int row = slot_row[t * k + j];
                        if (row >= 0 && row < cap_rows) {
                            const int r = topk_idx[t * k + j] / experts_per_rank;
                            u[jj] = reinterpret_cast<const uint4*>(
                                reinterpret_cast<const __nv_bfloat16*>(bufs.p[r]) + (long long)row * H)[v];
                            wj[jj] = w ? w[t * k + j] : 1.f;
                        }
                    }
                }
#pragma unroll
                for (int jj = 0; jj < kChunk; ++jj) {
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u[jj]);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float2 f = __bfloat1622float2(h[q]);
                        acc[2 * q] += wj[jj] * f.x;
                        acc[2 * q + 1] += wj[jj] * f.y;
                    }
                }
            }
            if (addend) {
                const uint4 ua = reinterpret_cast<const uint4*>(addend + t * H)[v];
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&ua);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = __bfloat1622float2(h[q]);
                    acc[2 * q] += f.x;
                    acc[2 * q + 1] += f.y;
                }
            }
            reinterpret_cast<uint4*>(out + t * H)[v] =
                make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]),
                           pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
        }
    }
}

// Expert side of the combine backward, one warp per row:
//   dwrow[r] = <g[r], y[r]>;   g[r] *= scale[r]   (in place)
__global__ void __launch_bounds__(256)
scale_rows_dot_kernel(__nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ y,
                      const float* __restrict__ scale, float* __restrict__ dwrow,
                      const int* __restrict__ total_rows, int H, int cap_rows) {
    const int lane = threadIdx.x & 31;
    const int rows = min(*total_rows, cap_rows);
    const int nvec = H / 8;
    for (long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); r < rows; r += (long long)gridDim.x * 8) {
        uint4* gr = reinterpret_cast<uint4*>(g + r * H);
        const uint4* yr = reinterpret_cast<const uint4*>(y + r * H);
        const float sc = scale[r];
        float dot = 0.f;
        for (int v = lane; v < nvec; v += 32) {
            uint4 gu = gr[v];
            const uint4 yu = yr[v];
            __nv_bfloat162* gh = reinterpret_cast<__nv_bfloat162*>(&gu);
            const __nv_bfloat162* yh = reinterpret_cast<const __nv_bfloat162*>(&yu);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 a = __bfloat1622float2(gh[q]), b = __bfloat1622float2(yh[q]);
                dot += a.x * b.x + a.y * b.y;
                gh[q] = __floats2bfloat162_rn(a.x * sc, a.y * sc);
            }
            gr[v] = gu;
        }
        dot = wsum(dot);
        if (lane == 0) dwrow[r] = dot;
    }
}

// SwiGLU backward on the expert side with the routing weight folded in. Per row r (one warp each):
//   act      = silu(gate) * up                      (from the saved pre-activations)
//   dwrow[r] = <dact_u[r], act>                      = d loss / d routing weight of the row
//   dpre[r]  = w[r] * swiglu'(pre[r]) (.) dact_u[r]
//   act_w[r] = w[r] * act                            (left operand of the down-projection weight gradient)
// where dact_u = dout_rows W_down is the unscaled activation gradient. <dout, y> = <dout W_down, act>, so
// neither the expert output rows nor a pre-scaled copy of the incoming gradient is needed. dpre may be pre and
// act_w may be dact_u (in place): a thread reads the vectors it overwrites before it writes them.
__global__ void __launch_bounds__(256)
swiglu_bwd_weighted_kernel(const __nv_bfloat16* pre, const __nv_bfloat16* dact,
                           const float* __restrict__ w, __nv_bfloat16* dpre,
                           __nv_bfloat16* act_w, float* __restrict__ dwrow,
                           const int* __restrict__ total_rows, int F, int cap_rows) {
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
                const float sx = sigmoid_fast(g.x), sy = sigmoid_fast(g.y);
                // the forward rounded act to bf16 before the down projection; use the same value here
                const float2 a = __bfloat1622float2(__floats2bfloat162_rn(g.x * sx * u.x, g.y * sy * u.y));
                dot += d.x * a.x + d.y * a.y;
                const float dx = d.x * sc, dy = d.y * sc;
                ouh[q] = __floats2bfloat162_rn(dx * g.x * sx, dy * g.y * sy);
                ogh[q] = __floats2bfloat162_rn(dx * u.x * sx * (1.f + g.x * (1.f - sx)),
                                               dy * u.y * sy * (1.f + g.y * (1.f - sy)));
                oah[q] = __floats2bfloat162_rn(a.x * sc, a.y * sc);
            }
            *reinterpret_cast<uint4*>(dpre + r * 2 * F + v * 8) = og;
            *reinterpret_cast<uint4*>(dpre + r * 2 * F + F + v * 8) = ou;
            *reinterpret_cast<uint4*>(act_w + r * F + v * 8) = oa;
        }
        dot = wsum(dot);
        if (lane == 0) dwrow[r] = dot;
    }
}

// dw[t,j] = dwrow_bufs[rank(t,j)][row(t,j)]
__global__ void gather_slot_values_kernel(const __grid_constant__ PeerPtrs vbufs,
                                          const int* __restrict__ topk_idx,
                                          const int* __restrict__ slot_row, float* __restrict__ out,
                                          long long n_slots, int experts_per_rank, int cap_rows) {
    const long long s = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n_slots) return;
    const int row = slot_row[s];
    out[s] = (row < 0 || row >= cap_rows) ? 0.f : reinterpret_cast<const float*>(vbufs.p[topk_idx[s] / experts_per_rank])[row];
}

// per-expert token counts for load metrics / balancing (no host sync)
__global__ void expert_load_kernel(const int* __restrict__ counts, int E, long long* __restrict__ acc) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e < E) acc[e] += counts[e];
}

}  // namespace halo

using namespace halo;

extern "C" {

#define HALO_LAUNCH_CHECK() (cudaGetLastError() == cudaSuccess ? 0 : -11)

// Blocks of the row-moving kernels: four per SM (half of an SM's thread slots, no shared memory), so that a GEMM
// CTA launched on another stream can become resident beside them. HALO_ROW_BLOCKS_PER_SM overrides (0 = one block per row).
static int g_row_blocks_per_sm = -1;
static unsigned row_grid(long long T) {
    if (g_row_blocks_per_sm < 0) {
        const char* e = getenv("HALO_ROW_BLOCKS_PER_SM");
        g_row_blocks_per_sm = e ? atoi(e) : 4;
    }
    if (g_row_blocks_per_sm == 0) return (unsigned)T;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long cap = (long long)sms * g_row_blocks_per_sm;
    return (unsigned)(T < cap ? T : cap);
}

int halo_router_topk_fwd(const float* logits, int* idx, float* w, float* probs, const float* sel_bias,
                         long long T, int E, int k, int renorm, void* stream) {
    if (E % 32 || E > 256 || k > 16 || k > E) return -1;
    dim3 grid((unsigned)((T + 7) / 8));
    cudaStream_t s = (cudaStream_t)stream;
    switch (E / 32) {
#define RT(V) case V: router_topk_fwd_kernel<V><<<grid, 256, 0, s>>>(logits, idx, w, probs, sel_bias, T, k, renorm); break;
        RT(1) RT(2) RT(3) RT(4) RT(5) RT(6) RT(7) RT(8)
#undef RT
        default: return -2;
    }
    return HALO_LAUNCH_CHECK();
}

int halo_router_topk_bwd(const float* logits, const int* idx, const float* dw, float* dlogits,
                         long long T, int E, int k, int renorm, void* stream) {
    if (E % 32 || E > 256 || k > 16) return -1;
    dim3 grid((unsigned)((T + 7) / 8));
    cudaStream_t s = (cudaStream_t)stream;
    switch (E / 32) {
#define RT(V) case V: router_topk_bwd_kernel<V><<<grid, 256, 0, s>>>(logits, idx, dw, dlogits, T, k, renorm); break;
        RT(1) RT(2) RT(3) RT(4) RT(5) RT(6) RT(7) RT(8)
#undef RT
        default: return -2;
    }
    return HALO_LAUNCH_CHECK();
}

int halo_route_blocks(long long n_slots) { return (int)((n_slots + kSlotsPerBlock - 1) / kSlotsPerBlock); }

// block_hist: int scratch [halo_route_blocks(n_slots) * E]; counts: [E]
int halo_route_count(const int* idx, long long n_slots, int E, int* block_hist, int* counts,
                     void* stream) {
    const int nb = halo_route_blocks(n_slots);
    cudaStream_t s = (cudaStream_t)stream;
    if (nb > 0) route_hist_kernel<<<nb, 256, E * sizeof(int), s>>>(idx, n_slots, E, block_hist);
    route_scan_kernel<<<(E + 127) / 128, 128, 0, s>>>(block_hist, nb, E, counts);
    return HALO_LAUNCH_CHECK();
}

int halo_route_layout(const int* counts_all, int n_ranks, int E, int me, int* seg_start,
                      int* seg_rows, int* dst_base, int* total_rows, int cap_rows, int* status,
                      void* stream) {
    if (E % n_ranks) return -1;
    route_layout_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(counts_all, n_ranks, E, me, seg_start,
                                                           seg_rows, dst_base, total_rows, cap_rows,
                                                           status);
    return HALO_LAUNCH_CHECK();
}

static int route_place_launch(const int* idx, long long n_slots, int E, const int* block_hist, const int* dst_base,
                              int* slot_row, const int* my_prefix, int* send_slot, void* stream) {
    const int nb = halo_route_blocks(n_slots);
    if (nb == 0) return 0;
    const int smem = (E + 32 * E) * sizeof(int);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        if (cudaFuncSetAttribute(route_place_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem) != cudaSuccess)
            return -10;
        configured = true;
    }
    route_place_kernel<<<nb, 1024, smem, (cudaStream_t)stream>>>(idx, n_slots, E, block_hist, dst_base,
                                                                slot_row, my_prefix, send_slot);
    return HALO_LAUNCH_CHECK();
}

int halo_route_place(const int* idx, long long n_slots, int E, const int* block_hist,
                     const int* dst_base, int* slot_row, void* stream) {
    return route_place_launch(idx, n_slots, E, block_hist, dst_base, slot_row, nullptr, nullptr, stream);
}

// As halo_route_place, and also send_slot[p] = the slot that sits at position p of this rank's destination-ordered
// send list (my_prefix[e] = first position of expert e's slots in that list).
int halo_route_place_send(const int* idx, long long n_slots, int E, const int* block_hist, const int* dst_base,
                          int* slot_row, const int* my_prefix, int* send_slot, void* stream) {
    return route_place_launch(idx, n_slots, E, block_hist, dst_base, slot_row, my_prefix, send_slot, stream);
}

static int fill_peers(PeerPtrs* out, void* const* host_ptrs, int n) {
    if (n < 1 || n > kMaxPeers) return -1;
    for (int i = 0; i < kMaxPeers; ++i) out->p[i] = i < n ? host_ptrs[i] : nullptr;
    return 0;
}

// bufs / wbufs: HOST arrays of n_ranks device pointers (rank r's row buffer / per-row float buffer)
int halo_dispatch_rows(const void* x, const int* idx, const int* slot_row, const float* slot_w,
                       void* const* bufs, void* const* wbufs, int n_ranks, long long T, int k, int H,
                       int experts_per_rank, int cap_rows, int* status, void* stream) {
    if (H % 8) return -1;
    if (T == 0) return 0;
    PeerPtrs pb, pw;
    if (fill_peers(&pb, bufs, n_ranks)) return -2;
    if (wbufs) { if (fill_peers(&pw, wbufs, n_ranks)) return -2; } else { for (int i = 0; i < kMaxPeers; ++i) pw.p[i] = nullptr; }
    dispatch_rows_kernel<<<row_grid(T), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, idx, slot_row, slot_w, pb, pw, wbufs ? 1 : 0, T, k, H,
        experts_per_rank, cap_rows, status);
    return HALO_LAUNCH_CHECK();
}

int halo_zero_pad_rows(void* buf, const int* seg_start, const int* seg_rows, int n_local, int H,
                       int cap_rows, void* stream) {
    if (n_local == 0) return 0;
    zero_pad_rows_kernel<<<dim3(n_local, 16), 256, 0, (cudaStream_t)stream>>>(
        (__nv_bfloat16*)buf, seg_start, seg_rows, H, cap_rows);
    return HALO_LAUNCH_CHECK();
}

int halo_combine_rows(void* const* bufs, int n_ranks, const int* idx, const int* slot_row, const float* w,
                      const void* addend, void* out, long long T, int k, int H, int experts_per_rank,
                      int cap_rows, void* stream) {
    if (H % 8) return -1;
    if (T == 0) return 0;
    PeerPtrs pb;
    if (fill_peers(&pb, bufs, n_ranks)) return -2;
    combine_rows_kernel<<<row_grid(T), 256, 0, (cudaStream_t)stream>>>(
        pb, idx, slot_row, w, (const __nv_bfloat16*)addend,
        (__nv_bfloat16*)out, T, k, H, experts_per_rank, cap_rows);
    return HALO_LAUNCH_CHECK();
}

int halo_scale_rows_dot(void* g, const void* y, const float* scale, float* dwrow,
                        const int* total_rows, int H, int cap_rows, void* stream) {
    scale_rows_dot_kernel<<<1184, 256, 0, (cudaStream_t)stream>>>(
        (__nv_bfloat16*)g, (const __nv_bfloat16*)y, scale, dwrow, total_rows, H, cap_rows);
    return HALO_LAUNCH_CHECK();
}

int halo_swiglu_bwd_weighted(const void* pre, const void* dact, const float* w, void* dpre, void* act_w, float* dwrow,
                             const int* total_rows, int F, int cap_rows, void* stream) {
    if (F % 8) return -1;
    swiglu_bwd_weighted_kernel<<<2368, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)pre, (const __nv_bfloat16*)dact, w, (__nv_bfloat16*)dpre, (__nv_bfloat16*)act_w, dwrow,
        total_rows, F, cap_rows);
    return HALO_LAUNCH_CHECK();
}

int halo_gather_slot_values(void* const* vbufs, int n_ranks, const int* idx, const int* slot_row, float* out,
                            long long n_slots, int experts_per_rank, int cap_rows, void* stream) {
    if (n_slots == 0) return 0;
    PeerPtrs pv;
    if (fill_peers(&pv, vbufs, n_ranks)) return -2;
    gather_slot_values_kernel<<<(unsigned)((n_slots + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        pv, idx, slot_row, out, n_slots, experts_per_rank, cap_rows);
    return HALO_LAUNCH_CHECK();
}

int halo_expert_load_add(const int* counts, int E, long long* acc, void* stream) {
    expert_load_kernel<<<(E + 127) / 128, 128, 0, (cudaStream_t)stream>>>(counts, E, acc);
    return HALO_LAUNCH_CHECK();
}

}  // extern "C"
