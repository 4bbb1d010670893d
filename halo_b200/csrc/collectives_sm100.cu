// Collectives fused with their compute, over NVLink peer memory (plain loads / stores through
// pointers into the other GPUs' symmetric buffers; no library collective carries the payload).
//
//   rs_sum_norm     gradient reduce-scatter: every rank sums, in fp32 and in rank order, the
//                   slice of the flat gradient buffer it owns across all peers, keeps the fp32
//                   sum locally and emits per-block partial sums of squares for the global norm
//   adam_allgather  AdamWBF16 on the owned slice (same arithmetic and rounding noise as the
//                   unsharded optimizer kernel) whose epilogue stores the updated bf16 weights
//                   straight into every peer's parameter buffer: the all-gather is the store
//   broadcast_rows  trainer -> rollout weight copy: one read of the local weights, one store per
//                   destination GPU
//   allreduce_small one-shot all-reduce of a small fp32 vector (norm scalars, router gradients)
//
// Every kernel also has an NVLS form for buffers that are bound to an NVLink multicast object (their `mc` argument is
// the multicast address of the same symmetric buffer): reductions read with multimem.ld_reduce, which sums the ranks'
// values inside the switch, and the all-gather / broadcast stores are multimem.st, which the switch replicates to
// every rank, so each byte crosses this GPU's links once whatever the number of peers.
//
// A phase boundary (all peers' gradients written / all slices summed / all weights stored) is a
// device-side barrier issued by the host between the launches; the kernels themselves never spin
// on another GPU.
//
// Together they replace the reduce-scatter -> cast/scale -> AdamWBF16 -> all-gather sequence the
// reference gets from FSDP2 + NCCL + its Triton optimizer (halo/distributed/fsdp.py:319-403,
// halo/optimizers/adamw_bf16.py:99-187), its bucketed all-reduce sweeps
// (halo/distributed/grad_reduce.py:117-181) and its packed NCCL weight broadcast
// (halo/weight_sync/transport/packed_broadcast.py:39-74).
//
// Compiled with -fmad=false so the optimizer arithmetic matches halo_b200/optim/adamw_bf16.py.
#include "sm100_common.cuh"

namespace halo {

constexpr int kMaxPeersC = 16;
struct Peers {
    void* p[kMaxPeersC];
};

// ---- Philox / splitmix, identical to optim.cu ------------------------------------------------
__device__ __forceinline__ void philox_c(uint32_t k0, uint32_t k1, uint32_t c0, uint32_t c1, uint32_t (&o)[4]) {
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
    o[0] = c[0]; o[1] = c[1]; o[2] = c[2]; o[3] = c[3];
}
__device__ __forceinline__ uint64_t splitmix_c(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__device__ __forceinline__ __nv_bfloat16 sr_bf16_c(float x, uint32_t noise16) {
    return __ushort_as_bfloat16((unsigned short)((__float_as_uint(x) + noise16) >> 16));
}

// ---------------------------------------------------------------------------------------------
// phase 1: sum[i] = sum_r grads_r[lo + i]  (fp32, rank order);  partial[b] = sum of squares
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rs_sum_norm_kernel(const __grid_constant__ Peers grads, int n_ranks, long long lo, long long count, float* __restrict__ sum_out,
                   float* __restrict__ partial) {
    __shared__ float red[8];
    float acc = 0.f;
    const long long nvec = count / 8;
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
        float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int r = 0; r < n_ranks; ++r) {
            const uint4 u = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(grads.p[r]) + lo)[v];
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = __bfloat1622float2(h[q]);
                s[2 * q] += f.x;
                s[2 * q + 1] += f.y;
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += s[j] * s[j];
        reinterpret_cast<float4*>(sum_out)[2 * v] = make_float4(s[0], s[1], s[2], s[3]);
        reinterpret_cast<float4*>(sum_out)[2 * v + 1] = make_float4(s[4], s[5], s[6], s[7]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < 8; ++i) t += red[i];
        partial[blockIdx.x] = t;
    }
}

// ---------------------------------------------------------------------------------------------
// phase 2: AdamWBF16 on the owned slice, weights stored to every peer.
// Segments: the pieces of the slice that belong to one tensor each.
//   seg_off[s]   first element of the segment, relative to the slice start (multiple of 8)
//   seg_len[s]   elements in the segment (multiple of 8, tensors are padded in the flat buffer)
//   seg_toff[s]  offset of the segment's first element inside its tensor (multiple of 4)
//   seg_hash[s]  blake2b hash of the tensor's name
//   seg_wd[s]    1 - lr * weight_decay of the tensor's group
// ---------------------------------------------------------------------------------------------
struct SliceTable {
    const long long* seg_off;
    const long long* seg_len;
    const long long* seg_toff;
    const unsigned long long* seg_hash;
    const float* seg_wd;
    const int* block_start;  // [n_seg + 1]
    int n_seg;
};
constexpr int kSliceElemsPerBlock = 256 * 8 * 8;

__global__ void __launch_bounds__(256)
adam_allgather_kernel(const __grid_constant__ Peers params, __nv_bfloat16* mc_params, int n_ranks, int my_rank, long long lo,
                      const float* __restrict__ gsum,
                      __nv_bfloat16* __restrict__ m, __nv_bfloat16* __restrict__ v, SliceTable tab, float beta1,
                      float beta2, float omb1, float omb2, float step_size, float bc2_sqrt, float eps,
                      unsigned long long key_step, const float* __restrict__ grad_scale, const int* __restrict__ skip) {
    if (skip && *skip) return;
    int a = 0, b = tab.n_seg;
    while (b - a > 1) {
        const int mid = (a + b) >> 1;
        if (tab.block_start[mid] <= (int)blockIdx.x) a = mid; else b = mid;
    }
    const int sg = a;
    const long long seg_off = tab.seg_off[sg], seg_len = tab.seg_len[sg], toff = tab.seg_toff[sg];
    const float wd_factor = tab.seg_wd[sg];
    const uint64_t mixed = splitmix_c(splitmix_c(key_step) ^ tab.seg_hash[sg]);
    const uint32_t k0 = (uint32_t)mixed, k1 = (uint32_t)(mixed >> 32);
    const float scale = grad_scale ? *grad_scale : 1.f;
    const long long chunk0 = (long long)(blockIdx.x - tab.block_start[sg]) * kSliceElemsPerBlock;
    const __nv_bfloat16* my_params = reinterpret_cast<const __nv_bfloat16*>(params.p[my_rank]) + lo;
#pragma unroll 1
    for (int it = 0; it < 8; ++it) {
        const long long e = chunk0 + ((long long)it * 256 + threadIdx.x) * 8;   // 8 elements = two noise quads
        if (e >= seg_len) break;
        const long long i = seg_off + e;      // index inside the slice
        const uint4 pu = *reinterpret_cast<const uint4*>(my_params + i);
        const uint4 mu = *reinterpret_cast<const uint4*>(m + i);
        const uint4 vu = *reinterpret_cast<const uint4*>(v + i);
        const float4 g0 = reinterpret_cast<const float4*>(gsum + i)[0];
        const float4 g1 = reinterpret_cast<const float4*>(gsum + i)[1];
        const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const __nv_bfloat162* ph = reinterpret_cast<const __nv_bfloat162*>(&pu);
        const __nv_bfloat162* mh = reinterpret_cast<const __nv_bfloat162*>(&mu);
        const __nv_bfloat162* vh = reinterpret_cast<const __nv_bfloat162*>(&vu);
        float pf[8], mf[8], vf[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float2 t = __bfloat1622float2(ph[q]); pf[2 * q] = t.x; pf[2 * q + 1] = t.y;
            t = __bfloat1622float2(mh[q]); mf[2 * q] = t.x; mf[2 * q + 1] = t.y;
            t = __bfloat1622float2(vh[q]); vf[2 * q] = t.x; vf[2 * q + 1] = t.y;
        }
        uint32_t rnd[8];
        {
            const unsigned long long quad = (unsigned long long)(toff + e) >> 2;
            uint32_t r0[4], r1[4];
            philox_c(k0, k1, (uint32_t)quad, (uint32_t)(quad >> 32), r0);
            philox_c(k0, k1, (uint32_t)(quad + 1), (uint32_t)((quad + 1) >> 32), r1);
#pragma unroll
            for (int j = 0; j < 4; ++j) { rnd[j] = r0[j]; rnd[4 + j] = r1[j]; }
        }
        __nv_bfloat16 po[8], mo[8], vo[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float gj = g[j] * scale;
            const float mn = mf[j] * beta1 + gj * omb1;
            const float vn = vf[j] * beta2 + (gj * gj) * omb2;
            const float denom = sqrtf(vn) / bc2_sqrt + eps;
            const float pn = pf[j] * wd_factor - (step_size * mn) / denom;
            mo[j] = __float2bfloat16_rn(mn);
            vo[j] = sr_bf16_c(vn, rnd[j] >> 16);
            po[j] = sr_bf16_c(pn, rnd[j] & 0xFFFFu);
        }
        *reinterpret_cast<uint4*>(m + i) = *reinterpret_cast<uint4*>(mo);
        *reinterpret_cast<uint4*>(v + i) = *reinterpret_cast<uint4*>(vo);
        const uint4 out = *reinterpret_cast<uint4*>(po);
        if (mc_params) {
            // the all-gather as ONE store: the switch writes it into every rank's parameter buffer
            asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_params + lo + i),
                         "r"(out.x), "r"(out.y), "r"(out.z), "r"(out.w)
                         : "memory");
        } else {
            for (int r = 0; r < n_ranks; ++r)   // the all-gather: one 16-byte store per peer
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + lo + i) = out;
        }
    }
}

// dst_r[i] = src[i] for every destination rank (16-byte vectors; n_bytes multiple of 16)
__global__ void __launch_bounds__(256)
broadcast_bytes_kernel(const uint4* __restrict__ src, const __grid_constant__ Peers dst, int n_dst, long long dst_offset_vec,
                       long long nvec) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
        const uint4 u = src[i];
        for (int r = 0; r < n_dst; ++r) reinterpret_cast<uint4*>(dst.p[r])[dst_offset_vec + i] = u;
    }
}

// All-gather by pulls: dst[r * nvec + i] = shard_r[src_off + i] for every rank r (16-byte vectors; shard_r may be a peer
// GPU's memory). Four loads in flight per thread cover the NVLink round trip. Used to assemble a layer's sharded
// parameters in local memory right before the layer runs.
__global__ void __launch_bounds__(256)
allgather_pull_kernel(uint4* __restrict__ dst, const __grid_constant__ Peers shards, int n_ranks, long long src_off_vec,
                      long long nvec) {
    const long long total = nvec * n_ranks;
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < total; i += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const long long j = i + q * stride;
            const int r = (int)(j / nvec);
            v[q] = reinterpret_cast<const uint4*>(shards.p[r])[src_off_vec + (j - (long long)r * nvec)];
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) dst[i + q * stride] = v[q];
    }
    for (; i < total; i += stride) {
        const int r = (int)(i / nvec);
        dst[i] = reinterpret_cast<const uint4*>(shards.p[r])[src_off_vec + (i - (long long)r * nvec)];
    }
}

// dst[i] = src[i] where src may be another GPU's memory mapped into this process (16-byte vectors, four
// loads in flight per thread to cover the NVLink round trip).
__global__ void __launch_bounds__(256)
peer_pull_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long long nvec) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
        const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
        dst[i] = a; dst[i + stride] = b; dst[i + 2 * stride] = c; dst[i + 3 * stride] = d;
    }
    for (; i < nvec; i += stride) dst[i] = src[i];
}

// dst[i] += src[i] on bf16 pairs (fp32 add, one rounding); src may be a peer's memory.
__global__ void __launch_bounds__(256)
peer_pull_add_bf16_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long long nvec) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const uint4 s = src[i];
        uint4 d = dst[i];
        const __nv_bfloat162* sh = reinterpret_cast<const __nv_bfloat162*>(&s);
        __nv_bfloat162* dh = reinterpret_cast<__nv_bfloat162*>(&d);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 a = __bfloat1622float2(sh[q]), b = __bfloat1622float2(dh[q]);
            dh[q] = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
        }
        dst[i] = d;
    }
}

// out[i] = sum_r bufs_r[i]   (fp32, n small)
__global__ void allreduce_small_kernel(const __grid_constant__ Peers bufs, int n_ranks, float* __restrict__ out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = 0.f;
    for (int r = 0; r < n_ranks; ++r) s += reinterpret_cast<const float*>(bufs.p[r])[i];
    out[i] = s;
}

// ---------------------------------------------------------------------------------------------
// NVLS forms (multimem.* on a multicast address)
// ---------------------------------------------------------------------------------------------
// sum[i] = sum over ranks of grads[lo + i], reduced inside the switch with fp32 accumulation and returned rounded to
// bf16 (what a bf16 all-reduce delivers); partial[b] = sum of squares of the rounded sums.
__global__ void __launch_bounds__(256)
rs_sum_norm_mc_kernel(const __nv_bfloat16* mc_grads, long long lo, long long count, float* __restrict__ sum_out,
                      float* __restrict__ partial) {
    __shared__ float red[8];
    float acc = 0.f;
    const long long nvec = count / 8;
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
        uint32_t a, b, c, d;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
                     : "l"(mc_grads + lo + v * 8)
                     : "memory");
        const uint32_t u[4] = {a, b, c, d};
        float s[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u[q]));
            s[2 * q] = f.x;
            s[2 * q + 1] = f.y;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += s[j] * s[j];
        reinterpret_cast<float4*>(sum_out)[2 * v] = make_float4(s[0], s[1], s[2], s[3]);
        reinterpret_cast<float4*>(sum_out)[2 * v + 1] = make_float4(s[4], s[5], s[6], s[7]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < 8; ++i) t += red[i];
        partial[blockIdx.x] = t;
    }
}

// mc_dst[i] = src[i] on every rank of the multicast group (16-byte vectors)
__global__ void __launch_bounds__(256)
broadcast_bytes_mc_kernel(const uint4* __restrict__ src, uint4* mc_dst, long long nvec) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
        const uint4 u = src[i];
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_dst + i), "r"(u.x), "r"(u.y),
                     "r"(u.z), "r"(u.w)
                     : "memory");
    }
}

// out[i] = sum over ranks of buf[i], one multimem.ld_reduce per element
__global__ void allreduce_small_mc_kernel(const float* mc, float* __restrict__ out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.f32 %0, [%1];" : "=f"(s) : "l"(mc + i) : "memory");
    out[i] = s;
}

static int fill(Peers* o, void* const* host_ptrs, int n) {
    if (n < 1 || n > kMaxPeersC) return -1;
    for (int i = 0; i < kMaxPeersC; ++i) o->p[i] = i < n ? host_ptrs[i] : nullptr;
    return 0;
}

}  // namespace halo

using namespace halo;

extern "C" {

int halo_rs_blocks(long long count) {
    long long b = (count / 8 + 255) / 256;
    return (int)(b < 1184 ? (b < 1 ? 1 : b) : 1184);
}

// grads: host array of n_ranks device pointers to the ranks' flat bf16 gradient buffers.
// Sums elements [lo, lo + count) (lo, count multiples of 8) into sum_out (fp32 [count]);
// partial: fp32 [halo_rs_blocks(count)].
int halo_rs_sum_norm(void* const* grads, int n_ranks, long long lo, long long count, float* sum_out, float* partial,
                     void* stream) {
    if ((lo % 8) || (count % 8)) return -1;
    Peers g;
    if (fill(&g, grads, n_ranks)) return -2;
    const int blocks = halo_rs_blocks(count);
    rs_sum_norm_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(g, n_ranks, lo, count, sum_out, partial);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// NVLS form of halo_rs_sum_norm: mc_grads is the multicast address of the flat bf16 gradient buffer.
int halo_rs_sum_norm_mc(const void* mc_grads, long long lo, long long count, float* sum_out, float* partial, void* stream) {
    if ((lo % 8) || (count % 8) || !mc_grads) return -1;
    const int blocks = halo_rs_blocks(count);
    rs_sum_norm_mc_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)mc_grads, lo, count, sum_out, partial);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// NVLS form of halo_broadcast_bytes: one multimem.st per 16 bytes reaches every rank of the multicast group.
int halo_broadcast_bytes_mc(const void* src, void* mc_dst, long long dst_offset, long long n_bytes, void* stream) {
    if ((n_bytes % 16) || (dst_offset % 16) || (reinterpret_cast<uintptr_t>(src) % 16) || !mc_dst) return -1;
    if (n_bytes == 0) return 0;
    const long long nvec = n_bytes / 16;
    long long blocks = (nvec + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    broadcast_bytes_mc_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
        (const uint4*)src, reinterpret_cast<uint4*>(reinterpret_cast<char*>(mc_dst) + dst_offset), nvec);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// NVLS form of halo_allreduce_small.
int halo_allreduce_small_mc(const void* mc, float* out, int n, void* stream) {
    if (n <= 0) return 0;
    if (!mc) return -1;
    allreduce_small_mc_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>((const float*)mc, out, n);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int halo_slice_elems_per_block() { return kSliceElemsPerBlock; }

// mc_params: the multicast address of the parameter buffer (null: store to every peer in turn)
int halo_adam_allgather(void* const* params, int n_ranks, int my_rank, long long lo, const float* gsum, void* m,
                        void* v, const long long* seg_off, const long long* seg_len, const long long* seg_toff,
                        const unsigned long long* seg_hash, const float* seg_wd, const int* block_start, int n_seg,
                        int total_blocks, float beta1, float beta2, float step_size, float bc2_sqrt, float eps,
                        unsigned long long key, unsigned long long step, const float* grad_scale, const int* skip,
                        void* stream, void* mc_params) {
    if (n_seg <= 0 || total_blocks <= 0) return 0;
    Peers p;
    if (fill(&p, params, n_ranks)) return -2;
    SliceTable t{seg_off, seg_len, seg_toff, seg_hash, seg_wd, block_start, n_seg};
    const float omb1 = (float)(1.0 - (double)beta1), omb2 = (float)(1.0 - (double)beta2);
    adam_allgather_kernel<<<total_blocks, 256, 0, (cudaStream_t)stream>>>(
        p, (__nv_bfloat16*)mc_params, n_ranks, my_rank, lo, gsum, (__nv_bfloat16*)m, (__nv_bfloat16*)v, t, beta1, beta2, omb1, omb2, step_size,
        bc2_sqrt, eps, key ^ step, grad_scale, skip);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Copy n_bytes (multiple of 16) from src to byte offset dst_offset (multiple of 16) of every destination buffer.
int halo_broadcast_bytes(const void* src, void* const* dsts, int n_dst, long long dst_offset, long long n_bytes,
                         void* stream) {
    if ((n_bytes % 16) || (dst_offset % 16) || (reinterpret_cast<uintptr_t>(src) % 16)) return -1;
    if (n_bytes == 0) return 0;
    Peers d;
    if (fill(&d, dsts, n_dst)) return -2;
    const long long nvec = n_bytes / 16;
    long long blocks = (nvec + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    broadcast_bytes_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, d, n_dst,
                                                                             dst_offset / 16, nvec);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// dst: n_ranks * n_bytes_per_rank local bytes; shards[r] + src_offset: rank r's n_bytes_per_rank bytes.
int halo_allgather_pull(void* dst, void* const* shards, int n_ranks, long long src_offset, long long n_bytes_per_rank,
                        void* stream) {
    if ((n_bytes_per_rank % 16) || (src_offset % 16) || (reinterpret_cast<uintptr_t>(dst) % 16)) return -1;
    if (n_bytes_per_rank == 0) return 0;
    Peers p;
    if (fill(&p, shards, n_ranks)) return -2;
    const long long nvec = n_bytes_per_rank / 16;
    long long blocks = (nvec * n_ranks + 1023) / 1024;
    if (blocks > 148 * 4) blocks = 148 * 4;
    if (blocks < 1) blocks = 1;
    allgather_pull_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((uint4*)dst, p, n_ranks, src_offset / 16, nvec);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Copy (accumulate == 0) or bf16-add (accumulate != 0) n_bytes from src, which may be a peer's mapped memory.
int halo_peer_pull(void* dst, const void* src, long long n_bytes, int accumulate, void* stream) {
    if ((n_bytes % 16) || (reinterpret_cast<uintptr_t>(src) % 16) || (reinterpret_cast<uintptr_t>(dst) % 16)) return -1;
    if (n_bytes == 0) return 0;
    const long long nvec = n_bytes / 16;
    long long blocks = (nvec + 1023) / 1024;
    if (blocks > 148 * 4) blocks = 148 * 4;
    if (blocks < 1) blocks = 1;
    if (accumulate)
        peer_pull_add_bf16_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((uint4*)dst, (const uint4*)src, nvec);
    else
        peer_pull_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((uint4*)dst, (const uint4*)src, nvec);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int halo_allreduce_small(void* const* bufs, int n_ranks, float* out, int n, void* stream) {
    if (n <= 0) return 0;
    Peers b;
    if (fill(&b, bufs, n_ranks)) return -2;
    allreduce_small_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(b, n_ranks, out, n);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
