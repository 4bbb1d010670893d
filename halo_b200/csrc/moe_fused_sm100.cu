// Expert-parallel MoE products with the token movement inside the GEMM kernels.
//
//   handshake   every rank publishes its per-expert slot counts into every peer's control block, raises a flag there
//               and waits (bounded) for all peers' flags; the receive layout of every rank follows from the counts.
//               No collective library call: plain stores / acquire loads on peer-mapped memory.
//   kernel A    "dispatch + grouped GEMM": one persistent CTA per SM. Four push warps copy this rank's token rows
//               (in destination order, 128-row units) straight into the owners' expert-grouped receive buffers over
//               NVLink and add the unit's row count to the owner's per-tile arrival counter (release, system scope).
//               The TMA producer of the same kernel issues the loads of an A tile only once its arrival counter is
//               full, tiles being walked in the order their rows arrive, so the tensor cores run under the transfer.
//   kernel B    "grouped GEMM + combine": the epilogue stores every output row straight into the token owner's
//               [tokens x top_k] slot buffer over NVLink (rows are transposed through shared memory so that each
//               store instruction writes whole 256-byte row segments); the owner then sums its k slots locally in
//               fp32 in slot order, which keeps the result bitwise reproducible.
//
// Every wait on a peer is bounded: when it runs out the kernel records kStatusPeerTimeout, raises the CTA's abort
// flag, lets its copies drain, frees its TMEM and returns. TMA loads never use cluster multicast and never read a
// peer's memory: remote rows are first written into this GPU's own buffer by their sender.
//
// Stands where the reference runs DeepEP dispatch -> permute -> grouped_mm -> unpermute -> DeepEP combine
// (halo/distributed/expert_parallel/moe_layer/layer.py:301-342, halo/distributed/expert_parallel/deepep/dispatcher.py:51-245).
#include "gemm_sm100.cuh"

#include <stdio.h>

namespace halo {

int make_tmap_bf16(CUtensorMap* m, const void* base, long long rows, long long cols, long long ld, int box_rows);  // gemm_sm100.cu

constexpr int kEpMaxPeers = 16;
constexpr int kPushWarps = 4;
constexpr int kEpPushThreads = kGemmThreads + kPushWarps * 32 + 32;   // 352: GEMM roles, push warps, one gate warp
constexpr int kMetaSlotBits = 24;                                // row tag = (source rank << 24) | slot index at the source

struct IntPeers { int* p[kEpMaxPeers]; };

// 128-row (or shorter) run of this rank's slots that lands in one tile of one owner's receive buffer
struct PushUnit {
    int pos0;      // first position in send_slot[]
    int n_rows;
    int dst_rank;
    int dst_row0;  // first destination row in the owner's buffer
};

// one 128-row tile of this rank's receive buffer, in the order the tiles' rows arrive
struct EpTile {
    int le;        // local expert
    int tm;        // tile index inside the expert's segment
    int row0;      // first row of the tile in the receive buffer
    int expect;    // real rows of the tile (what its arrival counter reaches)
};

struct EpParams {
    // ---- push side (kernel A) ----
    const __nv_bfloat16* x;       // [T, H] this rank's token rows
    const int* send_slot;         // [T * k] slot ids (t * k + j) in destination order
    const PushUnit* units;
    const int* n_units;
    const float* slot_w;          // [T * k] routing weights travelling with the rows (backward) or null
    void* row_bufs[kEpMaxPeers];  // every rank's receive buffer [cap, H] bf16
    int* meta_bufs[kEpMaxPeers];  // every rank's row tags [cap]
    float* w_bufs[kEpMaxPeers];   // every rank's per-row weights [cap] (backward) or null
    int* arrive_bufs[kEpMaxPeers];  // every rank's arrival counters of this call's parity
    const int* arrive;            // this rank's arrival counters (same memory as arrive_bufs[me])
    int H, k, me;
    // ---- scatter side (kernel B) ----
    void* slot_bufs[kEpMaxPeers];  // every rank's slot buffer [T * k, H] bf16
    const int* meta;               // this rank's row tags [cap]
    unsigned long long wait_budget_ns;
};

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_sys(int* p, int v) {
    asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait until *ctr >= want. On expiry: abort flag, status word, false.
__device__ __forceinline__ bool wait_counter_ge(const int* ctr, int want, volatile int* abort_flag, int* status,
                                                unsigned long long budget_ns) {
    if (ld_acquire_sys(ctr) >= want) return true;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while (true) {
        if (ld_acquire_sys(ctr) >= want) return true;
        __nanosleep(40);
        if ((++spins & 63u) == 0u) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > budget_ns) {
                *abort_flag = 1;
                if (status) atomicCAS(status, kStatusOk, kStatusPeerTimeout);
                return false;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Handshake + receive layout. One block of 256 threads.
//   ctrl layout (ints, the same on every rank): [2][N][E] counts, then [N] flags, then [2][max_tiles] arrival counters
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_handshake_kernel(const __grid_constant__ IntPeers ctrl, int me, int N, int E, int seq, int max_tiles,
                     const int* __restrict__ counts /* [E] or null */, int cap_rows,
                     int* __restrict__ seg_start, int* __restrict__ seg_rows, int* __restrict__ dst_base,
                     int* __restrict__ total_rows, int* __restrict__ my_prefix, int* status,
                     unsigned long long budget_ns) {
    __shared__ int s_rows[256], s_before[256], s_mine[256];
    __shared__ int s_fail;
    const int tid = threadIdx.x;
    const int parity = seq & 1;
    const int off_flags = 2 * N * E;
    const int off_arrive = off_flags + N;
    int* mine = ctrl.p[me];
    if (tid == 0) s_fail = 0;
    // this call's arrival counters start at zero before any peer may add to them
    for (int i = tid; i < max_tiles; i += blockDim.x) mine[off_arrive + parity * max_tiles + i] = 0;
    if (counts) {
        for (int idx = tid; idx < N * E; idx += blockDim.x) {
            const int r = idx / E, e = idx - r * E;
            ctrl.p[r][parity * N * E + me * E + e] = counts[e];
        }
    }
    __syncthreads();
    if (tid < N) {
        __threadfence_system();
        st_release_sys(ctrl.p[tid] + off_flags + me, seq);
        // wait for rank `tid` to have reached the same call
        const int* f = mine + off_flags + tid;
        const uint64_t t0 = global_timer_ns();
        while (ld_acquire_sys(f) < seq) {
            __nanosleep(100);
            if (global_timer_ns() - t0 > budget_ns) {
                if (status) atomicCAS(status, kStatusOk, kStatusPeerTimeout);
                s_fail = 1;
                break;
            }
        }
    }
    __syncthreads();
    if (!counts || s_fail) return;
    // ---- layout from every rank's counts ----
    const int e_loc = E / N;
    const int* call = mine + parity * N * E;
    if (tid < E) {
        int rows = 0, before = 0;
        for (int s = 0; s < N; ++s) {
            const int c = call[s * E + tid];
            if (s < me) before += c;
            rows += c;
        }
        s_rows[tid] = rows;
        s_before[tid] = before;
        s_mine[tid] = counts[tid];
    }
    __syncthreads();
    const int cap_floor = cap_rows / 128 * 128;
    if (tid < E) {
        const int r = tid / e_loc, le = tid - r * e_loc;
        int row = 0;
        for (int j = 0; j < le; ++j) row += (s_rows[r * e_loc + j] + 127) / 128 * 128;
        dst_base[tid] = row + s_before[tid];
        if (r == me) {
            // a segment that would run past the provisioned buffer is truncated (and flagged): senders drop the
            // same rows by the same rule (destination row >= cap_floor)
            const int s0 = min(row, cap_floor);
            const int fit = max(0, min(s_rows[tid], cap_floor - s0));
            seg_start[le] = s0;
            seg_rows[le] = fit;
            if (fit != s_rows[tid] && status) atomicCAS(status, kStatusOk, kStatusBounds);
            if (le == e_loc - 1) total_rows[0] = min(row + (s_rows[tid] + 127) / 128 * 128, cap_rows);
        }
        // position of expert `tid` in this rank's destination-ordered send list: experts are visited starting with
        // this rank's own (local copies give the GEMM its first tiles), then rank me+1's, and so on
        const int first = me * e_loc;
        const int ord = (tid - first + E) % E;
        int pre = 0;
        for (int j = 0; j < ord; ++j) pre += s_mine[(first + j) % E];
        my_prefix[tid] = pre;
    }
}

// Push units of this rank in destination order. One block of 256 threads (E <= 256).
__global__ void __launch_bounds__(256)
moe_plan_push_kernel(const int* __restrict__ counts, const int* __restrict__ dst_base, const int* __restrict__ my_prefix,
                     int me, int N, int E, int cap_rows, PushUnit* __restrict__ units, int* __restrict__ n_units,
                     int max_units) {
    __shared__ int s_n[256], s_base[257];
    const int tid = threadIdx.x;
    const int e_loc = E / N;
    const int cap_floor = cap_rows / 128 * 128;
    int e = 0, a = 0, b = 0;
    if (tid < E) {
        e = (me * e_loc + tid) % E;          // expert visited at position `tid`
        a = min(dst_base[e], cap_floor);
        b = min(dst_base[e] + counts[e], cap_floor);
        s_n[tid] = b > a ? (b - 1) / 128 - a / 128 + 1 : 0;
    }
    __syncthreads();
    if (tid == 0) {
        int acc = 0;
        for (int i = 0; i < E; ++i) {
            s_base[i] = acc;
            acc += s_n[i];
        }
        s_base[E] = acc;
        *n_units = min(acc, max_units);
    }
    __syncthreads();
    if (tid < E && b > a) {
        int u = s_base[tid];
        for (int t = a / 128; t <= (b - 1) / 128; ++t, ++u) {
            if (u >= max_units) break;
            const int lo = max(a, t * 128), hi = min(b, (t + 1) * 128);
            PushUnit pu;
            pu.pos0 = my_prefix[e] + (lo - dst_base[e]);
            pu.n_rows = hi - lo;
            pu.dst_rank = e / e_loc;
            pu.dst_row0 = lo;
            units[u] = pu;
        }
    }
}

// Tiles of this rank's receive buffer in arrival order. Source s reaches this rank at step (me - s) mod N (every
// source starts with its own experts and walks the ranks upwards); a tile is ready at the latest step of the sources
// whose rows it holds. One block of 256 threads (local experts <= 256).
__global__ void __launch_bounds__(256)
moe_plan_tiles_kernel(const __grid_constant__ IntPeers ctrl, int me, int N, int E, int seq,
                      const int* __restrict__ seg_start, const int* __restrict__ seg_rows,
                      EpTile* __restrict__ tiles, int* __restrict__ n_tiles, int max_tiles) {
    extern __shared__ int sh[];          // [N][e_loc] tile counts per (step, local expert), then their bases
    const int tid = threadIdx.x;
    const int e_loc = E / N;
    const int parity = seq & 1;
    const int* call = ctrl.p[me] + parity * N * E;
    for (int i = tid; i < N * e_loc; i += blockDim.x) sh[i] = 0;
    __syncthreads();
    auto tile_step = [&](int e, int lo, int hi) {
        // latest arrival step among the sources with rows in [lo, hi) of expert e's segment
        int off = 0, step = 0;
        for (int s = 0; s < N; ++s) {
            const int c = call[s * E + e];
            if (c > 0 && off < hi && off + c > lo) step = max(step, (me - s + N) % N);
            off += c;
        }
        return step;
    };
    if (tid < e_loc) {
        const int e = me * e_loc + tid;
        const int rows = seg_rows[tid];
        for (int tm = 0; tm * 128 < rows; ++tm) {
            const int st = tile_step(e, tm * 128, min(rows, tm * 128 + 128));
            sh[st * e_loc + tid] += 1;
        }
    }
    __syncthreads();
    if (tid == 0) {
        int acc = 0;
        for (int i = 0; i < N * e_loc; ++i) {
            const int c = sh[i];
            sh[i] = acc;
            acc += c;
        }
        *n_tiles = min(acc, max_tiles);
    }
    __syncthreads();
    if (tid < e_loc) {
        const int e = me * e_loc + tid;
        const int rows = seg_rows[tid];
        for (int tm = 0; tm * 128 < rows; ++tm) {
            const int hi = min(rows, tm * 128 + 128);
            const int st = tile_step(e, tm * 128, hi);
            const int at = sh[st * e_loc + tid]++;
            if (at < max_tiles) {
                EpTile t;
                t.le = tid;
                t.tm = tm;
                t.row0 = seg_start[tid] + tm * 128;
                t.expect = hi - tm * 128;
                tiles[at] = t;
            }
        }
    }
}

// GEMM work items for rows grouped along M, tiles in the given order: C[tile rows] = A[tile rows] * op(B_le).
__global__ void __launch_bounds__(256)
moe_plan_items_kernel(const EpTile* __restrict__ tiles, const int* __restrict__ n_tiles, int n_cols, int k_dim,
                      int b_mn_stride, int b_k_stride, int swiglu_f, int gated, GemmWork* __restrict__ list,
                      int* __restrict__ count, int max_items) {
    const int tile_n = swiglu_f ? 128 : kBlockN;
    const int width = swiglu_f ? swiglu_f : n_cols;
    const int tiles_n = (width + tile_n - 1) / tile_n;
    const int total = min(*n_tiles * tiles_n, max_items);
    if (blockIdx.x == 0 && threadIdx.x == 0) *count = total;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const EpTile t = tiles[i / tiles_n];
        const int tn = i % tiles_n;
        GemmWork w;
        w.a_mn = t.row0;
        w.a_k = 0;
        w.b_k = t.le * b_k_stride;
        w.k_iters = (k_dim + kBlockK - 1) / kBlockK;
        w.c_row = t.row0;
        w.m_valid = kBlockM;          // whole 128-row blocks: the pad rows are zero on input and come out as zeros
        if (swiglu_f) {
            w.b_mn = t.le * b_mn_stride + tn * 128;
            w.b_mn2 = t.le * b_mn_stride + swiglu_f + tn * 128;
            w.c_col = tn * 128;
            w.n_valid = min(128, swiglu_f - tn * 128);
        } else {
            w.b_mn = t.le * b_mn_stride + tn * kBlockN;
            w.b_mn2 = w.b_mn + 128;
            w.c_col = tn * kBlockN;
            w.n_valid = min(kBlockN, n_cols - tn * kBlockN);
        }
        w.pad0 = gated ? t.row0 / 128 + 1 : 0;   // arrival counter of the tile (+1; 0 = no wait)
        w.pad1 = t.expect;
        list[i] = w;
    }
}

// Pad rows [seg_start + seg_rows, next multiple of 128) of the receive buffer: zero data, tag -1, weight 0.
__global__ void __launch_bounds__(256)
moe_zero_pads_kernel(__nv_bfloat16* __restrict__ buf, int* __restrict__ meta, float* __restrict__ roww,
                     const int* __restrict__ seg_start, const int* __restrict__ seg_rows, int H, int cap_rows) {
    const int le = blockIdx.x;
    const int first = min(seg_start[le] + seg_rows[le], cap_rows);
    const int last = min((first + 127) / 128 * 128, cap_rows);
    const int nvec = H / 8;
    for (int r = first + blockIdx.y; r < last; r += gridDim.y) {
        uint4* dst = reinterpret_cast<uint4*>(buf + (long long)r * H);
        for (int v = threadIdx.x; v < nvec; v += blockDim.x) dst[v] = make_uint4(0, 0, 0, 0);
        if (threadIdx.x == 0) {
            if (meta) meta[r] = -1;
            if (roww) roww[r] = 0.f;
        }
    }
}

// out[t] = sum_j w[t, j] * slots[t * k + j]  (w == null: plain sum), fp32 in slot order. Slots whose row was dropped
// (slot_row outside [0, cap_floor)) contribute nothing.
__global__ void __launch_bounds__(256)
moe_slot_sum_kernel(const __nv_bfloat16* __restrict__ slots, const int* __restrict__ slot_row, const float* __restrict__ w,
                    __nv_bfloat16* __restrict__ out, long long T, int k, int H, int cap_floor) {
    const int nvec = H / 8;
    constexpr int kChunk = 8;
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
                        if (row >= 0 && row < cap_floor) {
                            u[jj] = reinterpret_cast<const uint4*>(slots + (t * k + j) * H)[v];
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
            reinterpret_cast<uint4*>(out + t * H)[v] =
                make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]),
                           pack_bf16(acc[6], acc[7]));
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The fused GEMM. A is K-major and grouped along M (the receive buffer or an activation buffer); B is the expert
// bank, K-major or N-major. kPush adds four push warps and gates every A tile on its arrival counter; kScatter
// replaces the epilogue's local store by stores into the token owners' slot buffers.
// ---------------------------------------------------------------------------------------------
template <bool kPush, bool kTwoRows>
__device__ __forceinline__ void push_units(const EpParams& ep, volatile int* abort_flag, int lane, int pw, int ptid) {
    if (!kPush) return;
    const int n_units = *ep.n_units;
    const int nvec = ep.H / 8;
    // no abort check in this loop: pushing never waits on anyone, and the four warps must meet at every unit's barrier
    for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
        const PushUnit pu = ep.units[u];
        __nv_bfloat16* dst_buf = reinterpret_cast<__nv_bfloat16*>(ep.row_bufs[pu.dst_rank]);
        // This warp's rows are pw, pw + 4, ...: at most 32 of a unit's 128. Lane j fetches the routing slot of the warp's
        // j-th row up front, so that no row's copy starts with a dependent index load. kTwoRows: rows go two at a time
        // (sixteen 16-byte loads in flight per lane). Measured on 2 GPUs at the 30B-A3B shapes: two rows at a time shorten
        // the backward's first kernel (2.98 -> 2.73 ms: its GEMM is short, the pushes are the long pole) and lengthen the
        // forward's (3.48 -> 3.93 ms: the pushes then crowd the operand loads of a GEMM that is the long pole), so only
        // the backward instantiation uses them.
        const int n_mine = pu.n_rows > pw ? (pu.n_rows - pw + kPushWarps - 1) / kPushWarps : 0;
        const int my_slot = lane < n_mine ? ep.send_slot[pu.pos0 + pw + lane * kPushWarps] : 0;
        const float my_w = (ep.slot_w && lane < n_mine) ? ep.slot_w[my_slot] : 0.f;
        for (int r = 0; r < n_mine; r += (kTwoRows ? 2 : 1)) {
            const bool two = kTwoRows && r + 1 < n_mine;
            const int slot0 = __shfl_sync(0xffffffffu, my_slot, r);
            const int slot1 = __shfl_sync(0xffffffffu, my_slot, two ? r + 1 : r);
            const int drow0 = pu.dst_row0 + pw + r * kPushWarps;
            const int drow1 = drow0 + kPushWarps;
            const uint4* src0 = reinterpret_cast<const uint4*>(ep.x + (long long)(slot0 / ep.k) * ep.H);
            const uint4* src1 = reinterpret_cast<const uint4*>(ep.x + (long long)(slot1 / ep.k) * ep.H);
            uint4* dst0 = reinterpret_cast<uint4*>(dst_buf + (long long)drow0 * ep.H);
            uint4* dst1 = reinterpret_cast<uint4*>(dst_buf + (long long)drow1 * ep.H);
            for (int v0 = 0; v0 < nvec; v0 += 32 * 8) {
                uint4 a[8], b[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int v = v0 + q * 32 + lane;
                    if (v < nvec) {
                        a[q] = src0[v];
                        if (two) b[q] = src1[v];
                    }
                }
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int v = v0 + q * 32 + lane;
                    if (v < nvec) {
                        dst0[v] = a[q];
                        if (two) dst1[v] = b[q];
                    }
                }
            }
        }
        // row metadata: lane j writes what belongs to the warp's j-th row
        if (lane < n_mine) {
            const int drow = pu.dst_row0 + pw + lane * kPushWarps;
            ep.meta_bufs[pu.dst_rank][drow] = (ep.me << kMetaSlotBits) | my_slot;
            if (ep.slot_w) ep.w_bufs[pu.dst_rank][drow] = my_w;
        }
        // all four push warps have issued their stores of this unit; one thread publishes the rows
        asm volatile("bar.sync 1, %0;" ::"n"(kPushWarps * 32) : "memory");
        if (ptid == 0) {
            __threadfence_system();
            red_add_release_sys(ep.arrive_bufs[pu.dst_rank] + pu.dst_row0 / 128, pu.n_rows);
        }
    }
}

// One epilogue warp's 32 rows x n_valid columns of a finished tile, sent to the token owners. Every lane owns one
// accumulator row: it rounds 128 columns at a time to bf16 into its own 256-byte line of the warp's staging buffer and
// hands that line to the copy engine (cp.async.bulk, shared -> global), which writes it into the owner's slot buffer -
// local or across NVLink - as one 256-byte burst while the warp goes on with the next columns. The lines are 272
// bytes apart so that the 32 lanes' 16-byte stores spread over all banks.
constexpr int kScatterLine = 272;
constexpr int kScatterStageBytesPerWarp = 32 * kScatterLine;   // 8,704

__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void epilogue_scatter(const GemmParams& p, const EpParams& ep, const GemmWork& w,
                                                 uint32_t t_row, int row_in_tile, uint32_t stage) {
    const int lane = threadIdx.x & 31;
    const uint32_t line = stage + lane * kScatterLine;
    int tag = -1;
    if (row_in_tile < w.m_valid) tag = ep.meta[w.c_row + row_in_tile];
    __nv_bfloat16* dst = nullptr;
    if (tag >= 0)
        dst = reinterpret_cast<__nv_bfloat16*>(ep.slot_bufs[tag >> kMetaSlotBits]) +
              (long long)(tag & ((1 << kMetaSlotBits) - 1)) * p.ldc + w.c_col;
#pragma unroll 1
    for (int c0 = 0; c0 < kBlockN; c0 += 128) {
        if (c0 >= w.n_valid) break;                       // uniform across the warp
        tma_store_wait_read<0>();                         // the copy engine has read this lane's previous line
#pragma unroll 1
        for (int cc = 0; cc < 128; cc += 32) {
            uint32_t r[32];
            tmem_ld_32x32(t_row + c0 + cc, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                uint32_t o[4];
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    o[q] = pack_bf16(__uint_as_float(r[j + 2 * q]) * p.alpha, __uint_as_float(r[j + 2 * q + 1]) * p.alpha);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(line + (cc + j) * 2), "r"(o[0]), "r"(o[1]),
                             "r"(o[2]), "r"(o[3])
                             : "memory");
            }
        }
        fence_proxy_async_smem();                         // this lane's line, written by ordinary stores, is read by the copy engine
        const int ncols = min(128, w.n_valid - c0);
        if (dst) bulk_store(dst + c0, line, (uint32_t)ncols * 2u);
        tma_store_commit();
    }
}

template <bool B_MN, bool kPush, bool kScatter>
__global__ void __launch_bounds__(kPush ? kEpPushThreads : kGemmThreads, 1)
gemm_ep_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ GemmParams p, const __grid_constant__ EpParams ep) {
    if (status_poisoned(p.status)) return;
    // Dynamic shared memory only (no static variables in front of it), declared 1024-byte aligned: operand stages, the
    // epilogue's staging lines, then the barriers and two scalars.
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int kEpiRegion = 4 * (kScatter ? kScatterStageBytesPerWarp : kEpiStageBytesPerWarp);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + kStages * kStageBytes + kEpiRegion);
    uint64_t* bar_full = bars;
    uint64_t* bar_empty = bars + kStages;
    uint64_t* bar_tfull = bars + 2 * kStages;
    uint64_t* bar_tempty = bars + 2 * kStages + 2;
    uint32_t& tmem_base_slot = *reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
    volatile int& abort_flag = *reinterpret_cast<volatile int*>(bars + 2 * kStages + 5);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t tiles_base = smem_u32(smem_raw);
    if (tiles_base & 1023u) {      // uniform over the CTA: nobody has touched a barrier or TMEM yet
        if (threadIdx.x == 0 && p.status) atomicCAS(p.status, kStatusOk, kStatusBadArgument);
        return;
    }

    if (threadIdx.x == 0) {
        abort_flag = 0;
        *reinterpret_cast<volatile int*>(bars + 2 * kStages + 6) = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bar_tfull[a]), 1);
            mbar_init(smem_u32(&bar_tempty[a]), 4);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    // Work items are dealt to the CTAs round-robin: the CTAs running together then share a handful of 128-row tiles
    // (their column tiles) and one expert's weights through L2. (Whole column groups per CTA measured slower: 148
    // different row tiles in flight at once spill the freshly pushed rows out of L2.)
    const int n_items = *p.list_count;
    const int total = (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;   // items of this CTA
    auto item_of = [&](int it) { return (int)blockIdx.x + it * (int)gridDim.x; };
    volatile int& ready_items = *reinterpret_cast<volatile int*>(bars + 2 * kStages + 6);   // items whose rows have arrived
    // consumers of tiles whose producer may be waiting for another GPU's rows outlast that wait
    const uint64_t budget = kPush ? ep.wait_budget_ns + HALO_WAIT_BUDGET_NS : HALO_WAIT_BUDGET_NS;

    if (warp == 0) {
        // ---------------- TMA producer, gated on the arrival of each tile's rows ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int seen = 0;    // items known to have their rows (the gate warp counts them in shared memory)
            for (int it = 0; it < total && !abort_flag; ++it) {
                const GemmWork w = p.list[item_of(it)];
                if (kPush && it >= seen) {
                    // the gate warp polls the arrival counters ahead of this thread, so that the round trip to a
                    // counter (and to the other GPUs behind it) never sits between two tiles' loads
                    const uint64_t t0 = global_timer_ns();
                    uint32_t spins = 0;
                    while ((seen = ready_items) <= it) {
                        if ((++spins & 63u) == 0u && (abort_flag || global_timer_ns() - t0 > budget)) break;
                    }
                    if (seen <= it) {
                        if (!abort_flag) {
                            abort_flag = 1;
                            if (p.status) atomicCAS(p.status, kStatusOk, kStatusPeerTimeout);
                        }
                        break;
                    }
                    __threadfence_block();
                    // the rows were written by ordinary stores (some by other GPUs); the loads below go through TMA
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                }
                bool ok = true;
                for (int kb = 0; kb < w.k_iters; ++kb) {
                    if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, &abort_flag, p.status, budget)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full = smem_u32(&bar_full[stage]);
                    const uint32_t sa = tiles_base + stage * kStageBytes;
                    const uint32_t sb = sa + kATileBytes;
                    mbar_expect_tx(full, kStageBytes);
                    tma_load_2d(sa, &tmA, full, w.a_k + kb * kBlockK, w.a_mn);
                    if (B_MN) {
                        tma_load_2d(sb, &tmB, full, w.b_mn, w.b_k + kb * kBlockK);
                        tma_load_2d(sb + 8192, &tmB, full, w.b_mn + 64, w.b_k + kb * kBlockK);
                        tma_load_2d(sb + 16384, &tmB, full, w.b_mn2, w.b_k + kb * kBlockK);
                        tma_load_2d(sb + 24576, &tmB, full, w.b_mn2 + 64, w.b_k + kb * kBlockK);
                    } else {
                        tma_load_2d(sb, &tmB, full, w.b_k + kb * kBlockK, w.b_mn);
                        tma_load_2d(sb + 16384, &tmB, full, w.b_k + kb * kBlockK, w.b_mn2);
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_bf16(kBlockM, kBlockN, 0, B_MN ? 1 : 0);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            for (int it = 0; it < total && !abort_flag; ++it) {
                const int k_iters = p.list[item_of(it)].k_iters;
                if (!mbar_wait(smem_u32(&bar_tempty[acc]), acc_phase ^ 1u, &abort_flag, p.status, budget)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kBlockN;
                bool ok = true;
                for (int kb = 0; kb < k_iters; ++kb) {
                    if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &abort_flag, p.status, budget)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = tiles_base + stage * kStageBytes;
                    const uint32_t sb = sa + kATileBytes;
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k) {
                        const uint64_t da = make_smem_desc(sa + k * 32, 16, 1024);
                        const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024)
                                                 : make_smem_desc(sb + k * 32, 16, 1024);
                        tc_mma_f16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&bar_empty[stage]));
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                tc_commit(smem_u32(&bar_tfull[acc]));
                if (++acc == 2) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    } else if (warp < 6) {
        // ---------------- epilogue ----------------
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t epi_stage = tiles_base + kStages * kStageBytes +
                                   quarter * (kScatter ? kScatterStageBytesPerWarp : kEpiStageBytesPerWarp);
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int it = 0; it < total && !abort_flag; ++it) {
            const GemmWork w = p.list[item_of(it)];
            if (!mbar_wait(smem_u32(&bar_tfull[acc]), acc_phase, &abort_flag, p.status, budget)) break;
            tc_fence_after();
            const uint32_t t_row = tmem_base + acc * kBlockN + (uint32_t(quarter * 32) << 16);
            if (kScatter) epilogue_scatter(p, ep, w, t_row, row_in_tile, epi_stage);
            else epilogue_tile(p, w, t_row, row_in_tile, epi_stage);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[acc]));
            if (++acc == 2) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
        if (kScatter) tma_store_wait<0>();     // every line this lane handed to the copy engine has been written
    } else if (warp < 6 + kPushWarps) {
        // ---------------- push warps: this rank's rows to their owners ----------------
        push_units<kPush, B_MN != 0>(ep, &abort_flag, lane, warp - 6, (int)threadIdx.x - kGemmThreads);
    } else if (kPush && lane == 0) {
        // ---------------- gate: walk this CTA's items ahead of the producer, wait for each tile's rows ----------------
        int ready = 0;   // pad0 of the last tile found complete
        for (int it = 0; it < total && !abort_flag; ++it) {
            const GemmWork w = p.list[item_of(it)];
            if (w.pad0 > 0 && w.pad0 != ready) {
                if (!wait_counter_ge(ep.arrive + (w.pad0 - 1), w.pad1, &abort_flag, p.status, ep.wait_budget_ns)) break;
                ready = w.pad0;
            }
            __threadfence_block();          // the acquire above is ordered before the count the producer reads
            ready_items = it + 1;
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// SwiGLU backward on the expert side with the routing weight folded in (see swiglu_bwd_weighted_kernel in moe.cu),
// which also hands every row's routing-weight gradient straight to the token owner: dw_bufs[src][slot] = <dact_u, act>.
__global__ void __launch_bounds__(256)
swiglu_bwd_weighted_scatter_kernel(const __nv_bfloat16* pre, const __nv_bfloat16* dact, const float* __restrict__ w,
                                   __nv_bfloat16* dpre, __nv_bfloat16* act_w, const int* __restrict__ meta,
                                   const __grid_constant__ EpParams ep_dw /* w_bufs = every rank's [T*k] float buffer */,
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
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (lane == 0) {
            const int tag = meta[r];
            if (tag >= 0) ep_dw.w_bufs[tag >> kMetaSlotBits][tag & ((1 << kMetaSlotBits) - 1)] = dot;
        }
    }
}

static int ep_num_sms() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

// operand stages + epilogue staging (the scatter form's lines are padded: 4 x 8,704 bytes) + barriers; the kernels
// declare their dynamic shared memory 1024-byte aligned and check that it is, so no alignment slack is provisioned
constexpr int kEpSmemBytes = kStages * kStageBytes + 4 * kEpiStageBytesPerWarp + 128;
constexpr int kEpScatterSmemBytes = kStages * kStageBytes + 4 * kScatterStageBytesPerWarp + 128;

template <bool B_MN, bool kPush, bool kScatter>
static int launch_ep(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, const EpParams& ep, cudaStream_t s) {
    constexpr int smem = kScatter ? kEpScatterSmemBytes : kEpSmemBytes;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_ep_kernel<B_MN, kPush, kScatter>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem) != cudaSuccess)
            return -10;
        configured = true;
    }
    gemm_ep_kernel<B_MN, kPush, kScatter><<<ep_num_sms(), kPush ? kEpPushThreads : kGemmThreads, smem, s>>>(ta, tb, p, ep);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

static unsigned long long g_peer_wait_ns = 0;
static unsigned long long peer_wait_ns() {
    if (!g_peer_wait_ns) {
        const char* e = getenv("HALO_PEER_WAIT_MS");
        const long long ms = e ? atoll(e) : 20000;
        g_peer_wait_ns = (unsigned long long)(ms > 0 ? ms : 20000) * 1000000ull;
    }
    return g_peer_wait_ns;
}

}  // namespace halo

using namespace halo;

extern "C" {

// ints a control block must hold for N ranks, E experts and max_tiles 128-row tiles per receive buffer
long long halo_moe_ctrl_ints(int N, int E, int max_tiles) { return 2LL * N * E + N + 2LL * max_tiles; }

// ctrl: HOST array of N device pointers (rank r's control block as mapped here). counts: this rank's [E] slot counts,
// or null for a call that only needs the handshake (a backward over a known routing).
int halo_moe_handshake(void* const* ctrl, int me, int N, int E, int seq, int max_tiles, const int* counts, int cap_rows,
                       int* seg_start, int* seg_rows, int* dst_base, int* total_rows, int* my_prefix, int* status,
                       void* stream) {
    if (N < 1 || N > kEpMaxPeers || E > 256 || E % N || seq < 1) return -1;
    IntPeers c;
    for (int i = 0; i < kEpMaxPeers; ++i) c.p[i] = i < N ? reinterpret_cast<int*>(ctrl[i]) : nullptr;
    moe_handshake_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(c, me, N, E, seq, max_tiles, counts, cap_rows, seg_start,
                                                             seg_rows, dst_base, total_rows, my_prefix, status,
                                                             peer_wait_ns());
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int halo_moe_push_unit_bytes() { return (int)sizeof(PushUnit); }
int halo_moe_tile_bytes() { return (int)sizeof(EpTile); }

int halo_moe_plan_push(const int* counts, const int* dst_base, const int* my_prefix, int me, int N, int E, int cap_rows,
                       void* units, int* n_units, int max_units, void* stream) {
    if (E > 256 || E % N) return -1;
    moe_plan_push_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(counts, dst_base, my_prefix, me, N, E, cap_rows,
                                                             reinterpret_cast<PushUnit*>(units), n_units, max_units);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int halo_moe_plan_tiles(void* const* ctrl, int me, int N, int E, int seq, const int* seg_start, const int* seg_rows,
                        void* tiles, int* n_tiles, int max_tiles, void* stream) {
    if (N < 1 || N > kEpMaxPeers || E > 256 || E % N) return -1;
    IntPeers c;
    for (int i = 0; i < kEpMaxPeers; ++i) c.p[i] = i < N ? reinterpret_cast<int*>(ctrl[i]) : nullptr;
    moe_plan_tiles_kernel<<<1, 256, E * sizeof(int), (cudaStream_t)stream>>>(c, me, N, E, seq, seg_start, seg_rows,
                                                                            reinterpret_cast<EpTile*>(tiles), n_tiles,
                                                                            max_tiles);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int halo_moe_plan_items(const void* tiles, const int* n_tiles, int n_cols, int k_dim, int b_mn_stride, int b_k_stride,
                        int swiglu_f, int gated, void* list, int* count, int max_items, void* stream) {
    moe_plan_items_kernel<<<64, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<const EpTile*>(tiles), n_tiles, n_cols,
                                                               k_dim, b_mn_stride, b_k_stride, swiglu_f, gated,
                                                               reinterpret_cast<GemmWork*>(list), count, max_items);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int halo_moe_zero_pads(void* buf, int* meta, float* roww, const int* seg_start, const int* seg_rows, int n_local, int H,
                       int cap_rows, void* stream) {
    if (n_local == 0) return 0;
    moe_zero_pads_kernel<<<dim3(n_local, 16), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)buf, meta, roww, seg_start,
                                                                             seg_rows, H, cap_rows);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int halo_moe_slot_sum(const void* slots, const int* slot_row, const float* w, void* out, long long T, int k, int H,
                      int cap_rows, void* stream) {
    if (H % 8) return -1;
    if (T == 0) return 0;
    const long long cap = (long long)ep_num_sms() * 8;
    moe_slot_sum_kernel<<<(unsigned)(T < cap ? T : cap), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)slots, slot_row, w, (__nv_bfloat16*)out, T, k, H, cap_rows / 128 * 128);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Kernel A: push this rank's rows (x, in send_slot order, by `units`) into the owners' receive buffers while multiplying
// the tiles of this rank's own receive buffer `A` (list items gated on `arrive`) with the expert bank B.
//   row_bufs / meta_bufs / w_bufs / arrive_bufs: HOST arrays of n_ranks device pointers (w_bufs and slot_w may be null).
//   epi: kEpiStoreBf16 or kEpiSwiglu (C, aux as in halo_gemm_bf16_list).
int halo_moe_dispatch_gemm(const void* x, const int* send_slot, const void* units, const int* n_units, const float* slot_w,
                           void* const* row_bufs, void* const* meta_bufs, void* const* w_bufs, void* const* arrive_bufs,
                           int n_ranks, int me, int H, int k,
                           const void* A, long long a_rows, const void* B, long long b_rows, long long b_cols, long long ldb,
                           void* C, void* aux, long long ldc, long long ld_aux, int b_mn_major, int epi, int swiglu_f,
                           int tiles_n, const void* list, const int* list_count, int* status, void* stream) {
    if (n_ranks < 1 || n_ranks > kEpMaxPeers || H % 8 || me < 0 || me >= n_ranks) return -1;
    if (epi != kEpiStoreBf16 && epi != kEpiSwiglu) return -2;
    CUtensorMap ta, tb;
    int rc = make_tmap_bf16(&ta, A, a_rows, H, H, 128);
    if (rc) return rc;
    rc = make_tmap_bf16(&tb, B, b_rows, b_cols, ldb, b_mn_major ? 64 : 128);
    if (rc) return rc * 10;
    GemmParams p{};
    p.C = C; p.aux = aux; p.ldc = ldc; p.ld_aux = ld_aux; p.epi = epi; p.alpha = 1.f; p.swiglu_f = swiglu_f;
    p.tiles_n = tiles_n;
    p.list = reinterpret_cast<const GemmWork*>(list);
    p.list_count = list_count;
    p.status = status;
    EpParams ep{};
    ep.x = (const __nv_bfloat16*)x; ep.send_slot = send_slot; ep.units = reinterpret_cast<const PushUnit*>(units);
    ep.n_units = n_units; ep.slot_w = slot_w;
    for (int i = 0; i < n_ranks; ++i) {
        ep.row_bufs[i] = row_bufs[i];
        ep.meta_bufs[i] = reinterpret_cast<int*>(meta_bufs[i]);
        ep.w_bufs[i] = w_bufs ? reinterpret_cast<float*>(w_bufs[i]) : nullptr;
        ep.arrive_bufs[i] = reinterpret_cast<int*>(arrive_bufs[i]);
    }
    ep.arrive = ep.arrive_bufs[me];
    ep.H = H; ep.k = k; ep.me = me;
    ep.wait_budget_ns = peer_wait_ns();
    if (slot_w && !w_bufs) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    return b_mn_major ? launch_ep<true, true, false>(ta, tb, p, ep, s) : launch_ep<false, true, false>(ta, tb, p, ep, s);
}

// Kernel B: grouped product of local rows A [a_rows, a_cols] with the expert bank, every output row stored into the
// token owner's slot buffer (slot_bufs: HOST array of n_ranks device pointers to [T * k, ldc] bf16) by its tag meta[row].
int halo_moe_gemm_combine(const void* A, long long a_rows, long long a_cols, long long lda, const void* B, long long b_rows,
                          long long b_cols, long long ldb, void* const* slot_bufs, const int* meta, int n_ranks,
                          long long ldc, int b_mn_major, int tiles_n, const void* list, const int* list_count, int* status,
                          void* stream) {
    if (n_ranks < 1 || n_ranks > kEpMaxPeers || ldc % 8) return -1;
    CUtensorMap ta, tb;
    int rc = make_tmap_bf16(&ta, A, a_rows, a_cols, lda, 128);
    if (rc) return rc;
    rc = make_tmap_bf16(&tb, B, b_rows, b_cols, ldb, b_mn_major ? 64 : 128);
    if (rc) return rc * 10;
    GemmParams p{};
    p.C = nullptr; p.aux = nullptr; p.ldc = ldc; p.ld_aux = 0; p.epi = kEpiStoreBf16; p.alpha = 1.f; p.swiglu_f = 0;
    p.tiles_n = tiles_n;
    p.list = reinterpret_cast<const GemmWork*>(list);
    p.list_count = list_count;
    p.status = status;
    EpParams ep{};
    for (int i = 0; i < n_ranks; ++i) ep.slot_bufs[i] = slot_bufs[i];
    ep.meta = meta;
    ep.wait_budget_ns = peer_wait_ns();
    cudaStream_t s = (cudaStream_t)stream;
    return b_mn_major ? launch_ep<true, false, true>(ta, tb, p, ep, s) : launch_ep<false, false, true>(ta, tb, p, ep, s);
}

int halo_moe_swiglu_bwd_scatter(const void* pre, const void* dact, const float* w, void* dpre, void* act_w, const int* meta,
                                void* const* dw_bufs, int n_ranks, const int* total_rows, int F, int cap_rows, void* stream) {
    if (F % 8 || n_ranks < 1 || n_ranks > kEpMaxPeers) return -1;
    EpParams ep{};
    for (int i = 0; i < n_ranks; ++i) ep.w_bufs[i] = reinterpret_cast<float*>(dw_bufs[i]);
    swiglu_bwd_weighted_scatter_kernel<<<2368, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)pre, (const __nv_bfloat16*)dact, w, (__nv_bfloat16*)dpre, (__nv_bfloat16*)act_w, meta, ep,
        total_rows, F, cap_rows);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
