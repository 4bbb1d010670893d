"""Tensor parallelism with sequence-sharded activations.

Between blocks every rank of the tensor-parallel group holds ``T / tp`` tokens of the packed row (norms,
residuals, the router, the experts and the loss are token-local, exactly as under context parallelism). Inside
an attention or dense-FFN block the tokens are gathered, the block runs on ``1 / tp`` of the heads (or of the
FFN width) with column-sliced first and row-sliced second projection, and the partial outputs are summed and
scattered back to token shards:

    h_shard --gather--> h [T, H] --W1 slice--> ... --W2 slice--> partial [T, H] --reduce-scatter--> y_shard

The reference keeps activations replicated and all-reduces them (halo/distributed/tensor_parallel/
local_linears.py:94-111, parallelize_attention.py:40-193); gather + reduce-scatter moves the same bytes and leaves
every token-local op with ``1 / tp`` of the work.

On GPUs both collectives run on this framework's own kernels over peer-mapped memory. The gather publishes the
shard in a symmetric buffer and pulls the peers' shards with the peer-copy kernel. The second projection is ONE
kernel with its reduce-scatter's transfer (``halo_gemm_bf16_reduce_scatter``): the tcgen05 GEMM's epilogue stores
every output tile straight into the staging slot of the rank that owns those rows, other owners' tiles first, so
the NVLink stores drain under the remaining tiles' math; each rank then sums its slots in fp32
(``rs_sum_norm_kernel``, the kernel of the sharded optimizer's gradient reduction). A stand-alone reduce-scatter of
an existing tensor (the backward of the gather) publishes the tensor and sums over the peers' buffers with the same
kernel. CPU tensors take ``torch.distributed`` collectives so that gloo tests cover slicing, layouts and gradients.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from halo_b200.ops import _lib


class TensorParallel:
    def __init__(self, group, device, hidden: int = 0, max_tokens: int = 0):
        self.group = group
        self.size, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = torch.device(device)
        self.sym = None
        if self.device.type == "cuda":
            if not (hidden and max_tokens):
                raise ValueError("the GPU tensor-parallel path needs hidden and max_tokens to size its symmetric buffers")
            import torch.distributed._symmetric_memory as symm

            self.sym = symm.empty((max_tokens, hidden), dtype=torch.bfloat16, device=self.device)
            self.handle = symm.rendezvous(self.sym, group)
            self.ptrs = list(self.handle.buffer_ptrs)
            self._ptr_table = (_lib.c_void_p * self.size)(*self.ptrs)

    def barrier(self) -> None:
        self.handle.barrier(channel=12)

    def shard_rows(self, total: int) -> tuple[int, int]:
        if total % self.size:
            raise ValueError(f"{total} tokens cannot be cut into {self.size} equal shards: pad the row")
        n = total // self.size
        return self.rank * n, (self.rank + 1) * n


# ---- the two collectives -------------------------------------------------------------------------------
def _all_gather_rows(x: torch.Tensor, tp: TensorParallel) -> torch.Tensor:
    n = x.shape[0]
    if not x.is_cuda:
        parts = [torch.empty_like(x) for _ in range(tp.size)]
        dist.all_gather(parts, x.contiguous(), group=tp.group)
        return torch.cat(parts, dim=0)
    out = torch.empty((n * tp.size, x.shape[1]), dtype=x.dtype, device=x.device)
    tp.sym[:n].copy_(x)
    tp.barrier()
    row_bytes = x.shape[1] * x.element_size()
    L = _lib.lib()
    for r in range(tp.size):
        dst = out[r * n:(r + 1) * n]
        if r == tp.rank:
            dst.copy_(x)
        else:
            _lib.check(L.halo_peer_pull(_lib.ptr(dst), _lib.c_void_p(tp.ptrs[r]), _lib.c_ll(n * row_bytes), _lib.c_int(0),
                                        _lib.stream_ptr(x.device)), "halo_peer_pull")
    tp.barrier()                # peers have read the shard before its buffer is reused
    return out


def _reduce_scatter_rows(y: torch.Tensor, tp: TensorParallel) -> torch.Tensor:
    lo, hi = tp.shard_rows(y.shape[0])
    if not y.is_cuda:
        total = y.contiguous().clone()
        dist.all_reduce(total, group=tp.group)
        return total[lo:hi].clone()
    cols = y.shape[1]
    tp.sym[:y.shape[0]].copy_(y)
    tp.barrier()
    n = (hi - lo) * cols
    L = _lib.lib()
    gsum = torch.empty(n, dtype=torch.float32, device=y.device)
    partial = torch.empty(int(L.halo_rs_blocks(_lib.c_ll(n))), dtype=torch.float32, device=y.device)
    _lib.check(L.halo_rs_sum_norm(tp._ptr_table, _lib.c_int(tp.size), _lib.c_ll(lo * cols), _lib.c_ll(n), _lib.ptr(gsum),
                                  _lib.ptr(partial), _lib.stream_ptr(y.device)), "halo_rs_sum_norm")
    tp.barrier()
    return gsum.view(hi - lo, cols).to(y.dtype)


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return _all_gather_rows(x, tp)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_rows(g.contiguous(), ctx.tp), None


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, tp):
        ctx.tp = tp
        return _reduce_scatter_rows(y.contiguous(), tp)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_rows(g.contiguous(), ctx.tp), None


def _fused_gemm_reduce_scatter(x: torch.Tensor, w: torch.Tensor, tp: TensorParallel) -> torch.Tensor:
    """y_shard = rows of (x w^T summed over ranks) owned by this rank, with the transfer inside the GEMM: every
    output tile is stored by the epilogue straight into its owner's staging slot over NVLink (tiles of other owners
    first), then each rank sums its slots in fp32."""
    T, N = x.shape[0], w.shape[0]
    rows = T // tp.size
    if tp.sym.shape[0] * tp.sym.shape[1] < T * N:
        raise RuntimeError("the tensor-parallel staging buffer is smaller than the product")
    L = _lib.lib()
    dev = x.device
    tp.barrier()        # every rank has finished reading its staging slots of the previous product
    rc = L.halo_gemm_bf16_reduce_scatter(_lib.ptr(x), _lib.ptr(w), tp._ptr_table, _lib.c_int(tp.size), _lib.c_int(tp.rank),
                                         _lib.c_int(T), _lib.c_int(N), _lib.c_int(x.shape[1]), _lib.c_ll(x.stride(0)),
                                         _lib.c_ll(w.stride(0)), _lib.c_int(0), _lib.ptr(_lib.status_word(dev)),
                                         _lib.stream_ptr(dev))
    _lib.check(rc, "halo_gemm_bf16_reduce_scatter")
    tp.barrier()        # all partial tiles have landed
    n = rows * N
    slots = (_lib.c_void_p * tp.size)(*[tp.sym.data_ptr() + s * n * 2 for s in range(tp.size)])
    gsum = torch.empty(n, dtype=torch.float32, device=dev)
    partial = torch.empty(int(L.halo_rs_blocks(_lib.c_ll(n))), dtype=torch.float32, device=dev)
    _lib.check(L.halo_rs_sum_norm(slots, _lib.c_int(tp.size), _lib.c_ll(0), _lib.c_ll(n), _lib.ptr(gsum), _lib.ptr(partial),
                                  _lib.stream_ptr(dev)), "halo_rs_sum_norm")
    return gsum.view(rows, N).to(x.dtype)


class _RowParallelLinear(torch.autograd.Function):
    """y_shard = reduce_scatter(x w^T) for a row-sliced ``w`` ([N, K / tp]) and the matching slice of ``x``."""

    @staticmethod
    def forward(ctx, x, w, tp):
        from halo_b200.ops import gemm

        ctx.tp = tp
        ctx.save_for_backward(x, w)
        rows_ok = x.shape[0] % (128 * tp.size) == 0
        if x.is_cuda and x.dtype == torch.bfloat16 and rows_ok and x.stride(1) == 1 and w.is_contiguous():
            return _fused_gemm_reduce_scatter(x, w, tp)
        return _reduce_scatter_rows(gemm.matmul(x, w).contiguous(), tp)

    @staticmethod
    def backward(ctx, g):
        from halo_b200.ops import gemm

        x, w = ctx.saved_tensors
        dy = _all_gather_rows(g.contiguous(), ctx.tp)
        dx = gemm.matmul(dy, w, b_t=False) if ctx.needs_input_grad[0] else None
        dw = gemm.matmul(dy, x, a_t=True, b_t=False) if ctx.needs_input_grad[1] else None
        return dx, dw, None


def row_parallel_linear(x: torch.Tensor, w: torch.Tensor, tp: TensorParallel) -> torch.Tensor:
    """Second projection of a tensor-parallel block: [T, K / tp] x [N, K / tp]^T summed over ranks -> [T / tp, N]."""
    return _RowParallelLinear.apply(x, w, tp)


def gather_seq(x_shard: torch.Tensor, tp: TensorParallel) -> torch.Tensor:
    """[T/tp, H] token shards -> [T, H]; the backward sums and scatters the gradient."""
    return _GatherSeq.apply(x_shard, tp)


def reduce_scatter_seq(y_partial: torch.Tensor, tp: TensorParallel) -> torch.Tensor:
    """Partial [T, H] products of every rank -> this rank's token shard of their sum."""
    return _ReduceScatterSeq.apply(y_partial, tp)


# ---- weight slicing ------------------------------------------------------------------------------------
def slice_for_rank(kind: str, full: torch.Tensor, cfg, rank: int, size: int) -> torch.Tensor:
    """This rank's slice of a full weight. ``kind``: ``qkv`` (rows: heads of q, k, v), ``o`` (columns: q heads),
    ``gate_up`` (rows: gate and up halves), ``down`` (columns)."""
    D = cfg.head_dim
    if kind in ("qkv", "qkv_bias"):      # the bias of the fused projection is cut like its rows
        Hq, Hkv = cfg.num_attention_heads, cfg.num_key_value_heads
        q, k, v = full.split([Hq * D, Hkv * D, Hkv * D], dim=0)
        nq, nk = Hq // size * D, Hkv // size * D
        return torch.cat([q[rank * nq:(rank + 1) * nq], k[rank * nk:(rank + 1) * nk], v[rank * nk:(rank + 1) * nk]], dim=0)
    if kind == "o":
        n = full.shape[1] // size
        return full[:, rank * n:(rank + 1) * n]
    if kind == "gate_up":
        F = full.shape[0] // 2
        n = F // size
        return torch.cat([full[rank * n:(rank + 1) * n], full[F + rank * n:F + (rank + 1) * n]], dim=0)
    if kind == "down":
        n = full.shape[1] // size
        return full[:, rank * n:(rank + 1) * n]
    raise ValueError(f"unknown tensor-parallel slice kind {kind!r}")


def unslice(kind: str, parts: list[torch.Tensor], cfg) -> torch.Tensor:
    """Inverse of :func:`slice_for_rank` given every rank's slice in rank order."""
    size, D = len(parts), cfg.head_dim
    if kind in ("qkv", "qkv_bias"):
        nq, nk = cfg.num_attention_heads // size * D, cfg.num_key_value_heads // size * D
        qs, ks, vs = zip(*(p.split([nq, nk, nk], dim=0) for p in parts))
        return torch.cat(list(qs) + list(ks) + list(vs), dim=0)
    if kind in ("o", "down"):
        return torch.cat(parts, dim=1)
    if kind == "gate_up":
        gs, us = zip(*(p.chunk(2, dim=0) for p in parts))
        return torch.cat(list(gs) + list(us), dim=0)
    raise ValueError(f"unknown tensor-parallel slice kind {kind!r}")


def gather_full_weight(kind: str, local: torch.Tensor, cfg, tp: TensorParallel) -> torch.Tensor:
    """COLLECTIVE: the unsliced weight on every rank (checkpoint saves)."""
    parts = [torch.empty_like(local) for _ in range(tp.size)]
    dist.all_gather(parts, local.contiguous(), group=tp.group)
    return unslice(kind, parts, cfg)


def check_divisibility(cfg, size: int) -> None:
    if cfg.num_attention_heads % size or cfg.num_key_value_heads % size:
        raise ValueError(f"tensor_parallel_size {size} must divide the query heads ({cfg.num_attention_heads}) and the "
                         f"key/value heads ({cfg.num_key_value_heads})")
    if not cfg.is_moe and cfg.intermediate_size % size:
        raise ValueError(f"tensor_parallel_size {size} must divide the FFN width ({cfg.intermediate_size})")
