"""Context parallelism on packed rows: the row is cut into ``cp`` contiguous chunks, one per rank; everything
except attention is token-local; attention needs, for the documents that start before a rank's chunk, the keys
and values of their earlier tokens, which live on lower ranks.

Each rank publishes its chunk's K/V (after rotary) in a symmetric buffer; a rank pulls exactly the rows it
needs - the tail of the documents that straddle into its chunk - out of its peers' buffers with its own copy
kernel over NVLink, lays them in front of its local K/V and runs the ordinary flash kernels on that extended
index space with work lists that hold only its own query tiles. In the backward pass the key/value gradients
of the pulled rows are published the same way and each owner adds the contributions of higher ranks to its own
(in rank order: deterministic, no atomics).

With chat-length documents a chunk needs a few thousand foreign rows at most; with one long document it needs
all earlier chunks, which is the ring-attention case done as direct pulls (NVSwitch gives every pair full
bandwidth, so a ring's neighbour-only pattern buys nothing on this machine).

The reference's context parallelism is Ulysses all-to-all and refuses packed rows
(halo/distributed/context_parallel/ulysses_model.py:199-312, model_rules.py); this is the packed-row replacement.
The CPU path expresses the same exchange with a differentiable all-gather so that gloo tests cover the layout,
masks and gradient return.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch
import torch.distributed as dist

from halo_b200.ops import _lib
from halo_b200.ops import attention as attn_ops


@dataclass
class CPLayout:
    cp_rank: int
    cp_size: int
    total: int
    lo: int                    # first global token of this rank's chunk
    hi: int
    p0: int                    # first global token this rank needs keys for (start of the document holding ``lo``)
    cu_ext: np.ndarray         # document offsets of the extended local space [p0, hi), starting at 0
    sources: list = field(default_factory=list)   # (rank, row in that rank's chunk, n_rows, row in my prefix)
    returns: list = field(default_factory=list)   # (rank, row in my chunk, n_rows, row in that rank's prefix)

    @property
    def prefix(self) -> int:
        return self.lo - self.p0

    @property
    def local(self) -> int:
        return self.hi - self.lo


def chunk_bounds(total: int, cp_size: int, rank: int) -> tuple[int, int]:
    if total % cp_size:
        raise ValueError(f"a packed row of {total} tokens cannot be cut into {cp_size} equal chunks: pad the row")
    c = total // cp_size
    return rank * c, (rank + 1) * c


def _first_needed(cu: np.ndarray, lo: int) -> int:
    """Start of the document that contains token ``lo`` (``lo`` itself when a document starts there)."""
    d = int(np.searchsorted(cu, lo, side="right")) - 1
    return int(cu[d])


def make_layout(cu_seqlens, cp_rank: int, cp_size: int) -> CPLayout:
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    total = int(cu[-1])
    lo, hi = chunk_bounds(total, cp_size, cp_rank)
    p0 = _first_needed(cu, lo) if lo < total else lo
    inner = cu[(cu > p0) & (cu < hi)]
    cu_ext = np.concatenate([[p0], inner, [hi]]) - p0
    lay = CPLayout(cp_rank, cp_size, total, lo, hi, p0, cu_ext.astype(np.int64))
    for s in range(cp_rank):
        s_lo, s_hi = chunk_bounds(total, cp_size, s)
        a, b = max(p0, s_lo), min(lo, s_hi)
        if a < b:
            lay.sources.append((s, a - s_lo, b - a, a - p0))
    for s in range(cp_rank + 1, cp_size):
        s_lo, _ = chunk_bounds(total, cp_size, s)
        s_p0 = _first_needed(cu, s_lo)
        a, b = max(s_p0, lo), min(s_lo, hi)
        if a < b:
            lay.returns.append((s, a - lo, b - a, a - s_p0))
    return lay


def build_cp_plan(layout: CPLayout, device) -> attn_ops.AttentionPlan:
    """Tile lists over the extended space that hold only this rank's query tiles (and, for dK/dV, every key tile
    with the query range cut to this rank's queries)."""
    return attn_ops.build_plan(layout.cu_ext, device, q_lo=layout.prefix)


# ---- differentiable gather for the PyTorch path -----------------------------------------------------
class _GatherChunks(torch.autograd.Function):
    """cat over the group of equally long chunks; backward: sum over ranks of the matching slice."""

    @staticmethod
    def forward(ctx, x, group):
        world = dist.get_world_size(group)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        ctx.group, ctx.rows = group, x.shape[0]
        return torch.cat(parts, dim=0)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        r = dist.get_rank(ctx.group)
        return g[r * ctx.rows:(r + 1) * ctx.rows], None


class CPExchange:
    """Symmetric buffers and barriers of one context-parallel group (GPU path)."""

    def __init__(self, group, device, max_local_rows: int, max_prefix_rows: int, kv_cols: int):
        import torch.distributed._symmetric_memory as symm

        self.group, self.device = group, torch.device(device)
        self.n_ranks, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.kv = symm.empty((max_local_rows, kv_cols), dtype=torch.bfloat16, device=self.device)
        self.dkv = symm.empty((max(max_prefix_rows, 8), kv_cols), dtype=torch.bfloat16, device=self.device)
        self.h_kv = symm.rendezvous(self.kv, group)
        self.h_dkv = symm.rendezvous(self.dkv, group)
        self.kv_ptrs = list(self.h_kv.buffer_ptrs)
        self.dkv_ptrs = list(self.h_dkv.buffer_ptrs)
        self.row_bytes = kv_cols * 2

    def barrier(self) -> None:
        self.h_kv.barrier(channel=3)

    def pull(self, dst: torch.Tensor, base_ptr: int, first_row: int, n_rows: int, accumulate: bool) -> None:
        rc = _lib.lib().halo_peer_pull(_lib.ptr(dst), _lib.c_void_p(base_ptr + first_row * self.row_bytes),
                                       _lib.c_ll(n_rows * self.row_bytes), _lib.c_int(1 if accumulate else 0),
                                       _lib.stream_ptr(self.device))
        _lib.check(rc, "halo_peer_pull")


class _CPFlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, layout: CPLayout, plan, exchange: CPExchange, n_heads, n_kv_heads, scale):
        P, Tl = layout.prefix, layout.local
        dev = q.device
        D = attn_ops.HEAD_DIM
        kvd = n_kv_heads * D
        # publish this chunk's K | V, then pull the rows of straddling documents from their owners
        exchange.kv[:Tl, :kvd].copy_(k)
        exchange.kv[:Tl, kvd:].copy_(v)
        exchange.barrier()
        kv_ext = torch.empty((P + Tl, 2 * kvd), dtype=torch.bfloat16, device=dev)
        for rank, src_row, n, dst_row in layout.sources:
            exchange.pull(kv_ext[dst_row:dst_row + n], exchange.kv_ptrs[rank], src_row, n, accumulate=False)
        kv_ext[P:].copy_(exchange.kv[:Tl])
        exchange.barrier()       # peers are done reading before the next layer overwrites the published rows
        q_ext = torch.zeros((P + Tl, n_heads * D), dtype=torch.bfloat16, device=dev)   # zero queries in the prefix
        q_ext[P:].copy_(q)
        o_ext = torch.empty_like(q_ext)
        o_ext[:P].zero_()
        lse = torch.empty((n_heads, P + Tl), dtype=torch.float32, device=dev)
        k_ext, v_ext = kv_ext[:, :kvd], kv_ext[:, kvd:]
        attn_ops._launch_fwd(_lib.lib(), q_ext, k_ext, v_ext, o_ext, lse, plan, P + Tl, n_heads, n_kv_heads, scale, dev)
        ctx.save_for_backward(q_ext, kv_ext, o_ext, lse)
        ctx.meta = (layout, plan, exchange, n_heads, n_kv_heads, scale)
        return o_ext[P:]

    @staticmethod
    def backward(ctx, do):
        q_ext, kv_ext, o_ext, lse = ctx.saved_tensors
        layout, plan, exchange, n_heads, n_kv_heads, scale = ctx.meta
        P, Tl = layout.prefix, layout.local
        dev = do.device
        D = attn_ops.HEAD_DIM
        kvd = n_kv_heads * D
        Te = P + Tl
        do_ext = torch.zeros((Te, n_heads * D), dtype=torch.bfloat16, device=dev)
        do_ext[P:].copy_(do)
        dq_ext = torch.empty_like(q_ext)
        dkv_ext = torch.empty_like(kv_ext)
        delta = torch.empty((n_heads, Te), dtype=torch.float32, device=dev)
        k_ext, v_ext = kv_ext[:, :kvd], kv_ext[:, kvd:]
        dk, dv = dkv_ext[:, :kvd], dkv_ext[:, kvd:]
        L = _lib.lib()
        ld = attn_ops._ld
        rc = L.halo_attn_bwd(
            _lib.ptr(q_ext), _lib.ptr(k_ext), _lib.ptr(v_ext), _lib.ptr(o_ext), _lib.ptr(do_ext), _lib.ptr(lse), _lib.ptr(delta),
            _lib.ptr(dq_ext), _lib.ptr(dk), _lib.ptr(dv),
            _lib.ptr(plan.bwd_kv), _lib.c_int(plan.bwd_kv.shape[0]), _lib.ptr(plan.bwd_q), _lib.c_int(plan.bwd_q.shape[0]),
            _lib.c_ll(Te), _lib.c_int(n_heads), _lib.c_int(n_kv_heads), _lib.c_int(D),
            _lib.c_ll(ld(q_ext)), _lib.c_ll(ld(k_ext)), _lib.c_ll(ld(v_ext)), _lib.c_ll(ld(o_ext)), _lib.c_ll(ld(do_ext)),
            _lib.c_ll(ld(dq_ext)), _lib.c_ll(ld(dk)), _lib.c_ll(ld(dv)),
            _lib.c_float(scale), _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(dev))
        _lib.check(rc, "halo_attn_bwd")
        # publish the gradients of the pulled rows; each owner adds what higher ranks computed for its rows
        if P:
            exchange.dkv[:P].copy_(dkv_ext[:P])
        exchange.barrier()
        dkv_local = dkv_ext[P:].contiguous()
        for rank, my_row, n, src_row in layout.returns:          # ascending rank: a fixed summation order
            exchange.pull(dkv_local[my_row:my_row + n], exchange.dkv_ptrs[rank], src_row, n, accumulate=True)
        exchange.barrier()
        return dq_ext[P:], dkv_local[:, :kvd], dkv_local[:, kvd:], None, None, None, None, None, None


def cp_attention(q, k, v, layout: CPLayout, plan, group, exchange: CPExchange | None, n_heads: int, n_kv_heads: int,
                 scale: float | None = None):
    """Causal attention of this rank's chunk of a packed row. q: [T_local, Hq*D]; k, v: [T_local, Hkv*D]."""
    D = q.shape[1] // n_heads
    scale = float(scale if scale is not None else D**-0.5)
    if q.is_cuda:
        if exchange is None:
            raise RuntimeError("the GPU context-parallel path needs a CPExchange (symmetric K/V buffers)")
        return _CPFlashAttention.apply(q.contiguous(), k, v, layout, plan, exchange, n_heads, n_kv_heads, scale)
    # PyTorch path: gather every chunk's K/V (differentiably), attend over the extended space, keep the local rows
    k_all, v_all = _GatherChunks.apply(k, group), _GatherChunks.apply(v, group)
    k_ext, v_ext = k_all[layout.p0:layout.hi], v_all[layout.p0:layout.hi]
    q_ext = torch.cat([q.new_zeros((layout.prefix, q.shape[1])), q], dim=0)
    o_ext = attn_ops.attention_reference(q_ext, k_ext, v_ext, layout.cu_ext, n_heads, n_kv_heads, scale)
    return o_ext[layout.prefix:]


class ContextParallel:
    """Per-run state the model's forward context carries when ``context_parallel_size > 1``."""

    def __init__(self, group, device, cfg, max_row_tokens: int):
        self.group = group
        self.size, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = torch.device(device)
        self.exchange = None
        if self.device.type == "cuda":
            local = max_row_tokens // self.size
            self.exchange = CPExchange(group, device, local, max_row_tokens - local, 2 * cfg.num_key_value_heads * cfg.head_dim)

    def layout_and_plan(self, cu_seqlens):
        lay = make_layout(cu_seqlens, self.rank, self.size)
        return lay, build_cp_plan(lay, self.device)


def slice_batch(batch, cp_rank: int, cp_size: int):
    """This rank's chunk of a packed batch; ``cu_seqlens`` stays the whole row's (the layout needs it)."""
    from halo_b200.data.packing import PackedBatch

    lo, hi = chunk_bounds(batch.n_tokens, cp_size, cp_rank)
    labels = batch.labels[lo:hi]
    return PackedBatch(batch.input_ids[lo:hi], batch.position_ids[lo:hi], labels, batch.cu_seqlens,
                       int((labels != -100).sum()))
