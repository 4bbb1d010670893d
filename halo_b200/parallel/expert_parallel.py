"""Expert parallelism on any backend through plain collectives: the CPU / gloo path and the
reference implementation the peer-memory transport is checked against.

Every rank gathers all ranks' tokens and routing, applies its own experts to the tokens routed to
them, and the partial outputs are summed back to the owning rank. It moves far more data than the
push/pull transport (halo_b200.parallel.runtime.SymmetricTransport), which is the point: it shares
no code with it, so agreement between the two is meaningful. Gradients flow through the
collectives (an all-gather's backward is a reduce-scatter and vice versa).

Plays the part of the reference's loopback backend and EP-vs-no-EP equivalence harness
(tests/common/ep_stubs.py:24-58, tests/cpu/parallelism/test_ep_vs_reference_equivalence_cpu.py).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from halo_b200.ops.moe import moe_ffn_reference


def _row_counts(n: int, group) -> list[int]:
    world = dist.get_world_size(group)
    t = torch.tensor([n], dtype=torch.int64)
    out = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(out, t, group=group)
    return [int(o.item()) for o in out]


def _pad_rows(x, rows: int):
    if x.shape[0] == rows:
        return x.contiguous()
    pad = torch.zeros((rows - x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    return torch.cat([x, pad], dim=0)


class _GatherRows(torch.autograd.Function):
    """cat over ranks (row counts may differ per rank); backward: sum over ranks of the matching slice."""

    @staticmethod
    def forward(ctx, x, group, counts):
        world, widest = dist.get_world_size(group), max(counts)
        parts = [torch.empty((widest,) + tuple(x.shape[1:]), dtype=x.dtype) for _ in range(world)]
        dist.all_gather(parts, _pad_rows(x, widest), group=group)
        ctx.group, ctx.counts = group, counts
        return torch.cat([p[:c] for p, c in zip(parts, counts)], dim=0)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        r = dist.get_rank(ctx.group)
        lo = sum(ctx.counts[:r])
        return g[lo:lo + ctx.counts[r]], None, None


class _ScatterSumRows(torch.autograd.Function):
    """out_r = sum over ranks of this rank's row block of ``partial``; backward: gather of the gradient."""

    @staticmethod
    def forward(ctx, partial, group, counts):
        ctx.group, ctx.counts = group, counts
        total = partial.contiguous().clone()
        dist.all_reduce(total, group=group)
        r = dist.get_rank(group)
        lo = sum(counts[:r])
        return total[lo:lo + counts[r]].clone()

    @staticmethod
    def backward(ctx, g):
        world, widest = dist.get_world_size(ctx.group), max(ctx.counts)
        parts = [torch.empty((widest,) + tuple(g.shape[1:]), dtype=g.dtype) for _ in range(world)]
        dist.all_gather(parts, _pad_rows(g, widest), group=ctx.group)
        return torch.cat([p[:c] for p, c in zip(parts, ctx.counts)], dim=0), None, None


class CollectiveTransport:
    """Expert-parallel transport made of all-gather + reduce: works on gloo (CPU) and NCCL."""

    def __init__(self, group=None):
        self.group = group
        self.n_ranks = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.stable_until_backward = True

    def reference_ffn(self, x, topk_idx, topk_w, w_gate_up, w_down):
        e_local = w_gate_up.shape[0]
        counts = _row_counts(x.shape[0], self.group)
        xs = _GatherRows.apply(x, self.group, counts)
        ws = _GatherRows.apply(topk_w.to(torch.float32), self.group, counts)
        idx = _GatherRows.apply(topk_idx, self.group, counts)
        partial = moe_ffn_reference(xs, idx, ws, w_gate_up, w_down, expert_offset=self.rank * e_local)
        return _ScatterSumRows.apply(partial, self.group, counts)

    # the CUDA kernels never see this transport
    def capacity(self, n_slots, n_local):  # pragma: no cover
        raise RuntimeError("CollectiveTransport serves the PyTorch path only")


def moe_experts_collective(x, topk_idx, topk_w, w_gate_up, w_down, transport: CollectiveTransport):
    return transport.reference_ffn(x, topk_idx, topk_w, w_gate_up, w_down)
