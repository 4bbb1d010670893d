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


class _GatherRows(torch.autograd.Function):
    """cat over ranks of equally-shaped tensors; backward: sum over ranks of the matching slice."""

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


class _ScatterSumRows(torch.autograd.Function):
    """out_r = sum over ranks of partial[r*rows:(r+1)*rows]; backward: gather of the gradient."""

    @staticmethod
    def forward(ctx, partial, group):
        world = dist.get_world_size(group)
        ctx.group = group
        total = partial.contiguous().clone()
        dist.all_reduce(total, group=group)
        rows = partial.shape[0] // world
        r = dist.get_rank(group)
        return total[r * rows:(r + 1) * rows].clone()

    @staticmethod
    def backward(ctx, g):
        world = dist.get_world_size(ctx.group)
        parts = [torch.empty_like(g) for _ in range(world)]
        dist.all_gather(parts, g.contiguous(), group=ctx.group)
        return torch.cat(parts, dim=0), None


class CollectiveTransport:
    """Expert-parallel transport made of all-gather + reduce: works on gloo (CPU) and NCCL."""

    def __init__(self, group=None):
        self.group = group
        self.n_ranks = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.stable_until_backward = True

    def reference_ffn(self, x, topk_idx, topk_w, w_gate_up, w_down):
        e_local = w_gate_up.shape[0]
        xs = _GatherRows.apply(x, self.group)
        ws = _GatherRows.apply(topk_w.to(torch.float32), self.group)
        idx_parts = [torch.empty_like(topk_idx) for _ in range(self.n_ranks)]
        dist.all_gather(idx_parts, topk_idx.contiguous(), group=self.group)
        idx = torch.cat(idx_parts, dim=0)
        partial = moe_ffn_reference(xs, idx, ws, w_gate_up, w_down, expert_offset=self.rank * e_local)
        return _ScatterSumRows.apply(partial, self.group)

    # the CUDA kernels never see this transport
    def capacity(self, n_slots, n_local):  # pragma: no cover
        raise RuntimeError("CollectiveTransport serves the PyTorch path only")


def moe_experts_collective(x, topk_idx, topk_w, w_gate_up, w_down, transport: CollectiveTransport):
    return transport.reference_ffn(x, topk_idx, topk_w, w_gate_up, w_down)
