"""Expert tensor parallelism: the intermediate width of every routed expert is cut over the ranks of a group.

Each rank of the group sees the SAME tokens and the same routing, holds ``1 / etp`` of every expert's gate/up rows and
down columns, and produces a partial expert output; the partial outputs are summed in token space, outside the
dispatch -> combine path (halo/distributed/expert_parallel/moe_layer/compute.py:106-127, layer.py:316-340,
halo/distributed/grad_reduce.py:58-86). Two autograd identities carry it:

    copy_to_group(h):     forward identity,  backward all-reduce   (every rank's slice contributes to d h)
    sum_from_group(y):    forward all-reduce, backward identity    (every rank needs the whole d y)
"""

from __future__ import annotations

import torch
import torch.distributed as dist


class ExpertTensorParallel:
    def __init__(self, group):
        self.group = group
        self.size, self.rank = dist.get_world_size(group), dist.get_rank(group)

    def check(self, cfg) -> None:
        if cfg.moe_intermediate_size % self.size:
            raise ValueError(f"expert_tensor_parallel_size {self.size} must divide the expert width ({cfg.moe_intermediate_size})")


class _CopyToGroup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _SumFromGroup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, group):
        y = y.contiguous().clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


def copy_to_group(x: torch.Tensor, etp: ExpertTensorParallel) -> torch.Tensor:
    return _CopyToGroup.apply(x, etp.group)


def sum_from_group(y: torch.Tensor, etp: ExpertTensorParallel) -> torch.Tensor:
    return _SumFromGroup.apply(y, etp.group)


def slice_expert_bank(kind: str, full: torch.Tensor, rank: int, size: int) -> torch.Tensor:
    """``gate_up`` ``[E, 2F, H]`` -> rows of this rank's part of gate and of up; ``down`` ``[E, H, F]`` -> its columns."""
    if kind == "gate_up":
        F = full.shape[1] // 2
        n = F // size
        return torch.cat([full[:, rank * n:(rank + 1) * n], full[:, F + rank * n:F + (rank + 1) * n]], dim=1)
    if kind == "down":
        n = full.shape[2] // size
        return full[:, :, rank * n:(rank + 1) * n]
    raise ValueError(f"unknown expert bank kind {kind!r}")


def unslice_expert_bank(kind: str, parts: list[torch.Tensor]) -> torch.Tensor:
    if kind == "gate_up":
        gs, us = zip(*(p.chunk(2, dim=1) for p in parts))
        return torch.cat(list(gs) + list(us), dim=1)
    if kind == "down":
        return torch.cat(parts, dim=2)
    raise ValueError(f"unknown expert bank kind {kind!r}")
