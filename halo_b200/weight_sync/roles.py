"""Trainer and rollout roles inside one job.

The last ``rollout_gpus`` ranks of the job hold a serving copy of the policy and take no part in
training; the others train. After an optimizer step the trainers gather the expert banks to the
forwarding rank (trainer rank 0), which announces a push with a one-integer control broadcast and then
moves the packed weights into every rollout rank (peer stores into the rollout ranks' arena on CUDA,
a packed broadcast on CPU). A control value of 0 ends the rollout ranks' loop.

The reference runs the rollout side as separate vLLM / SGLang servers fed by NCCL broadcasts behind an
HTTP control plane (halo/weight_sync/clients/base.py:126, halo/trainers/grpo/rollout/weight_push.py);
here both sides are ranks of one launcher, so control and payload share the job's process group.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from .group import BroadcastSync, ResidentCopySync, full_named_tensors

PUSH, STOP = 1, 0


@dataclass
class Roles:
    trainer_ranks: list[int]
    rollout_ranks: list[int]
    trainer_group: object
    is_trainer: bool
    rank: int

    @property
    def src_rank(self) -> int:
        return self.trainer_ranks[0]


def split_roles(rollout_gpus: int) -> Roles:
    """COLLECTIVE over the job: every rank creates the trainer subgroup."""
    world, rank = dist.get_world_size(), dist.get_rank()
    if not 0 < rollout_gpus < world:
        raise ValueError(f"rollout_gpus={rollout_gpus} must leave at least one trainer among {world} ranks")
    trainers = list(range(world - rollout_gpus))
    rollouts = list(range(world - rollout_gpus, world))
    return Roles(trainers, rollouts, dist.new_group(trainers), rank in trainers, rank)


def make_sync(roles: Roles, device, manifest, chunk_bytes: int | None = None):
    """COLLECTIVE over the job. Peer-store path on CUDA, packed broadcast elsewhere."""
    if torch.device(device).type == "cuda":
        return ResidentCopySync(dist.group.WORLD, device, manifest, roles.src_rank, roles.rollout_ranks, chunk_bytes)
    return BroadcastSync(dist.group.WORLD, device, manifest, roles.src_rank, chunk_bytes)


def _control(value: int, roles: Roles, device) -> int:
    t = torch.tensor([value], dtype=torch.int32, device=device)
    dist.broadcast(t, src=roles.src_rank)
    return int(t.item())


class ModelWeightPusher:
    """What the trainer calls after an optimizer step (``push(model)``) and at the end (``close()``)."""

    def __init__(self, sync, roles: Roles, device, ep_group=None):
        self.sync, self.roles, self.device, self.ep_group = sync, roles, torch.device(device), ep_group
        self.pushes = 0
        self.parity_tolerance = 0.0       # > 0: after the first push, compare one fixed row's scores with the rollout copy's
        self.parity_gap = None

    def push(self, model) -> None:
        gathered = dict(full_named_tensors(model, self.ep_group))    # collective over the trainers
        _control(PUSH, self.roles, self.device)
        self.sync.push(gathered if self.roles.rank == self.roles.src_rank else None)
        self.pushes += 1
        if self.pushes == 1 and self.parity_tolerance > 0:
            from . import parity

            mine = parity.score_fixed_row(model, self.device)           # collective over the trainers under expert parallelism
            if self.roles.rank == self.roles.src_rank:
                self.parity_gap = parity.compare(dist.distributed_c10d._get_default_store(), mine, self.parity_tolerance)

    def close(self) -> None:
        _control(STOP, self.roles, self.device)


def rollout_loop(sync, roles: Roles, device, serving_params: dict, on_update=None) -> int:
    """Run on a rollout rank until the trainers close the pusher. Returns the number of updates applied."""
    updates = 0
    while _control(STOP, roles, device) == PUSH:
        if isinstance(sync, BroadcastSync):
            sync.push(None, into=serving_params)
        else:
            sync.push(None)
            sync.receive_into(serving_params)
        updates += 1
        if on_update is not None:
            on_update(updates)
    return updates
