"""Training step of one pipeline stage: the micro-batches of a step run on the 1F1B (or GPipe) schedule, the global
gradient norm is assembled over the stages (each stage owns different parameters), every stage clips with the same
coefficient and steps its own optimizer, and the last stage's loss reaches every stage for logging
(halo/trainers/parallelism/pipeline_trainer.py, halo/distributed/pipeline_parallel/runner.py:183-191)."""

from __future__ import annotations

import torch
import torch.distributed as dist

from halo_b200.optim.adamw_bf16 import GradNorm
from halo_b200.parallel.pipeline import PipelineStage, broadcast_loss, run_schedule
from halo_b200.trainers.engine import StepOutput


class PipelineEngine:
    def __init__(self, stage: PipelineStage, optimizer, max_grad_norm: float = 1.0, schedule: str = "1f1b",
                 lr_scheduler=None, dp_group=None):
        self.stage, self.optimizer, self.max_grad_norm, self.schedule = stage, optimizer, max_grad_norm, schedule
        self.lr_scheduler, self.dp_group = lr_scheduler, dp_group
        self.device = stage.device
        self.grad_norm = GradNorm(self.device)
        self.step_count = 0

    def train_step(self, micro_batches: list) -> StepOutput:
        """Every stage is handed the same micro-batches (token ids matter on the first stage, labels on the last,
        positions and document boundaries everywhere)."""
        model = self.stage.model
        normalizer = float(max(1, sum(b.n_scored for b in micro_batches)))
        if self.device.type == "cuda":
            micro_batches = [b.to(self.device) for b in micro_batches]
        loss = broadcast_loss(self.stage, run_schedule(self.stage, micro_batches, normalizer, self.schedule))
        params = [p for p in model.parameters() if p.grad is not None]
        if self.dp_group is not None:                      # replicas of this stage
            for p in params:
                dist.all_reduce(p.grad, group=self.dp_group)
        self.grad_norm.accumulate([p.grad for p in params], first=True)
        dist.all_reduce(self.grad_norm.total_sq, group=self.stage.group)       # stages own disjoint parameters
        self.grad_norm.finish(self.max_grad_norm)
        if hasattr(self.optimizer, "defer_grad_scale"):
            self.optimizer.defer_grad_scale(self.grad_norm.coef)
            self.optimizer.arm_skip(self.grad_norm.skip)
        else:
            keep = (self.grad_norm.skip == 0).to(torch.float32)
            coef = torch.nan_to_num(self.grad_norm.coef * keep, nan=0.0)
            for p in params:
                p.grad.nan_to_num_(nan=0.0, posinf=0.0, neginf=0.0).mul_(coef.to(p.grad.dtype))
        self.optimizer.step()
        if self.lr_scheduler is not None:
            self.lr_scheduler.step()
        self.optimizer.zero_grad(set_to_none=True)
        self.step_count += 1
        return StepOutput(loss, self.grad_norm.norm, self.grad_norm.skip, sum(b.n_tokens for b in micro_batches))
