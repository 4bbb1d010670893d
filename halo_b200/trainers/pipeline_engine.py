"""Training step of one pipeline stage: the micro-batches of a step run on the 1F1B (or GPipe) schedule, the global
gradient norm is assembled over the stages (each stage owns different parameters) and over the stage's replicas
(data parallel, with the experts sharded over them under expert parallelism), every stage clips with the same
coefficient and steps its own optimizer, and the last stage's loss reaches every stage for logging
(halo/trainers/parallelism/pipeline_trainer.py, halo/distributed/pipeline_parallel/runner.py:183-215).

``PipelineEngine.train_step(batch, accumulate)`` has the signature of :class:`halo_b200.trainers.engine.TrainEngine`, so
the trainer spine drives either: micro-batches are collected while ``accumulate`` is set and the whole schedule runs
on the last one."""

from __future__ import annotations

import torch
import torch.distributed as dist

from halo_b200.optim.adamw_bf16 import GradNorm
from halo_b200.parallel.pipeline import PipelineStage, broadcast_loss, run_schedule
from halo_b200.trainers.engine import StepOutput


class PipelineEngine:
    returns_step_total = True      # the call that runs the schedule returns the whole step's loss; the others return zero

    def __init__(self, stage: PipelineStage, optimizer, max_grad_norm: float = 1.0, schedule: str = "1f1b",
                 lr_scheduler=None, dp_group=None, parallel=None, min_microbatches: int = 0):
        """``parallel``: the :class:`ParallelRuntime` of this stage's replicas (data parallel over ``dp_group``, experts
        sharded over its expert-parallel group); None on a pipeline without replicas. ``min_microbatches``: a 1F1B
        schedule needs at least as many micro-batches as stages to fill the pipe; a step that brings fewer is refused."""
        self.stage, self.optimizer, self.max_grad_norm, self.schedule = stage, optimizer, max_grad_norm, schedule
        self.lr_scheduler = lr_scheduler
        self.parallel = parallel
        self.dp_group = dp_group if dp_group is not None else (parallel.dp_group if parallel is not None else None)
        self.model = stage.model
        self.device = stage.device
        self.grad_norm = GradNorm(self.device)
        self.step_count = 0
        self.min_microbatches = min_microbatches
        self.skip_request = None
        self._held: list = []

    # ---- the TrainEngine seam ---------------------------------------------------------------------
    def train_step(self, batch, accumulate: bool = False) -> StepOutput:
        """One micro-batch (a list runs at once). While ``accumulate`` is set the micro-batch is only kept; the call
        without it runs the schedule over everything kept so far, clips and steps."""
        if isinstance(batch, (list, tuple)):
            return self.run_microbatches(list(batch))
        self._held.append(batch)
        if accumulate:
            zero = torch.zeros((), device=self.device)
            return StepOutput(zero, self.grad_norm.norm, self.grad_norm.skip, batch.n_tokens)
        held, self._held = self._held, []
        return self.run_microbatches(held)

    @torch.no_grad()
    def eval_step(self, batch) -> torch.Tensor:
        """Loss of one micro-batch through the stages (forward only), on every stage."""
        from halo_b200.parallel.pipeline import forward_only

        b = batch.to(self.device) if self.device.type == "cuda" else batch
        return broadcast_loss(self.stage, forward_only(self.stage, b, float(max(b.n_scored, 1))))

    def _global_scored(self, micro_batches) -> float:
        n = float(sum(b.n_scored for b in micro_batches))
        if self.dp_group is not None and dist.get_world_size(self.dp_group) > 1:
            t = torch.tensor([n], dtype=torch.float64, device=self.device)
            dist.all_reduce(t, group=self.dp_group)
            n = float(t.item())
        return max(n, 1.0)

    def run_microbatches(self, micro_batches: list) -> StepOutput:
        """Every stage of a chain is handed the same micro-batches (token ids matter on the first stage, labels on the
        last, positions and document boundaries everywhere)."""
        if self.schedule == "1f1b" and len(micro_batches) < max(self.min_microbatches, 1):
            raise ValueError(f"a 1F1B step over {self.stage.n_stages} stages needs at least {self.min_microbatches} "
                             f"micro-batches, got {len(micro_batches)}: raise gradient_accumulation_steps or pipeline_microbatches")
        model = self.model
        normalizer = self._global_scored(micro_batches)
        if self.device.type == "cuda":
            micro_batches = [b.to(self.device) for b in micro_batches]
        loss = broadcast_loss(self.stage, run_schedule(self.stage, micro_batches, normalizer, self.schedule))
        params = [p for p in model.parameters() if p.grad is not None]
        if self.parallel is not None:
            # replicas of this stage: replicated parameters are summed over them, expert shards are not; the squares of
            # both kinds are counted once each
            self.parallel.sync_gradients(model)
            self.parallel.global_grad_sq_norm(model, self.grad_norm)
        else:
            if self.dp_group is not None:
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
