"""The training step: host batch -> device, forward + fused loss, backward, gradient
synchronisation, device-side global-norm clip / non-finite guard, optimizer step.

``TrainEngine`` is the seam every trainer (SFT, preference, distillation, GRPO ...) drives; it owns
nothing method-specific. A step never reads the device: the clip coefficient and the skip flag stay
in device memory and are consumed by the optimizer kernel; the caller decides when to read the loss.

Counterpart of the reference's trainer spine around ``training_step`` / ``clip_grad_norm_`` /
``optimizer.step`` (halo/trainers/distributed_trainer.py:591-618,
halo/trainers/parallelism/grad_clipping.py:125-147, halo/trainers/loop/step_guard.py:104-131).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

import torch

from halo_b200.data.packing import PackedBatch
from halo_b200.optim.adamw_bf16 import GradNorm


@dataclass
class StepOutput:
    loss: torch.Tensor                 # device scalar (mean CE over the globally scored tokens)
    grad_norm: torch.Tensor            # device scalar
    skipped: torch.Tensor              # device int32 flag: the update was skipped (non-finite norm)
    n_tokens: int = 0
    extras: dict = field(default_factory=dict)


class TrainEngine:
    def __init__(self, model, optimizer, device, max_grad_norm: float = 1.0, parallel=None, lr_scheduler=None,
                 loss_fn: Callable | None = None):
        self.model = model
        self.optimizer = optimizer
        self.device = torch.device(device)
        self.max_grad_norm = max_grad_norm
        self.parallel = parallel          # halo_b200.parallel.runtime.ParallelRuntime or None
        self.lr_scheduler = lr_scheduler
        self.loss_fn = loss_fn
        self.grad_norm = GradNorm(self.device)
        self.step_count = 0
        self.consecutive_skips = 0
        # a device int32 flag a trainer may set before the optimizer step: non-zero on any rank skips this update on
        # every rank (consumed and cleared by the step)
        self.skip_request: torch.Tensor | None = None
        self.last_skip_was_requested: torch.Tensor | None = None
        if hasattr(optimizer, "wait_ready") and hasattr(model, "param_gate"):
            model.param_gate = optimizer.wait_ready

    # ---- pieces ---------------------------------------------------------------------------
    def to_device(self, batch: PackedBatch) -> PackedBatch:
        return batch.to(self.device, non_blocking=True) if self.device.type == "cuda" else batch

    def global_scored_tokens(self, batch: PackedBatch):
        """Normaliser shared by every data-parallel rank so that summed gradients average correctly."""
        if self.parallel is not None and self.parallel.dp_world > 1:
            return self.parallel.sum_scalar_over_dp(float(batch.n_scored))
        return float(max(batch.n_scored, 1))

    def compute_loss(self, dbatch: PackedBatch, normalizer):
        if self.loss_fn is not None:
            return self.loss_fn(self.model, dbatch, normalizer)
        return self.model(dbatch.input_ids, dbatch.position_ids, dbatch.cu_seqlens, dbatch.labels, normalizer)

    def _fused_clip_and_step(self, fused) -> None:
        """Replicated parameters go through the fused reduce-scatter / AdamW / all-gather kernels, the
        experts through the ordinary optimizer; one scalar all-reduce assembles the global norm."""
        import torch.distributed as dist

        shard_sq = fused.pack_and_reduce()
        experts = [p for p in self.model.parameters() if p.grad is not None and getattr(p, "is_expert", False)]
        self.grad_norm.accumulate([p.grad for p in experts], first=True)
        self.grad_norm.total_sq.add_(shard_sq)
        dist.all_reduce(self.grad_norm.total_sq, group=self.parallel.dp_group)
        self.grad_norm.finish(self.max_grad_norm)
        self._apply_skip_request()
        self.optimizer.defer_grad_scale(self.grad_norm.coef)
        self.optimizer.arm_skip(self.grad_norm.skip)
        self.optimizer.step()
        fused.step(self.grad_norm.coef, self.grad_norm.skip)
        if self.lr_scheduler is not None:
            self.lr_scheduler.step()
            fused.lr = self.optimizer.param_groups[0]["lr"]
        self.optimizer.zero_grad(set_to_none=True)
        fused.zero_grad()

    def _apply_skip_request(self) -> None:
        """Fold a trainer's skip request into the step's skip flag (after the gradient norm set it)."""
        req, self.skip_request = self.skip_request, None
        if req is None:
            return
        req = req.to(self.grad_norm.skip.dtype).reshape(self.grad_norm.skip.shape)
        if self.parallel is not None and self.parallel.dp_world > 1:
            import torch.distributed as dist

            dist.all_reduce(req, op=dist.ReduceOp.MAX, group=self.parallel.dp_group)
        self.grad_norm.skip.copy_(torch.maximum(self.grad_norm.skip, req))
        self.last_skip_was_requested = req

    def clip_and_step(self) -> None:
        fused = getattr(self.parallel, "fused_optimizer", None) if self.parallel is not None else None
        if fused is not None:
            return self._fused_clip_and_step(fused)
        params = [p for p in self.model.parameters() if p.grad is not None]
        zero3 = getattr(self.model, "zero3", None)
        if zero3 is not None:
            zero3.before_step()              # collective: nobody reads this rank's slices any more
        if self.parallel is not None:
            self.parallel.sync_gradients(self.model)
            self.parallel.global_grad_sq_norm(self.model, self.grad_norm)
        else:
            self.grad_norm.accumulate([p.grad for p in params], first=True)
        self.grad_norm.finish(self.max_grad_norm)
        self._apply_skip_request()
        if hasattr(self.optimizer, "defer_grad_scale"):
            self.optimizer.defer_grad_scale(self.grad_norm.coef)
            self.optimizer.arm_skip(self.grad_norm.skip)
        else:
            # a stock optimizer: apply the (device-resident) clip coefficient in place; a non-finite
            # norm zeroes the update by zeroing the gradients
            keep = (self.grad_norm.skip == 0).to(torch.float32)
            coef = torch.nan_to_num(self.grad_norm.coef * keep, nan=0.0)
            for p in params:
                p.grad.nan_to_num_(nan=0.0, posinf=0.0, neginf=0.0).mul_(coef.to(p.grad.dtype))
        self.optimizer.step()
        if self.lr_scheduler is not None:
            self.lr_scheduler.step()
        self.optimizer.zero_grad(set_to_none=True)
        if zero3 is not None:
            zero3.after_step()               # collective: every rank's slices hold the new values

    # ---- the step -------------------------------------------------------------------------
    def train_step(self, batch: PackedBatch, accumulate: bool = False) -> StepOutput:
        """One micro-batch forward/backward; unless ``accumulate``, also clip + optimizer step."""
        if self.parallel is not None and (self.parallel.context_parallel is not None or self.parallel.tensor_parallel is not None):
            batch = self.parallel.slice_batch(batch)      # this rank's tokens of the row, cut before the copy
        dbatch = self.to_device(batch)
        normalizer = self.global_scored_tokens(batch)
        loss = self.compute_loss(dbatch, normalizer)
        loss.backward()
        if not accumulate:
            self.clip_and_step()
            self.step_count += 1
        requested, self.last_skip_was_requested = self.last_skip_was_requested, None
        return StepOutput(loss.detach(), self.grad_norm.norm, self.grad_norm.skip, batch.n_tokens,
                          {} if requested is None else {"requested_skip": requested})

    @torch.no_grad()
    def eval_step(self, batch: PackedBatch) -> torch.Tensor:
        dbatch = self.to_device(batch)
        return self.compute_loss(dbatch, float(max(batch.n_scored, 1))).detach()
