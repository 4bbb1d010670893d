"""The trainer spine shared by every method: optimizer / scheduler construction, the accumulation
loop over packed batches, logging through callbacks, the non-finite step guard, periodic saves
(weights -> optimizer shards -> scheduler / RNG sidecars -> ``trainer_state.json`` last) and exact
resume from the newest complete checkpoint.

Method trainers (SFT, preference, reward, distillation, GRPO) subclass :class:`Trainer` and
override ``compute_loss`` (and, for RL, ``next_batches``); the parallel layout never leaks into
them. Counterpart of the reference's ``DistributedTrainerMixin`` and its loop helpers
(halo/trainers/distributed_trainer.py:175-684, halo/trainers/loop/checkpointing.py,
halo/trainers/loop/step_guard.py, halo/checkpoint/parallel/resume_source.py).
"""

from __future__ import annotations

import logging
import os
import re
import shutil
import time
from typing import Callable, Iterable, Iterator

import torch

from halo_b200.checkpoint import optimizer_state as opt_io
from halo_b200.checkpoint.atomic import atomic_torch_save, atomic_write_json
from halo_b200.checkpoint.save import is_complete, mark_complete, save_model
from halo_b200.configs.arguments import TrainingArguments
from halo_b200.data.packing import PackedBatch
from halo_b200.optim.factory import build_optimizer
from halo_b200.optim.schedule import LRScheduler
from halo_b200.trainers.engine import TrainEngine

log = logging.getLogger(__name__)
CHECKPOINT_RE = re.compile(r"^checkpoint-(\d+)$")


class NonFiniteRun(RuntimeError):
    """Too many consecutive steps had a non-finite gradient norm."""


class Callback:
    def on_train_begin(self, trainer): ...
    def on_batch(self, trainer, batch): ...
    def on_step_end(self, trainer, logs: dict): ...
    def on_log(self, trainer, logs: dict): ...
    def on_save(self, trainer, directory: str): ...
    def on_train_end(self, trainer): ...


def list_checkpoints(output_dir: str) -> list[tuple[int, str]]:
    out = []
    if os.path.isdir(output_dir):
        for name in os.listdir(output_dir):
            m = CHECKPOINT_RE.match(name)
            if m:
                out.append((int(m.group(1)), os.path.join(output_dir, name)))
    return sorted(out)


def newest_complete_checkpoint(output_dir: str) -> str | None:
    """The newest checkpoint whose completeness marker exists (an interrupted save is skipped)."""
    for _, path in reversed(list_checkpoints(output_dir)):
        if is_complete(path):
            return path
    return None


class Trainer:
    def __init__(self, model, args: TrainingArguments, train_batches: Iterable[PackedBatch] | Callable[[], Iterator],
                 eval_batches: Iterable[PackedBatch] | None = None, device=None, parallel=None,
                 callbacks: list[Callback] | None = None, optimizer=None, parallelism_fingerprint: dict | None = None):
        if isinstance(parallel, dict):
            # a pipeline rank is handed its stage's description; the runtime of the stage's replicas is one field of it
            parallel = parallel.get("parallel")
        self.model, self.args, self.parallel = model, args, parallel
        self.device = torch.device(device or next(model.parameters()).device)
        self.train_batches, self.eval_batches = train_batches, eval_batches
        self.callbacks = list(callbacks or [])
        self.optimizer = optimizer or build_optimizer(
            model, args.optim if self.device.type == "cuda" or args.optim == "adamw_torch" else
            ("adamw_bf16" if next(model.parameters()).dtype == torch.bfloat16 else "adamw_torch"),
            lr=args.learning_rate, weight_decay=args.weight_decay, betas=(args.adam_beta1, args.adam_beta2),
            eps=args.adam_epsilon)
        total = args.max_steps if args.max_steps > 0 else 0
        warmup = args.warmup_steps or int(args.warmup_ratio * total)
        self.lr_scheduler = LRScheduler(self.optimizer, args.lr_scheduler_type, total, warmup)
        spec = getattr(model, "parallel_runtime", None)
        if isinstance(spec, dict) and spec.get("kind") == "pp":
            # a pipeline stage: the step is a schedule over the step's micro-batches, run by the stage's own engine (the
            # next-token loss lives on the last stage; objectives that need more than that are refused by the rules)
            from halo_b200.entrypoints.script import finish_pipeline_runtime

            if type(self).compute_loss is not Trainer.compute_loss and not getattr(self, "pipeline_ready", False):
                raise ValueError(f"{type(self).__name__} computes its own loss; under pipeline parallelism only the "
                                 "next-token objective (SFT / pre-training) runs")
            self.parallel = spec["parallel"]
            self.engine = finish_pipeline_runtime(spec, model, self.optimizer, row_len=spec.get("row_len", 0) or self._row_len(),
                                                  max_grad_norm=args.max_grad_norm, lr_scheduler=self.lr_scheduler)
            pc = spec["pc"]
            args.gradient_accumulation_steps = pc.pp_microbatch_count(args.gradient_accumulation_steps)
        else:
            self.engine = TrainEngine(model, self.optimizer, self.device, args.max_grad_norm, parallel, self.lr_scheduler,
                                      loss_fn=self._loss_adapter)
        self.global_step = 0
        self.tokens_seen = 0
        self.fingerprint = parallelism_fingerprint or {"world_size": self.world_size}
        self.log_history: list[dict] = []
        self._pending_skip = None
        self._consecutive_skips = 0
        self.collective_group = None      # set by a job whose ranks are not all trainers (split trainer / rollout roles)
        self.rank = int(os.environ.get("RANK", "0"))
        if parallel is not None and parallel.dp_group is not None:
            import torch.distributed as dist

            self.rank = dist.get_rank(parallel.dp_group)   # rank among the trainers of the job

    def _row_len(self) -> int:
        """Tokens per packed row of the training stream (pipeline messages have one fixed shape)."""
        src = self.train_batches() if callable(self.train_batches) else self.train_batches
        first = next(iter(src))
        first = first[0] if isinstance(first, (list, tuple)) else first
        return int(first.n_tokens)

    # ---- hooks for subclasses --------------------------------------------------------------
    def compute_loss(self, model, batch: PackedBatch, normalizer):
        return model(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels, normalizer)

    # True on trainers whose compute_loss returns the MEAN over this rank's sequences (pairs, documents): gradients are
    # summed over the data-parallel ranks, so such a loss is re-weighted to its share of the global mean
    sequence_mean_loss = False

    def _loss_adapter(self, model, batch, normalizer):
        loss = self.compute_loss(model, batch, normalizer)
        if self.sequence_mean_loss and self.parallel is not None and self.parallel.dp_world > 1:
            n_local = float(max(len(batch.cu_seqlens) - 1, 1))
            n_global = self.parallel.sum_scalar_over_dp(n_local)          # device scalar, one tiny reduction
            loss = loss * (n_local / n_global.to(loss.dtype).reshape(()))
        return loss

    def after_optimizer_step(self) -> None:
        """Hook for trainers that act on fresh weights (pushing them to a rollout copy, say)."""

    def next_batches(self) -> Iterator[PackedBatch]:
        """The training stream. An item is either one micro-batch (``gradient_accumulation_steps`` of them make an
        optimizer step) or a LIST of micro-batches that together make exactly one optimizer step (a source whose
        steps have a varying number of micro-batches, such as a GRPO round, yields those)."""
        src = self.train_batches() if callable(self.train_batches) else self.train_batches
        return iter(src)

    def skip_consumed(self, it: Iterator) -> Iterator:
        """A resumed run passes over what the interrupted run consumed: ``global_step`` optimizer steps' worth of
        single micro-batches. Sources that yield whole steps override this."""
        for _ in range(self.global_step * self.args.gradient_accumulation_steps):
            next(it, None)
        return it

    def step_groups(self, it: Iterator) -> Iterator[tuple[list, bool]]:
        """The micro-batches of one optimizer step at a time, with a flag: True when the source delivered the step
        as one list (its micro-batch losses share one denominator and add up to the step's loss), False when the
        step was assembled from ``gradient_accumulation_steps`` independent micro-batches (the step's loss is their
        mean). The accumulation count is read per step, before the step's first micro-batch is consumed."""
        while True:
            first = next(it, None)
            if first is None:
                return
            if isinstance(first, (list, tuple)):
                if first:
                    yield list(first), True
                continue
            micro = [first]
            for _ in range(self.args.gradient_accumulation_steps - 1):
                b = next(it, None)
                if b is None:
                    break
                micro.append(b)
            yield micro, False

    @property
    def world_size(self) -> int:
        if self.parallel is not None and self.parallel.dp_group is not None:
            import torch.distributed as dist

            return dist.get_world_size(self.parallel.dp_group)
        return int(os.environ.get("WORLD_SIZE", "1"))

    @property
    def group(self):
        """The ranks that take part in this trainer's collectives (None = the whole job)."""
        if self.collective_group is not None:
            return self.collective_group
        return self.parallel.dp_group if self.parallel is not None else None

    @property
    def is_main(self) -> bool:
        return self.rank == 0

    # ---- the loop --------------------------------------------------------------------------
    def train(self, resume_from_checkpoint: str | None = None) -> dict:
        args = self.args
        resume = resume_from_checkpoint if resume_from_checkpoint is not None else args.resume_from_checkpoint
        if resume == "auto":
            resume = newest_complete_checkpoint(args.output_dir)
        if resume:
            self.load_checkpoint(resume)
        for cb in self.callbacks:
            cb.on_train_begin(self)
        it = self.step_groups(self.skip_consumed(self.next_batches()))
        t_last = time.perf_counter()
        while True:
            group = next(it, None)
            if group is None:
                break
            micro, shares = group
            out, step_loss = None, None
            for i, b in enumerate(micro):
                out = self.engine.train_step(b, accumulate=i < len(micro) - 1)
                # every micro-batch's loss is its share of the step's loss (one shared denominator)
                step_loss = out.loss if step_loss is None else step_loss + out.loss
                self.tokens_seen += b.n_tokens
                for cb in self.callbacks:
                    on_batch = getattr(cb, "on_batch", None)
                    if on_batch is not None:
                        on_batch(self, b)
            if not shares and not getattr(self.engine, "returns_step_total", False):
                step_loss = step_loss / len(micro)
            self.global_step += 1
            self.after_optimizer_step()
            self._guard_non_finite(out)
            if args.logging_steps and self.global_step % args.logging_steps == 0:
                now = time.perf_counter()
                # every rank's loss is its share of the step's global loss (one shared denominator): the logged number is
                # their sum, whatever the layout (every rank reaches this line at the same steps)
                step_loss = step_loss.detach().reshape(-1)[:1].float().clone()
                if self.parallel is not None and getattr(self.parallel, "dp_world", 1) > 1:
                    import torch.distributed as dist

                    dist.all_reduce(step_loss, group=self.parallel.dp_group)
                logs = {"step": self.global_step, "loss": float(step_loss.reshape(-1)[0].item()),
                        "grad_norm": float(out.grad_norm.item()), "lr": self.lr_scheduler.get_last_lr()[0],
                        "tokens": self.tokens_seen, "step_seconds": (now - t_last) / args.logging_steps}
                t_last = now
                logs.update(self.extra_logs())
                self.log_history.append(logs)
                for cb in self.callbacks:
                    cb.on_log(self, logs)
                if self.is_main:
                    extras = "".join(f" {k} {v:.4g}" for k, v in logs.items() if k not in
                                     ("step", "loss", "grad_norm", "lr", "tokens", "step_seconds") and isinstance(v, (int, float)))
                    log.info("step %d loss %.4f grad_norm %.3f lr %.3g%s", logs["step"], logs["loss"], logs["grad_norm"], logs["lr"],
                             extras)
            for cb in self.callbacks:
                cb.on_step_end(self, {"step": self.global_step})
            if args.save_steps and self.global_step % args.save_steps == 0:
                self.save_checkpoint()
            if args.eval_steps and self.eval_batches is not None and self.global_step % args.eval_steps == 0:
                self.evaluate()
            if 0 < args.max_steps <= self.global_step:
                break
        for cb in self.callbacks:
            cb.on_train_end(self)
        return {"global_step": self.global_step, "log_history": self.log_history}

    def extra_logs(self) -> dict:
        """Method-specific scalars added to every log record."""
        return {}

    def _guard_non_finite(self, out) -> None:
        """The skip flag of a step is read one step late, so the read never stalls the step it guards."""
        prev, prev_requested = self._pending_skip, getattr(self, "_pending_requested", None)
        self._pending_skip = out.skipped.clone() if out is not None else None
        self._pending_requested = out.extras.get("requested_skip") if out is not None else None
        if prev is not None and prev_requested is not None and int(prev_requested.item()):
            log.warning("step %d was skipped on the trainer's request (trust-region breaker)", self.global_step - 1)
        elif prev is not None and int(prev.item()):
            self._consecutive_skips += 1
            log.warning("step %d was skipped: non-finite gradient norm", self.global_step - 1)
            if self._consecutive_skips >= self.args.max_consecutive_nonfinite_steps:
                raise NonFiniteRun(f"{self._consecutive_skips} consecutive steps had a non-finite gradient norm")
        elif prev is not None:
            self._consecutive_skips = 0

    @torch.no_grad()
    def evaluate(self) -> dict:
        losses = [float(self.engine.eval_step(b).reshape(-1)[0].item()) for b in self.eval_batches]
        logs = {"step": self.global_step, "eval_loss": sum(losses) / max(1, len(losses))}
        self.log_history.append(logs)
        for cb in self.callbacks:
            cb.on_log(self, logs)
        return logs

    # ---- save / resume ---------------------------------------------------------------------
    def checkpoint_dir(self, step: int | None = None) -> str:
        return os.path.join(self.args.output_dir, f"checkpoint-{self.global_step if step is None else step}")

    def save_checkpoint(self) -> str:
        d = self.checkpoint_dir()
        # the free-space check runs on the writer rank only, but its verdict is agreed over the group BEFORE any rank
        # enters the collective gathers of save_model: a lone raise there would leave the others waiting in them
        reason = None
        if self.is_main:
            from halo_b200.checkpoint.preflight import checkpoint_bytes, require_free_space

            ep_world = self.parallel.ep_world if self.parallel is not None else 1
            try:
                require_free_space(self.args.output_dir, checkpoint_bytes(self.model, ep_world=ep_world))
            except Exception as exc:  # noqa: BLE001 - any failure of the check must reach every rank
                reason = f"{type(exc).__name__}: {exc}"
        if self.parallel is not None or self.collective_group is not None:
            from halo_b200.runtime.consensus import reject_across_ranks

            reject_across_ranks(reason, group=self.group, what="checkpoint preflight")
        elif reason is not None:
            raise RuntimeError(f"checkpoint preflight: {reason}")
        os.makedirs(d, exist_ok=True)
        save_model(self.model, d, sharded_experts=self.args.save_sharded_ep, save_dtype=None,
                   group=self.group)  # exact resume: keep the dtype
        opt_io.save_optimizer_shard(self.optimizer, d, self.rank, self.fingerprint, write_meta=self.is_main)
        atomic_torch_save({"cpu": torch.get_rng_state(),
                           "cuda": torch.cuda.get_rng_state(self.device) if self.device.type == "cuda" else None},
                          os.path.join(d, f"rng_state_{self.rank}.pth"))
        if self.parallel is not None or self.collective_group is not None:
            import torch.distributed as dist

            dist.barrier(group=self.group)
        if self.is_main:
            atomic_torch_save(self.lr_scheduler.state_dict(), os.path.join(d, "scheduler.pt"))
            mark_complete(d, {"global_step": self.global_step, "tokens_seen": self.tokens_seen,
                              "log_history": self.log_history[-50:], "world_size": self.world_size})
            self._rotate()
        for cb in self.callbacks:
            cb.on_save(self, d)
        return d

    def _rotate(self) -> None:
        limit = self.args.save_total_limit
        if limit and limit > 0:
            done = [p for _, p in list_checkpoints(self.args.output_dir) if is_complete(p)]
            for p in done[:-limit]:
                shutil.rmtree(p, ignore_errors=True)

    def load_checkpoint(self, directory: str) -> None:
        import json

        from halo_b200.checkpoint.load import load_model_weights

        if not is_complete(directory):
            raise FileNotFoundError(f"{directory!r} has no completeness marker: the save was interrupted")
        if getattr(self.model, "lora_spec", None) is not None:
            from halo_b200.peft.lora import load_adapters      # the frozen base came from the model path

            load_adapters(self.model, directory)
        else:
            load_model_weights(self.model, directory)
        opt_io.load_optimizer_shard(self.optimizer, directory, self.rank, self.fingerprint,
                                    self.args.allow_optimizer_warm_restart)
        state = json.load(open(os.path.join(directory, "trainer_state.json")))
        self.global_step, self.tokens_seen = state["global_step"], state.get("tokens_seen", 0)
        sched = os.path.join(directory, "scheduler.pt")
        if os.path.isfile(sched):
            self.lr_scheduler.load_state_dict(torch.load(sched, weights_only=False))
        rng = os.path.join(directory, f"rng_state_{self.rank}.pth")
        if os.path.isfile(rng):
            blob = torch.load(rng, weights_only=False)
            torch.set_rng_state(blob["cpu"])
            if blob.get("cuda") is not None and self.device.type == "cuda":
                torch.cuda.set_rng_state(blob["cuda"], self.device)
        self.engine.step_count = self.global_step
