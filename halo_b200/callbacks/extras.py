"""Smaller callbacks of the roster: torch profiler schedule, parameter statistics, variable schedules, early stop,
the recomputation plan (halo/callbacks/{torch_profiler,parameter_stats,variable_scheduler,early_stop,
gradient_checkpointing_plan}.py) and the factory that builds a run's callbacks from its arguments
(halo/callbacks/factory.py:28-103)."""

from __future__ import annotations

import math

import torch

from halo_b200.diagnostics.profiling import make_profiler
from halo_b200.trainers.base import Callback


class TorchProfilerCallback(Callback):
    """Steps a ``torch.profiler`` schedule (wait 5, warm-up 1, active 3) on the selected ranks."""

    def __init__(self, rank: int = 0, ranks: str = "0", world: int = 1, out_dir: str | None = None):
        self.prof = make_profiler(rank, ranks, world, out_dir=out_dir)

    def on_train_begin(self, trainer):
        if self.prof is not None:
            self.prof.__enter__()

    def on_step_end(self, trainer, logs):
        if self.prof is not None:
            self.prof.step()

    def on_train_end(self, trainer):
        if self.prof is not None:
            self.prof.__exit__(None, None, None)
            self.prof = None


class ParameterStatsCallback(Callback):
    """Every ``every`` logs: global weight norm and the largest absolute weight, computed on the device and read
    once (non-finite weights raise on the spot: the run cannot recover from them)."""

    def __init__(self, every: int = 10):
        self.every, self._n = every, 0

    def on_log(self, trainer, logs):
        self._n += 1
        if self._n % self.every:
            return
        sq = torch.zeros((), dtype=torch.float32, device=trainer.device)
        mx = torch.zeros((), dtype=torch.float32, device=trainer.device)
        for p in trainer.model.parameters():
            pf = p.detach().float()
            sq += pf.pow(2).sum()
            mx = torch.maximum(mx, pf.abs().max())
        norm, biggest = float(sq.sqrt()), float(mx)
        if not (math.isfinite(norm) and math.isfinite(biggest)):
            raise FloatingPointError("the model's weights are no longer finite")
        logs.update({"weights/norm": norm, "weights/max_abs": biggest})


class VariableSchedulerCallback(Callback):
    """Piecewise-linear schedules of scalar attributes of the trainer's argument objects, e.g.
    ``{"pref.beta": [(0, 0.1), (1000, 0.5)]}`` ramps ``trainer.pref.beta`` from 0.1 to 0.5 over 1000 steps."""

    def __init__(self, schedules: dict[str, list[tuple[int, float]]]):
        self.schedules = {k: sorted(v) for k, v in schedules.items()}

    @staticmethod
    def value_at(points, step: int) -> float:
        if step <= points[0][0]:
            return points[0][1]
        for (s0, v0), (s1, v1) in zip(points, points[1:]):
            if step <= s1:
                return v0 + (v1 - v0) * (step - s0) / max(1, s1 - s0)
        return points[-1][1]

    def on_step_end(self, trainer, logs):
        for path, points in self.schedules.items():
            obj = trainer
            *parents, leaf = path.split(".")
            for name in parents:
                obj = getattr(obj, name)
            setattr(obj, leaf, self.value_at(points, trainer.global_step))


class EarlyStopCallback(Callback):
    """Stop when the logged ``metric`` has not improved by ``min_delta`` for ``patience`` logs."""

    def __init__(self, metric: str = "eval_loss", patience: int = 3, min_delta: float = 0.0, mode: str = "min"):
        self.metric, self.patience, self.min_delta = metric, patience, min_delta
        self.sign = 1.0 if mode == "min" else -1.0
        self.best, self.bad = None, 0

    def on_log(self, trainer, logs):
        if self.metric not in logs:
            return
        v = self.sign * float(logs[self.metric])
        if self.best is None or v < self.best - self.min_delta:
            self.best, self.bad = v, 0
        else:
            self.bad += 1
            if self.bad >= self.patience:
                trainer.args.max_steps = trainer.global_step         # the loop ends after this step


class RecomputePlanCallback(Callback):
    """After the first optimizer step (the probe), give as many layers as the free memory allows the lighter
    recomputation policy; the count is agreed across ranks (halo/callbacks/gradient_checkpointing_plan.py)."""

    def __init__(self, tokens_per_step: int, reserve_gb: float = 8.0, headroom: float = 0.92, group=None):
        self.tokens, self.reserve, self.headroom, self.group = tokens_per_step, int(reserve_gb * 2**30), headroom, group
        self.done = False
        self.light_layers = 0

    def on_step_end(self, trainer, logs):
        if self.done or trainer.device.type != "cuda":
            return
        from halo_b200.models.qwen3 import plan_recompute

        total = torch.cuda.get_device_properties(trainer.device).total_memory
        free = int(self.headroom * total) - torch.cuda.max_memory_reserved(trainer.device)
        self.light_layers = plan_recompute(trainer.model, self.tokens, free, self.reserve, self.group)
        self.done = True


def build_callbacks(trainer_args, model, world_size: int = 1, rank: int = 0, group=None, tokens_per_step: int = 0) -> list[Callback]:
    """The run's callbacks in a fixed order: efficiency first (it owns the step clock), integrations last."""
    from halo_b200.callbacks.balancing import BalancingCallback
    from halo_b200.callbacks.efficiency import EfficiencyCallback

    out: list[Callback] = [EfficiencyCallback(model.cfg, world_size)]
    if model.cfg.is_moe and trainer_args.moe_balancing != "none":
        out.append(BalancingCallback(model, trainer_args.moe_balancing, aux_coef=trainer_args.router_aux_loss_coef, group=group))
    if trainer_args.gradient_checkpointing and getattr(trainer_args, "gradient_checkpointing_plan", "full") == "auto" and tokens_per_step:
        out.append(RecomputePlanCallback(tokens_per_step, group=group))
    out.append(ParameterStatsCallback())
    if trainer_args.enable_torch_profiler:
        out.append(TorchProfilerCallback(rank, "0", world_size))
    return out
