"""Learning-rate schedules as pure functions of the step (so a resumed run continues exactly) and
a tiny scheduler object that applies them to an optimizer's param groups."""

from __future__ import annotations

import math


def lr_factor(kind: str, step: int, total_steps: int, warmup_steps: int) -> float:
    if warmup_steps > 0 and step < warmup_steps:
        return (step + 1) / warmup_steps if kind != "constant" else 1.0
    if kind in ("constant", "constant_with_warmup") or total_steps <= 0:
        return 1.0
    progress = min(1.0, max(0.0, (step - warmup_steps) / max(1, total_steps - warmup_steps)))
    if kind == "linear":
        return 1.0 - progress
    if kind == "cosine":
        return 0.5 * (1.0 + math.cos(math.pi * progress))
    raise ValueError(f"unknown lr schedule {kind!r}")


class LRScheduler:
    def __init__(self, optimizer, kind: str, total_steps: int, warmup_steps: int = 0, last_step: int = 0):
        self.optimizer, self.kind, self.total, self.warmup = optimizer, kind, total_steps, warmup_steps
        self.base_lrs = [g["lr"] for g in optimizer.param_groups]
        self.step_count = last_step
        self._apply()

    def _apply(self):
        f = lr_factor(self.kind, self.step_count, self.total, self.warmup)
        for g, base in zip(self.optimizer.param_groups, self.base_lrs):
            g["lr"] = base * f

    def step(self):
        self.step_count += 1
        self._apply()

    def get_last_lr(self):
        return [g["lr"] for g in self.optimizer.param_groups]

    def state_dict(self):
        return {"step_count": self.step_count, "base_lrs": self.base_lrs, "kind": self.kind, "total": self.total,
                "warmup": self.warmup}

    def load_state_dict(self, sd):
        self.step_count = sd["step_count"]
        self.base_lrs = list(sd["base_lrs"])
        self._apply()
