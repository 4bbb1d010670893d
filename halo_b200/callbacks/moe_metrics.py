"""Expert-load metrics and the auxiliary-loss-free balancing bias
(halo/callbacks/moe_metrics.py:28-296, halo/callbacks/balancing.py:98-429).

Loads are accumulated on the device from each router's own selection (a scatter-add, no host
sync) and read once per log. The bias update is the sign rule of DeepSeek-V3: after each step an
over-loaded expert's selection bias goes down by ``rate``, an under-loaded one's up."""

from __future__ import annotations

import torch

from halo_b200.trainers.base import Callback


class ExpertLoadCounter:
    def __init__(self, num_layers: int, num_experts: int, device):
        self.counts = torch.zeros((num_layers, num_experts), dtype=torch.int64, device=device)

    def add(self, layer: int, topk_idx: torch.Tensor) -> None:
        flat = topk_idx.reshape(-1).long()
        self.counts[layer].scatter_add_(0, flat, torch.ones_like(flat))

    def summary(self, reset: bool = True) -> dict:
        c = self.counts.float()
        mean = c.mean(1).clamp_min(1)
        out = {"moe/max_over_mean_load": float((c.max(1).values / mean).max()),
               "moe/load_cv": float((c.std(1) / mean).mean()), "moe/dead_experts": int((c == 0).sum())}
        if reset:
            self.counts.zero_()
        return out


def bias_update(bias: torch.Tensor, counts: torch.Tensor, rate: float = 1e-3) -> torch.Tensor:
    """bias += rate * sign(mean_load - load), per layer."""
    c = counts.float()
    return bias + rate * torch.sign(c.mean(-1, keepdim=True) - c)


class MoEMetricsCallback(Callback):
    def __init__(self, counter: ExpertLoadCounter, group=None):
        self.counter, self.group = counter, group

    def on_log(self, trainer, logs):
        if self.group is not None:
            import torch.distributed as dist

            dist.all_reduce(self.counter.counts, group=self.group)
        logs.update(self.counter.summary())
