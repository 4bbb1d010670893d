"""Expert-load balancing driven from the trainer loop (halo/callbacks/balancing.py:98-429).

Modes (``moe_balancing``):
  ``aux_loss``     the switch-style auxiliary loss is added by the SFT trainer; this callback only reports loads
  ``bias_update``  auxiliary-loss-free balancing: after every optimizer step each MoE layer's selection bias moves
                   by ``rate * sign(mean load - load)`` computed from loads summed over ALL ranks; the bias is
                   saved beside each checkpoint and restored on resume
  ``none``         nothing
  ``auto``         ``bias_update`` when the model's config carries no auxiliary-loss coefficient, else ``aux_loss``
The mode is agreed across ranks before the first step (a divergent setting raises everywhere)."""

from __future__ import annotations

import os

import torch

from halo_b200.callbacks.moe_metrics import ExpertLoadCounter, bias_update
from halo_b200.checkpoint.atomic import atomic_torch_save
from halo_b200.trainers.base import Callback

SIDECAR = "router_selection_bias.pt"


def moe_layers(model):
    return [(i, layer.mlp) for i, layer in enumerate(model.layers) if hasattr(layer.mlp, "selection_bias")]


def resolve_mode(mode: str, cfg, aux_coef: float) -> str:
    if mode != "auto":
        return mode
    return "aux_loss" if (aux_coef or cfg.router_aux_loss_coef) else "bias_update"


class BalancingCallback(Callback):
    def __init__(self, model, mode: str = "auto", rate: float = 1e-3, aux_coef: float = 0.0, group=None):
        self.model, self.rate, self.group = model, rate, group
        self.mode = resolve_mode(mode, model.cfg, aux_coef)
        self.layers = moe_layers(model)
        self.counter = None
        if self.layers and self.mode in ("bias_update", "aux_loss"):
            dev = next(model.parameters()).device
            self.counter = ExpertLoadCounter(len(self.layers), model.cfg.num_experts, dev)
            for slot, (_, mlp) in enumerate(self.layers):
                mlp.load_counter = (self.counter, slot)
                if self.mode == "bias_update" and mlp.selection_bias is None:
                    mlp.selection_bias = torch.zeros(model.cfg.num_experts, dtype=torch.float32, device=dev)

    def on_train_begin(self, trainer):
        from halo_b200.runtime.consensus import reject_divergent_settings

        reject_divergent_settings({"moe_balancing": self.mode}, group=self.group)

    def on_step_end(self, trainer, logs):
        if self.counter is None or self.mode != "bias_update":
            return
        counts = self.counter.counts.clone()
        if self.group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()):
            torch.distributed.all_reduce(counts, group=self.group)
        for slot, (_, mlp) in enumerate(self.layers):
            mlp.selection_bias.copy_(bias_update(mlp.selection_bias, counts[slot], self.rate))
        self.last_counts = counts
        self.counter.counts.zero_()

    def on_log(self, trainer, logs):
        if self.counter is not None and self.mode == "aux_loss":
            logs.update(self.counter.summary())
        elif getattr(self, "last_counts", None) is not None:
            c = self.last_counts.float()
            logs["moe/max_over_mean_load"] = float((c.max(1).values / c.mean(1).clamp_min(1)).max())

    def on_save(self, trainer, directory):
        if self.mode == "bias_update" and trainer.is_main:
            atomic_torch_save({i: mlp.selection_bias.cpu() for i, mlp in self.layers}, os.path.join(directory, SIDECAR))

    def load(self, directory: str) -> bool:
        path = os.path.join(directory, SIDECAR)
        if not os.path.isfile(path):
            return False
        blob = torch.load(path, weights_only=False)
        for i, mlp in self.layers:
            if i in blob and mlp.selection_bias is not None:
                mlp.selection_bias.copy_(blob[i])
        return True
