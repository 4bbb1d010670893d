"""Optimizer construction: decay / no-decay groups carrying parameter names (the rounding noise of
AdamWBF16 is keyed by name) and the choice between the optimizers (the role of
halo/optimizers/param_groups.py, halo/optimizers/registry.py and the trainer's optimizer selection)."""

from __future__ import annotations

import torch

from .adamw_bf16 import AdamWBF16

OPTIMIZERS = ("adamw_bf16", "adamw_bf16_host_state", "adamw_q8", "flash_adamw", "adamw_torch", "muon")


def decay_groups(named_params, weight_decay: float) -> list[dict]:
    """Matrices decay; norms, biases and other 1-D tensors do not."""
    decay, no_decay = {"params": [], "param_names": []}, {"params": [], "param_names": []}
    for name, p in named_params:
        if not p.requires_grad or getattr(p, "zero3_managed", False):
            continue          # frozen, or a layer matrix that lives in the rank's flat ZeRO-3 shard (stepped through that)
        g = no_decay if (p.dim() <= 1 and not getattr(p, "flat_matrices", False)) else decay
        g["params"].append(p)
        g["param_names"].append(name)
    groups = []
    if decay["params"]:
        groups.append({**decay, "weight_decay": weight_decay})
    if no_decay["params"]:
        groups.append({**no_decay, "weight_decay": 0.0})
    return groups


def build_optimizer(model, name: str = "adamw_bf16", lr: float = 1e-5, weight_decay: float = 0.01,
                    betas=(0.9, 0.999), eps: float = 1e-8, device_state_budget_bytes: int = 0):
    if name not in OPTIMIZERS:
        raise ValueError(f"optim must be one of {OPTIMIZERS}, got {name!r}")
    groups = decay_groups(model.named_parameters(), weight_decay)
    if name == "adamw_bf16":
        return AdamWBF16(groups, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
    if name == "adamw_bf16_host_state":
        from .offload import HostStateAdamWBF16

        return HostStateAdamWBF16(groups, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                  device_state_budget_bytes=device_state_budget_bytes)
    if name in ("adamw_q8", "flash_adamw"):          # flash_adamw: the reference's name for its 8-bit-state optimizer
        from .adamw_q8 import AdamWQ8

        return AdamWQ8(groups, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
    if name == "muon":
        from .muon import Muon

        return Muon(groups, lr=lr, weight_decay=weight_decay, adam_betas=betas, adam_eps=eps)
    plain = [{k: v for k, v in g.items() if k != "param_names"} for g in groups]
    return torch.optim.AdamW(plain, lr=lr, betas=betas, eps=eps)
