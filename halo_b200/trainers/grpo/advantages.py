"""Group-relative advantages (halo/trainers/grpo/objective/advantages.py:169-230).

``A = r - mean_group(r)``, optionally divided by ``max(std_group, std_floor) + 1e-4`` (unbiased std),
by the std of the whole batch, or by the group mean (MaxRL). Groups whose rewards are all equal
carry no signal and are masked out of the DAPO normaliser. Offline variants (z-norm, min-max,
quantile, robust) are provided for stored rollouts."""

from __future__ import annotations

import torch

STD_EPS = 1e-4
ZERO_SPREAD = 1e-6


def group_advantages(rewards: torch.Tensor, group_size: int, scale_rewards: str = "group", std_floor: float = 0.0,
                     batch_std: torch.Tensor | None = None):
    """rewards: [n_prompts * group_size], generations of a prompt contiguous. Returns (advantages, degenerate mask
    per sample: True where the whole group has zero spread)."""
    if rewards.numel() % group_size:
        raise ValueError(f"{rewards.numel()} rewards do not split into groups of {group_size}")
    if not torch.isfinite(rewards).all():
        raise ValueError("rewards contain non-finite values")
    r = rewards.float().reshape(-1, group_size)
    mean = r.mean(1, keepdim=True)
    adv = r - mean
    spread = r.max(1, keepdim=True).values - r.min(1, keepdim=True).values
    degenerate = (spread <= ZERO_SPREAD).expand_as(r)
    if scale_rewards == "group":
        std = r.std(1, keepdim=True, unbiased=True) if group_size > 1 else torch.zeros_like(mean)
        adv = adv / (torch.clamp(std, min=std_floor) + STD_EPS)
    elif scale_rewards == "batch":
        std = batch_std if batch_std is not None else (r.std(unbiased=True) if r.numel() > 1 else r.new_zeros(()))
        adv = adv / (torch.clamp(std, min=std_floor) + STD_EPS)
    elif scale_rewards == "maxrl":
        adv = adv / (mean.abs() + STD_EPS)
    elif scale_rewards != "none":
        raise ValueError(f"unknown scale_rewards {scale_rewards!r}")
    return adv.reshape(-1), degenerate.reshape(-1)


def offline_group_advantages(rewards: torch.Tensor, group_size: int, method: str = "z_norm", clip: float = 10.0):
    r = rewards.float().reshape(-1, group_size)
    if method == "z_norm":
        a = (r - r.mean(1, keepdim=True)) / (r.std(1, keepdim=True, unbiased=False) + STD_EPS)
    elif method == "minmax":
        lo, hi = r.min(1, keepdim=True).values, r.max(1, keepdim=True).values
        a = 2 * (r - lo) / (hi - lo + STD_EPS) - 1
    elif method == "quantile_uniform":
        ranks = r.argsort(1).argsort(1).float()
        a = 2 * ranks / max(group_size - 1, 1) - 1
    elif method == "robust":
        med = r.median(1, keepdim=True).values
        mad = (r - med).abs().median(1, keepdim=True).values
        a = (r - med) / (1.4826 * mad + STD_EPS)
    else:
        raise ValueError(f"unknown offline advantage method {method!r}")
    return a.clamp(-clip, clip).reshape(-1)
