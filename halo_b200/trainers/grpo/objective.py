"""Token-level GRPO objective (halo/trainers/grpo/objective/logratio.py:84-257,
offline_loss.py:20-125).

Per response token: ratio = exp(logp_train - logp_sampler) (exactly 1 on tokens that were not
sampled), clipped surrogate with asymmetric epsilons, optional k3 KL penalty against a reference
whose log-ratio tail is capped at 5 nats, and a truncated importance weight correcting for the
sampler/trainer mismatch. The loss is returned as numerator and normaliser so that gradient
accumulation and pipeline stages divide by whole-batch constants."""

from __future__ import annotations

import torch

KL_TAIL_CLAMP = 5.0


def importance_weights(logp_train: torch.Tensor, logp_sampler: torch.Tensor, sampled: torch.Tensor,
                       clip_max: float = 2.0) -> torch.Tensor:
    """Detached per-token ``min(exp(train - sampler), clip_max)``; 1 where the token was not sampled."""
    w = torch.exp((logp_train.detach() - logp_sampler).clamp(max=20.0)).clamp(max=clip_max)
    return torch.where(sampled, w, torch.ones_like(w))


def k3_kl(logp: torch.Tensor, logp_ref: torch.Tensor) -> torch.Tensor:
    d = (logp_ref - logp).clamp(max=KL_TAIL_CLAMP)
    return torch.exp(d) - d - 1.0


def grpo_token_loss(logp: torch.Tensor, logp_old: torch.Tensor, advantages_tok: torch.Tensor, mask: torch.Tensor,
                    epsilon: float = 0.2, epsilon_high: float | None = None, beta: float = 0.0,
                    logp_ref: torch.Tensor | None = None, is_weights: torch.Tensor | None = None):
    """Returns (numerator, per-token loss). ``mask``: response tokens that count."""
    eh = epsilon if epsilon_high is None else epsilon_high
    ratio = torch.exp(logp - logp_old)
    s1 = ratio * advantages_tok
    s2 = torch.clamp(ratio, 1.0 - epsilon, 1.0 + eh) * advantages_tok
    per_tok = -torch.minimum(s1, s2)
    if beta and logp_ref is not None:
        per_tok = per_tok + beta * k3_kl(logp, logp_ref)
    if is_weights is not None:
        per_tok = per_tok * is_weights
    m = mask.to(per_tok.dtype)
    return (per_tok * m).sum(), per_tok


def normalizer(loss_type: str, mask: torch.Tensor, seq_lengths: torch.Tensor | None, max_completion_length: int,
               degenerate_tok: torch.Tensor | None = None) -> torch.Tensor:
    """Whole-batch constant the numerator is divided by."""
    m = mask.to(torch.float32)
    if loss_type in ("dapo", "bnpo"):
        if degenerate_tok is not None:
            m = m * (~degenerate_tok).to(torch.float32)
        return m.sum().clamp_min(1.0)
    if loss_type == "dr_grpo":
        n_seq = seq_lengths.numel() if seq_lengths is not None else 1
        return torch.tensor(float(n_seq * max_completion_length), device=mask.device)
    if loss_type == "grpo":
        # mean over sequences of per-sequence means is formed by the caller with per-token 1/len weights
        return torch.tensor(float(seq_lengths.numel()), device=mask.device)
    raise ValueError(f"unknown loss_type {loss_type!r}")


def capped_fraction(is_weights: torch.Tensor, mask: torch.Tensor, clip_max: float) -> torch.Tensor:
    """Share of counted tokens whose importance weight sits at the cap (a device scalar)."""
    m = mask.to(torch.float32)
    return ((is_weights >= clip_max).to(torch.float32) * m).sum() / m.sum().clamp_min(1.0)


def trust_region_breaker(is_weights: torch.Tensor, mask: torch.Tensor, clip_max: float, max_fraction: float) -> bool:
    """True when so many tokens sit at the importance-weight cap that the round should be skipped."""
    return bool(capped_fraction(is_weights, mask, clip_max) > max_fraction)


# ---- optional mask stages (off by default; halo/trainers/grpo/objective/logratio.py:205-257) -------------------
def trajectory_sums(values: torch.Tensor, traj_ids: torch.Tensor, n_traj: int, mask: torch.Tensor) -> torch.Tensor:
    out = torch.zeros(n_traj, dtype=torch.float32, device=values.device)
    return out.scatter_add_(0, traj_ids.long(), values.float() * mask.float())


def geometric_mean_band_mask(logratio: torch.Tensor, traj_ids: torch.Tensor, n_traj: int, mask: torch.Tensor,
                             low: float = 0.5, high: float = 2.0) -> torch.Tensor:
    """Per trajectory: exp(mean log-ratio over its response tokens) must lie in [low, high]; trajectories outside
    the band are dropped whole. Returns a per-token bool mask (True = keep)."""
    s = trajectory_sums(logratio, traj_ids, n_traj, mask)
    n = trajectory_sums(torch.ones_like(logratio), traj_ids, n_traj, mask).clamp_min(1.0)
    g = torch.exp(s / n)
    keep = (g >= low) & (g <= high)
    return keep[traj_ids.long()]


def raw_ratio_veto_mask(logratio: torch.Tensor, traj_ids: torch.Tensor, n_traj: int, mask: torch.Tensor,
                        max_ratio: float = 100.0) -> torch.Tensor:
    """A single token whose raw ratio explodes vetoes its whole trajectory."""
    bad = (torch.exp(logratio.clamp(max=50.0)) > max_ratio) & mask
    hit = torch.zeros(n_traj, dtype=torch.float32, device=logratio.device).scatter_add_(0, traj_ids.long(), bad.float())
    return (hit == 0)[traj_ids.long()]


def off_policy_sequence_mask(logp_train: torch.Tensor, logp_sampler: torch.Tensor, advantages_tok: torch.Tensor,
                             traj_ids: torch.Tensor, n_traj: int, mask: torch.Tensor, delta: float = 0.1) -> torch.Tensor:
    """Off-policy sequence masking: a trajectory with NEGATIVE advantage whose mean sampler-to-trainer divergence
    exceeds ``delta`` is dropped (it would push the policy away from something it no longer does)."""
    div = trajectory_sums(logp_sampler - logp_train.detach(), traj_ids, n_traj, mask)
    n = trajectory_sums(torch.ones_like(logp_train), traj_ids, n_traj, mask).clamp_min(1.0)
    adv = torch.zeros(n_traj, dtype=torch.float32, device=logp_train.device).scatter_reduce_(
        0, traj_ids.long(), advantages_tok.float(), reduce="amin", include_self=False)
    drop = (adv < 0) & (div / n > delta)
    return (~drop)[traj_ids.long()]


# ---- relative rank rewards (halo/trainers/grpo/objective/relative_rewards.py:18-133) ------------------------------
def dense_rank_rewards(keys: list[tuple], group_size: int) -> torch.Tensor:
    """Hierarchical dense ranks inside each group: completions are ordered by a tuple of criteria (first criterion
    dominates, later ones break ties) and receive rewards evenly spaced in [0, 1] by dense rank (equal keys share a
    reward; a group whose keys are all equal gets 0.5 everywhere)."""
    n = len(keys)
    if n % group_size:
        raise ValueError(f"{n} completions do not form whole groups of {group_size}")
    out = torch.zeros(n, dtype=torch.float32)
    for g0 in range(0, n, group_size):
        group = keys[g0:g0 + group_size]
        distinct = sorted(set(group))
        if len(distinct) == 1:
            out[g0:g0 + group_size] = 0.5
            continue
        rank = {k: i for i, k in enumerate(distinct)}
        for i, k in enumerate(group):
            out[g0 + i] = rank[k] / (len(distinct) - 1)
    return out


def centered_logprobs(logp_token: torch.Tensor, candidate_logps: torch.Tensor, candidate_mask: torch.Tensor) -> torch.Tensor:
    """Score centring: subtract from a sampled token's log-prob the mean log-prob of the engine's candidate tokens
    at that position (a control variate computed from the sampler's own top candidates)."""
    m = candidate_mask.float()
    mean = (candidate_logps * m).sum(-1) / m.sum(-1).clamp_min(1.0)
    return logp_token - mean
