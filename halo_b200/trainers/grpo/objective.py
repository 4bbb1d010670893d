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


SAMPLER_CERTAIN_LOGPROB = 0.0   # a sampler log-prob of exactly 0: the engine emitted the token with probability 1


def corrected_tokens(logp_sampler: torch.Tensor, sampled: torch.Tensor) -> torch.Tensor:
    """Tokens the importance ratio corrects: sampled by the policy and not emitted with probability 1 (a forced or
    collapsed token carries no sampling choice, so no weight; halo/trainers/grpo/objective/logratio.py:103-109)."""
    return sampled & (logp_sampler < SAMPLER_CERTAIN_LOGPROB)


def importance_weights(logp_train: torch.Tensor, logp_sampler: torch.Tensor, sampled: torch.Tensor,
                       clip_max: float = 2.0) -> torch.Tensor:
    """Detached per-token ``min(exp(train - sampler), clip_max)`` on the corrected tokens; exactly 1 everywhere else
    (tokens that were not sampled, and tokens the sampler was certain of)."""
    corrected = corrected_tokens(logp_sampler, sampled)
    w = torch.exp((logp_train.detach() - logp_sampler).clamp(max=20.0)).clamp(max=clip_max)
    return torch.where(corrected, w, torch.ones_like(w))


def clamp_reference(logp_ref: torch.Tensor, logp: torch.Tensor) -> torch.Tensor:
    """Reference log-probs capped at ``policy + 5`` nats, with the ceiling taken from the DETACHED policy values: a
    ceiling that carried the gradient would cancel the policy term and leave a capped token without any pull back
    towards the reference (halo/trainers/grpo/objective/logratio.py:84-89)."""
    return torch.minimum(logp_ref, logp.detach() + KL_TAIL_CLAMP)


def k3_kl(logp: torch.Tensor, logp_ref: torch.Tensor) -> torch.Tensor:
    d = clamp_reference(logp_ref, logp) - logp
    return torch.exp(d) - d - 1.0


def grpo_token_loss(logp: torch.Tensor, logp_old: torch.Tensor, advantages_tok: torch.Tensor, mask: torch.Tensor,
                    epsilon: float = 0.2, epsilon_high: float | None = None, beta: float = 0.0,
                    logp_ref: torch.Tensor | None = None, is_weights: torch.Tensor | None = None,
                    token_weights: torch.Tensor | None = None):
    """Returns (numerator, per-token loss). ``mask``: response tokens that count. ``is_weights`` multiplies the
    surrogate only (a masked trajectory has weight 0 there and keeps its KL anchor); ``token_weights`` multiplies
    each token's whole term in the numerator (1 / sequence length for the per-sequence mean of ``loss_type='grpo'``)."""
    eh = epsilon if epsilon_high is None else epsilon_high
    ratio = torch.exp(logp - logp_old)
    s1 = ratio * advantages_tok
    s2 = torch.clamp(ratio, 1.0 - epsilon, 1.0 + eh) * advantages_tok
    per_tok = -torch.minimum(s1, s2)
    if is_weights is not None:
        per_tok = per_tok * is_weights
    if beta and logp_ref is not None:
        per_tok = per_tok + beta * k3_kl(logp, logp_ref)
    m = mask.to(per_tok.dtype)
    if token_weights is not None:
        m = m * token_weights.to(per_tok.dtype)
    return (per_tok * m).sum(), per_tok


def normalizer(loss_type: str, mask: torch.Tensor, seq_lengths: torch.Tensor | None, max_completion_length: int,
               degenerate_tok: torch.Tensor | None = None) -> torch.Tensor:
    """Constant the numerator of ONE batch is divided by (single micro-batch, single rank). Rounds that span
    micro-batches or ranks use :func:`round_denominator` instead, summed over all of them."""
    m = mask.to(torch.float32)
    if loss_type in ("dapo", "bnpo"):
        if degenerate_tok is not None:
            m = m * (~degenerate_tok).to(torch.float32)
        return m.sum().clamp_min(1.0)
    if loss_type == "dr_grpo":
        n_seq = seq_lengths.numel() if seq_lengths is not None else 1
        return torch.tensor(float(n_seq * max_completion_length), device=mask.device)
    if loss_type == "grpo":
        # mean over sequences of per-sequence means: the caller weighs every token by 1 / its sequence's length
        return torch.tensor(float(seq_lengths.numel()), device=mask.device)
    raise ValueError(f"unknown loss_type {loss_type!r}")


def round_denominator(loss_type: str, counted_tokens: list[int], degenerate: list[bool], max_completion_length: int) -> float:
    """This rank's share of a round's loss denominator, from host-side row facts: ``counted_tokens[i]`` is the number of
    policy-produced completion tokens of row i and ``degenerate[i]`` whether its group has no reward spread. The caller
    sums the shares over the data-parallel ranks; every micro-batch of the round then divides by that one number, so
    the loss scale depends neither on how the round was cut into micro-batches nor on the data-parallel width.

      dapo / bnpo   counted tokens of the rows that carry a signal
      dr_grpo       rows x max_completion_length
      grpo          rows with at least one counted token (each row contributes its own token mean)
    """
    if loss_type in ("dapo", "bnpo"):
        return float(sum(n for n, d in zip(counted_tokens, degenerate) if not d))
    if loss_type == "dr_grpo":
        return float(len(counted_tokens) * max_completion_length)
    if loss_type == "grpo":
        return float(sum(1 for n in counted_tokens if n > 0))
    raise ValueError(f"unknown loss_type {loss_type!r}")


def capped_fraction(is_weights: torch.Tensor, mask: torch.Tensor, clip_max: float) -> torch.Tensor:
    """Share of counted tokens whose importance weight sits at the cap (a device scalar)."""
    m = mask.to(torch.float32)
    return ((is_weights >= clip_max).to(torch.float32) * m).sum() / m.sum().clamp_min(1.0)


def trust_region_breaker(is_weights: torch.Tensor, mask: torch.Tensor, clip_max: float, max_fraction: float) -> bool:
    """True when so many tokens sit at the importance-weight cap that the round should be skipped."""
    return bool(capped_fraction(is_weights, mask, clip_max) > max_fraction)


# ---- optional mask stages (off by default; halo/trainers/grpo/objective/logratio.py:205-284) -------------------
def trajectory_sums(values: torch.Tensor, traj_ids: torch.Tensor, n_traj: int, mask: torch.Tensor) -> torch.Tensor:
    out = torch.zeros(n_traj, dtype=torch.float32, device=values.device)
    return out.scatter_add_(0, traj_ids.long(), values.float() * mask.float())


def trajectory_mean_logratio(logratio: torch.Tensor, traj_ids: torch.Tensor, n_traj: int, corrected: torch.Tensor) -> torch.Tensor:
    """Mean log-ratio of every trajectory over its corrected tokens (the geometric-mean ratio in log space)."""
    s = trajectory_sums(logratio, traj_ids, n_traj, corrected)
    n = trajectory_sums(torch.ones_like(logratio), traj_ids, n_traj, corrected).clamp_min(1.0)
    return s / n


def geometric_mean_band_mask(logratio: torch.Tensor, traj_ids: torch.Tensor, n_traj: int, corrected: torch.Tensor,
                             low: float = 0.5, high: float = 2.0) -> torch.Tensor:
    """Per trajectory: exp(mean log-ratio over its corrected tokens) must lie in [low, high]; trajectories outside
    the band are dropped whole. Returns a per-token bool mask (True = keep)."""
    g = torch.exp(trajectory_mean_logratio(logratio, traj_ids, n_traj, corrected))
    keep = (g >= low) & (g <= high)
    return keep[traj_ids.long()]


def raw_ratio_veto_mask(logratio: torch.Tensor, traj_ids: torch.Tensor, n_traj: int, corrected: torch.Tensor,
                        veto_min: float = 1e-4) -> torch.Tensor:
    """A single corrected token whose RAW ratio ``exp(train - sampler)`` falls below ``veto_min`` (a token the
    trainer finds all but impossible although the sampler produced it) vetoes its whole trajectory. The test reads
    the unclipped ratio, so the truncation cannot hide such a token."""
    raw = torch.where(corrected, torch.exp(logratio.float().clamp(max=50.0)), torch.ones_like(logratio, dtype=torch.float32))
    lowest = torch.ones(n_traj, dtype=torch.float32, device=logratio.device).scatter_reduce_(
        0, traj_ids.long(), raw, reduce="amin", include_self=True)
    return (lowest >= veto_min)[traj_ids.long()]


def off_policy_sequence_mask(logratio: torch.Tensor, corrected: torch.Tensor, advantages_tok: torch.Tensor,
                             traj_ids: torch.Tensor, n_traj: int, delta: float = 0.1) -> torch.Tensor:
    """Off-policy sequence masking: a trajectory with NEGATIVE advantage whose mean log-ratio between trainer and
    sampler exceeds ``delta`` nats in MAGNITUDE (either direction) is dropped. True = keep."""
    mean = trajectory_mean_logratio(logratio, traj_ids, n_traj, corrected)
    adv = torch.zeros(n_traj, dtype=torch.float32, device=logratio.device).scatter_reduce_(
        0, traj_ids.long(), advantages_tok.float(), reduce="amin", include_self=False)
    drop = (adv < 0) & (mean.abs() > delta)
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
