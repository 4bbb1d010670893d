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


def trust_region_breaker(is_weights: torch.Tensor, mask: torch.Tensor, clip_max: float, max_fraction: float) -> bool:
    """True when so many tokens sit at the importance-weight cap that the round should be skipped."""
    m = mask.to(torch.float32)
    frac = ((is_weights >= clip_max).to(torch.float32) * m).sum() / m.sum().clamp_min(1.0)
    return bool(frac > max_fraction)
