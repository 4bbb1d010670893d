"""Sequence-level objectives on per-token log-probabilities: DPO / IPO, KTO, SMPO, Bradley-Terry
reward, and the distillation divergences. Pure functions of tensors, shared by the method trainers
and tested on CPU (the objectives of halo/trainers/preference/*.py, halo/trainers/reward/*.py and
halo/trainers/distillation/*.py)."""

from __future__ import annotations

import torch
import torch.nn.functional as F


def segment_sums(values: torch.Tensor, cu_seqlens, mask: torch.Tensor | None = None) -> torch.Tensor:
    """Sum of ``values`` over every document of a packed stream -> [n_docs] (no host sync)."""
    cu = torch.as_tensor(cu_seqlens, dtype=torch.long, device=values.device)
    v = values if mask is None else values * mask.to(values.dtype)
    csum = torch.cat([v.new_zeros(1), torch.cumsum(v.float(), 0)])
    return csum[cu[1:]] - csum[cu[:-1]]


def dpo_loss(pol_chosen, pol_rejected, ref_chosen, ref_rejected, beta: float = 0.1, label_smoothing: float = 0.0,
             ipo: bool = False, reference_free: bool = False):
    """Sequence log-probs -> (loss, chosen rewards, rejected rewards)."""
    if reference_free:
        ref_chosen = torch.zeros_like(pol_chosen)
        ref_rejected = torch.zeros_like(pol_rejected)
    logits = (pol_chosen - pol_rejected) - (ref_chosen - ref_rejected)
    if ipo:
        loss = (logits - 1.0 / (2.0 * beta)) ** 2
    else:
        loss = -F.logsigmoid(beta * logits) * (1 - label_smoothing) - F.logsigmoid(-beta * logits) * label_smoothing
    return loss.mean(), beta * (pol_chosen - ref_chosen).detach(), beta * (pol_rejected - ref_rejected).detach()


def kto_loss(pol_logps, ref_logps, desirable: torch.Tensor, kl_estimate: torch.Tensor, beta: float = 0.1,
             desirable_weight: float = 1.0, undesirable_weight: float = 1.0):
    """Kahneman-Tversky objective on unpaired examples. ``desirable``: bool [n]; ``kl_estimate``: scalar
    (detached, clamped at 0) batch estimate of KL(policy || reference)."""
    ratio = pol_logps - ref_logps
    kl = kl_estimate.detach().clamp_min(0)
    good = 1 - torch.sigmoid(beta * (ratio - kl))
    bad = 1 - torch.sigmoid(beta * (kl - ratio))
    d = desirable.to(ratio.dtype)
    losses = d * desirable_weight * good + (1 - d) * undesirable_weight * bad
    return losses.mean()


def smpo_loss(pol_chosen, pol_rejected, len_chosen, len_rejected, beta: float = 2.0, margin: float = 1.0):
    """Reference-free, length-normalised margin objective: -log sigmoid(beta (avg_c - avg_r) - margin)."""
    avg_c = pol_chosen / len_chosen.clamp_min(1)
    avg_r = pol_rejected / len_rejected.clamp_min(1)
    return (-F.logsigmoid(beta * (avg_c - avg_r) - margin)).mean()


def bradley_terry_loss(score_chosen, score_rejected, margin: torch.Tensor | None = None, center_coef: float = 0.0):
    diff = score_chosen - score_rejected
    if margin is not None:
        diff = diff - margin
    loss = -F.logsigmoid(diff).mean()
    if center_coef:
        loss = loss + center_coef * ((score_chosen + score_rejected) ** 2).mean()
    return loss


def distillation_divergence(student_logits, teacher_logits, kind: str = "forward_kl", temperature: float = 1.0,
                            mask: torch.Tensor | None = None):
    """Token-level divergence between teacher and student distributions, summed over the vocabulary and
    averaged over scored tokens. forward_kl = KL(teacher || student)."""
    s = F.log_softmax(student_logits.float() / temperature, dim=-1)
    t = F.log_softmax(teacher_logits.float() / temperature, dim=-1)
    if kind == "forward_kl":
        per_tok = (t.exp() * (t - s)).sum(-1)
    elif kind == "reverse_kl":
        per_tok = (s.exp() * (s - t)).sum(-1)
    elif kind == "jsd":
        m = torch.logsumexp(torch.stack([s, t]), dim=0) - torch.log(torch.tensor(2.0))
        per_tok = 0.5 * (t.exp() * (t - m)).sum(-1) + 0.5 * (s.exp() * (s - m)).sum(-1)
    else:
        raise ValueError(f"unknown divergence {kind!r}")
    per_tok = per_tok * temperature**2
    if mask is None:
        return per_tok.mean()
    m = mask.to(per_tok.dtype)
    return (per_tok * m).sum() / m.sum().clamp_min(1)
