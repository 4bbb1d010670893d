"""Reward-model (Bradley-Terry), sequence-classification and embedding trainers: a small head on the
final hidden state of each document's last token (the role of halo/trainers/reward/*.py and
halo/trainers/embedding/*.py)."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from halo_b200.trainers import losses
from halo_b200.trainers.base import Trainer


class SequenceHead(nn.Module):
    """Linear head applied to the last token of every packed document."""

    def __init__(self, hidden: int, num_labels: int = 1, dtype=torch.float32, device=None):
        super().__init__()
        self.score = nn.Linear(hidden, num_labels, bias=False, dtype=dtype, device=device)

    def forward(self, hidden_states: torch.Tensor, cu_seqlens) -> torch.Tensor:
        last = torch.as_tensor(cu_seqlens[1:], dtype=torch.long, device=hidden_states.device) - 1
        return self.score(hidden_states[last].to(self.score.weight.dtype))


def last_token_states(model, batch):
    h = model.hidden_states(batch.input_ids, batch.position_ids, batch.cu_seqlens)
    last = torch.as_tensor(batch.cu_seqlens[1:], dtype=torch.long, device=h.device) - 1
    return h[last]


class RewardTrainer(Trainer):
    """Documents alternate chosen / rejected; loss = -log sigmoid(r_chosen - r_rejected)."""

    sequence_mean_loss = True

    def __init__(self, model, args, train_batches, head: SequenceHead, center_coef: float = 0.0, **kw):
        self.head = head
        super().__init__(_WithHead(model, head), args, train_batches, **kw)
        self.center_coef = center_coef

    def compute_loss(self, wrapped, batch, normalizer):
        h = wrapped.model.hidden_states(batch.input_ids, batch.position_ids, batch.cu_seqlens)
        scores = wrapped.head(h, batch.cu_seqlens)[:, 0]
        return losses.bradley_terry_loss(scores[0::2], scores[1::2], center_coef=self.center_coef)


class ClassificationTrainer(RewardTrainer):
    """One label per document (``batch.doc_labels``); cross-entropy over ``num_labels``."""

    def compute_loss(self, wrapped, batch, normalizer):
        h = wrapped.model.hidden_states(batch.input_ids, batch.position_ids, batch.cu_seqlens)
        logits = wrapped.head(h, batch.cu_seqlens)
        return F.cross_entropy(logits.float(), batch.doc_labels.to(logits.device))


class EmbeddingTrainer(Trainer):
    """Contrastive (in-batch negatives) training of last-token embeddings; documents alternate
    query, positive."""

    sequence_mean_loss = True

    def __init__(self, model, args, train_batches, temperature: float = 0.05, **kw):
        super().__init__(model, args, train_batches, **kw)
        self.temperature = temperature

    def compute_loss(self, model, batch, normalizer):
        e = F.normalize(last_token_states(model, batch).float(), dim=-1)
        q, p = e[0::2], e[1::2]
        sim = q @ p.t() / self.temperature
        target = torch.arange(sim.shape[0], device=sim.device)
        return 0.5 * (F.cross_entropy(sim, target) + F.cross_entropy(sim.t(), target))


class _WithHead(nn.Module):
    def __init__(self, model, head):
        super().__init__()
        self.model, self.head = model, head
        self.cfg = model.cfg
        self.transport = model.transport
        self.layer_range = model.layer_range

    def named_parameters(self, *a, **kw):
        yield from self.model.named_parameters(*a, **kw)
        for n, p in self.head.named_parameters():
            yield "score_head." + n, p
