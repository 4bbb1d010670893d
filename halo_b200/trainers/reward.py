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


def pooled_states(model, batch, pooling: str = "last_token"):
    """One vector per packed document: its last token's hidden state, or the mean over its tokens."""
    if pooling == "last_token":
        return last_token_states(model, batch)
    if pooling != "mean":
        raise ValueError(f"unknown pooling {pooling!r}: last_token or mean")
    h = model.hidden_states(batch.input_ids, batch.position_ids, batch.cu_seqlens)
    cu = torch.as_tensor(batch.cu_seqlens, dtype=torch.long, device=h.device)
    lengths = (cu[1:] - cu[:-1]).clamp(min=1)
    doc = torch.repeat_interleave(torch.arange(len(lengths), device=h.device), cu[1:] - cu[:-1])
    sums = torch.zeros(len(lengths), h.shape[-1], dtype=torch.float32, device=h.device).index_add_(0, doc, h[:len(doc)].float())
    return (sums / lengths[:, None]).to(h.dtype)


@torch.no_grad()
def embedding_metrics(q: torch.Tensor, p: torch.Tensor, raw_norm: torch.Tensor) -> dict:
    """What the reference's embedding trainer logs beside the loss: the mean norm of the vectors before normalisation,
    the spread of the normalised coordinates (a collapse shows as a shrinking ``embed/std``), the mean cosine of the true
    pairs and the mean reciprocal rank of a query's positive among the batch's positives."""
    sim = q @ p.t()
    rank = (sim > sim.diag()[:, None]).sum(dim=1) + 1
    return {"embed/norm": float(raw_norm.mean()), "embed/std": float(torch.cat([q, p]).std(dim=0).mean()),
            "embed/cos_sim": float(sim.diag().mean()), "embed/mrr": float((1.0 / rank.float()).mean())}


class EmbeddingTrainer(Trainer):
    """Contrastive (in-batch negatives) training of one embedding per document (last token or mean pooling); documents
    alternate query, positive."""

    sequence_mean_loss = True

    def __init__(self, model, args, train_batches, temperature: float = 0.05, pooling: str = "last_token", **kw):
        super().__init__(model, args, train_batches, **kw)
        self.temperature, self.pooling = temperature, pooling
        self._metrics: dict = {}

    def compute_loss(self, model, batch, normalizer):
        raw = pooled_states(model, batch, self.pooling).float()
        e = F.normalize(raw, dim=-1)
        q, p = e[0::2], e[1::2]
        sim = q @ p.t() / self.temperature
        target = torch.arange(sim.shape[0], device=sim.device)
        log_every = max(1, int(getattr(self.args, "logging_steps", 1) or 1))
        if (self.global_step + 1) % log_every == 0:               # on the steps that are logged next
            self._metrics = embedding_metrics(q.detach(), p.detach(), raw.detach().norm(dim=-1))
        return 0.5 * (F.cross_entropy(sim, target) + F.cross_entropy(sim.t(), target))

    def extra_logs(self) -> dict:
        return dict(self._metrics)


def write_sentence_transformers_layout(directory: str, hidden_size: int, pooling: str = "last_token", max_seq_length: int = 0,
                                       normalize: bool = True) -> None:
    """The pipeline description files beside a saved Hugging Face checkpoint that make ``SentenceTransformer(directory)``
    load it as transformer -> pooling (-> normalisation): ``modules.json``, ``sentence_bert_config.json``,
    ``config_sentence_transformers.json`` and the pooling module's ``config.json``. The weights stay where the
    checkpoint writer put them (the transformer module lives at the directory's root)."""
    import json
    import os

    modules = [{"idx": 0, "name": "0", "path": "", "type": "sentence_transformers.models.Transformer"},
               {"idx": 1, "name": "1", "path": "1_Pooling", "type": "sentence_transformers.models.Pooling"}]
    if normalize:
        modules.append({"idx": 2, "name": "2", "path": "2_Normalize", "type": "sentence_transformers.models.Normalize"})
        os.makedirs(os.path.join(directory, "2_Normalize"), exist_ok=True)
    os.makedirs(os.path.join(directory, "1_Pooling"), exist_ok=True)
    pool = {"word_embedding_dimension": int(hidden_size), "pooling_mode_cls_token": False,
            "pooling_mode_mean_tokens": pooling == "mean", "pooling_mode_max_tokens": False,
            "pooling_mode_mean_sqrt_len_tokens": False, "pooling_mode_weightedmean_tokens": False,
            "pooling_mode_lasttoken": pooling == "last_token", "include_prompt": True}
    files = {"modules.json": modules,
             "sentence_bert_config.json": {"max_seq_length": int(max_seq_length) or None, "do_lower_case": False},
             "config_sentence_transformers.json": {"prompts": {}, "default_prompt_name": None, "similarity_fn_name": "cosine"},
             os.path.join("1_Pooling", "config.json"): pool}
    for name, body in files.items():
        with open(os.path.join(directory, name), "w") as f:
            json.dump(body, f, indent=2)


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
