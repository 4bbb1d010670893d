"""Preference optimisation on packed rows: DPO / IPO, KTO and SMPO.

A preference batch is one packed stream in which documents alternate chosen, rejected, chosen, ...
(for KTO: any order with a per-document ``desirable`` flag). Sequence log-probabilities are segment
sums of the fused head's per-token log-probs, so neither the logits plane nor a padded batch ever
exists. Reference log-probs come from a frozen copy of the model or are passed in precomputed
(the trainers of halo/trainers/preference/*.py)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from halo_b200.configs.arguments import PreferenceArguments
from halo_b200.data.packing import PackedBatch
from halo_b200.trainers import losses
from halo_b200.trainers.base import Trainer


@dataclass
class PreferenceBatch(PackedBatch):
    ref_logps: torch.Tensor | None = None     # [n_docs] precomputed reference sequence log-probs
    desirable: torch.Tensor | None = None     # [n_docs] bool, KTO only

    def to(self, device, non_blocking: bool = True):
        base = PackedBatch.to(self, device, non_blocking)
        return PreferenceBatch(base.input_ids, base.position_ids, base.labels, base.cu_seqlens, base.n_scored,
                               None if self.ref_logps is None else self.ref_logps.to(device),
                               None if self.desirable is None else self.desirable.to(device))


def sequence_logps(model, batch):
    logp, _ = model.token_logprobs(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels)
    scored = (batch.labels.reshape(-1) != -100)
    return losses.segment_sums(logp, batch.cu_seqlens, scored), losses.segment_sums(scored.float(), batch.cu_seqlens)


class PreferenceTrainer(Trainer):
    sequence_mean_loss = True

    def __init__(self, model, args, train_batches, pref_args: PreferenceArguments | None = None, ref_model=None, **kw):
        super().__init__(model, args, train_batches, **kw)
        self.pref = pref_args or PreferenceArguments()
        self.ref_model = ref_model
        if self.ref_model is not None:
            for p in self.ref_model.parameters():
                p.requires_grad_(False)

    def reference_logps(self, batch):
        if getattr(batch, "ref_logps", None) is not None:
            return batch.ref_logps
        if self.ref_model is None or self.pref.reference_free or self.pref.preference_loss == "smpo":
            return None
        with torch.no_grad():
            return sequence_logps(self.ref_model, batch)[0]

    def compute_loss(self, model, batch, normalizer):
        pol, lens = sequence_logps(model, batch)
        ref = self.reference_logps(batch)
        kind = self.pref.preference_loss
        if kind == "kto":
            ref = ref if ref is not None else torch.zeros_like(pol)
            kl = (pol - ref).detach().mean()
            loss = losses.kto_loss(pol, ref, batch.desirable, kl, self.pref.beta, self.pref.kto_desirable_weight,
                                   self.pref.kto_undesirable_weight)
        else:
            c, r = pol[0::2], pol[1::2]
            if kind == "smpo":
                loss = losses.smpo_loss(c, r, lens[0::2], lens[1::2], self.pref.beta, self.pref.smpo_margin)
            else:
                rc = ref[0::2] if ref is not None else torch.zeros_like(c)
                rr = ref[1::2] if ref is not None else torch.zeros_like(r)
                loss, _, _ = losses.dpo_loss(c, r, rc, rr, self.pref.beta, self.pref.label_smoothing,
                                             ipo=(kind == "ipo"), reference_free=self.pref.reference_free)
            if self.pref.sft_loss_weight:
                loss = loss - self.pref.sft_loss_weight * (c / lens[0::2].clamp_min(1)).mean()
        return loss


DPOTrainer = PreferenceTrainer
KTOTrainer = PreferenceTrainer
SMPOTrainer = PreferenceTrainer
