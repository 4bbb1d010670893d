"""Supervised fine-tuning: next-token cross-entropy over packed rows, optionally only on completion
tokens, with the router auxiliary loss re-weighted by its coefficient (the role of
halo/trainers/sft.py:92-252)."""

from __future__ import annotations

import torch

from halo_b200.trainers.base import Trainer


def load_balancing_loss(router_records, num_experts: int, top_k: int) -> torch.Tensor:
    """Switch-style auxiliary loss: num_experts * sum_e f_e * P_e, averaged over MoE layers.
    ``router_records``: list of (logits fp32 [T, E], topk_idx [T, k]) collected during the forward."""
    total = None
    for logits, idx in router_records:
        probs = torch.softmax(logits.float(), dim=-1)
        T = probs.shape[0]
        counts = torch.zeros(num_experts, dtype=torch.float32, device=probs.device)
        counts.scatter_add_(0, idx.reshape(-1).long(), torch.ones(idx.numel(), dtype=torch.float32, device=probs.device))
        f = counts / (T * top_k)
        P = probs.mean(0)
        term = num_experts * (f * P).sum()
        total = term if total is None else total + term
    if total is None:
        return torch.zeros(())
    return total / len(router_records)


class SFTTrainer(Trainer):
    """``Trainer`` with the SFT objective. Batches come from the packing collator
    (:func:`halo_b200.data.packing.pack_documents`) with labels already shifted and masked."""

    pipeline_ready = True      # the next-token objective: what a pipeline's last stage computes

    def compute_loss(self, model, batch, normalizer):
        coef = self.args.router_aux_loss_coef
        if not coef or not model.cfg.is_moe:
            return model(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels, normalizer)
        records: list = []
        ctx = model.make_context(batch.position_ids.reshape(-1), batch.cu_seqlens, record_routing=records)
        loss = model(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels, normalizer, ctx=ctx)
        # with per-layer recomputation the records of the differentiable pass arrive during backward;
        # the auxiliary term is therefore formed from the graph-free pass' logits re-attached through
        # the router weights only when recomputation is off
        live = [(lg, ix) for lg, ix in records if lg.requires_grad]
        if live:
            loss = loss + coef * load_balancing_loss(live, model.cfg.num_experts, model.cfg.num_experts_per_tok)
        return loss
