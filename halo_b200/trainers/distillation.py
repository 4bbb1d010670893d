"""Knowledge distillation: teacher -> student (forward KL / reverse KL / JSD on the token
distributions, optionally mixed with the hard-label loss) and offline self-distillation where the
"teacher" is a frozen earlier copy. The vocabulary-sized logits are formed chunk by chunk from the
final hidden states, so only ``chunk x vocab`` values are alive at once (the trainers of
halo/trainers/distillation/*.py)."""

from __future__ import annotations

import torch

from halo_b200.configs.arguments import DistillationArguments
from halo_b200.ops.gemm import linear
from halo_b200.trainers import losses
from halo_b200.trainers.base import Trainer


class _ChunkKD(torch.autograd.Function):
    """sum over tokens of divergence(student chunk logits, teacher chunk logits); the chunk logits
    are recomputed in the backward instead of being kept."""

    @staticmethod
    def forward(ctx, hs, ws, ht, wt, mask, kind, temperature):
        with torch.no_grad():
            ls = linear(hs, ws) if hs.is_cuda else hs @ ws.t()
            lt = linear(ht, wt) if ht.is_cuda else ht @ wt.t()
            s = torch.log_softmax(ls.float() / temperature, -1)
            t = torch.log_softmax(lt.float() / temperature, -1)
            out = _masked_sum(s, t, mask.to(torch.float32), kind, temperature)
        ctx.save_for_backward(hs, ws, ht, wt, mask)
        ctx.meta = (kind, temperature)
        return out

    @staticmethod
    def backward(ctx, g):
        hs, ws, ht, wt, mask = ctx.saved_tensors
        kind, temperature = ctx.meta
        with torch.enable_grad():
            hs2 = hs.detach().requires_grad_(True)
            ws2 = ws.detach().requires_grad_(True)
            ls = (linear(hs2, ws2) if hs.is_cuda else hs2 @ ws2.t())
            with torch.no_grad():
                lt = linear(ht, wt) if ht.is_cuda else ht @ wt.t()
            s = torch.log_softmax(ls.float() / temperature, -1)
            t = torch.log_softmax(lt.float() / temperature, -1)
            val = _masked_sum(s, t, mask.to(torch.float32), kind, temperature)
            dh, dw = torch.autograd.grad(val, (hs2, ws2), g)
        return dh, dw, None, None, None, None, None


def _masked_sum(s, t, m, kind, temperature):
    if kind == "forward_kl":
        per = (t.exp() * (t - s)).sum(-1)
    elif kind == "reverse_kl":
        per = (s.exp() * (s - t)).sum(-1)
    else:
        mix = torch.logsumexp(torch.stack([s, t]), 0) - 0.6931471805599453
        per = 0.5 * (t.exp() * (t - mix)).sum(-1) + 0.5 * (s.exp() * (s - mix)).sum(-1)
    return (per * m).sum() * temperature**2


def chunked_kd_sum(h_student, w_student, h_teacher, w_teacher, weights, kind="forward_kl", temperature=1.0,
                   chunk_rows: int = 2048):
    """Sum over rows of ``weights[row] * divergence(student row, teacher row)`` (times temperature squared)."""
    total = h_student.new_zeros((), dtype=torch.float32)
    for s in range(0, h_student.shape[0], chunk_rows):
        e = min(h_student.shape[0], s + chunk_rows)
        total = total + _ChunkKD.apply(h_student[s:e], w_student, h_teacher[s:e], w_teacher, weights[s:e], kind, temperature)
    return total


def chunked_kd_loss(h_student, w_student, h_teacher, w_teacher, mask, kind="forward_kl", temperature=1.0,
                    chunk_rows: int = 2048):
    total = chunked_kd_sum(h_student, w_student, h_teacher, w_teacher, mask, kind, temperature, chunk_rows)
    return total / mask.to(torch.float32).sum().clamp_min(1)


class DistillationTrainer(Trainer):
    def __init__(self, model, args, train_batches, teacher, distill_args: DistillationArguments | None = None, **kw):
        super().__init__(model, args, train_batches, **kw)
        self.teacher = teacher
        self.kd = distill_args or DistillationArguments()
        for p in self.teacher.parameters():
            p.requires_grad_(False)

    def compute_loss(self, model, batch, normalizer):
        if model.cfg.final_logit_softcapping or self.teacher.cfg.final_logit_softcapping:
            raise NotImplementedError("distillation between soft-capped output logits is not built")
        mask = batch.labels.reshape(-1) != -100
        hs = model.hidden_states(batch.input_ids, batch.position_ids, batch.cu_seqlens)
        with torch.no_grad():
            ht = self.teacher.hidden_states(batch.input_ids, batch.position_ids, batch.cu_seqlens)
        loss = self.kd.kd_weight * chunked_kd_loss(hs, model.head_weight(), ht, self.teacher.head_weight(), mask,
                                                   self.kd.kd_loss, self.kd.temperature)
        if self.kd.ce_weight:
            from halo_b200.ops.cross_entropy import fused_linear_cross_entropy

            loss = loss + self.kd.ce_weight * fused_linear_cross_entropy(hs, model.head_weight(), batch.labels.reshape(-1), normalizer)
        return loss


SelfDistillationTrainer = DistillationTrainer
