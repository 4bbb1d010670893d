"""Multi-token-prediction head: one extra decoder block that, at position ``t``, reads the trunk's last hidden state
``h_t`` together with the embedding of token ``t + 1`` and predicts token ``t + 2`` through the shared output head.

    h' = W_proj [ norm_e(embed(x_{t+1})) ; norm_h(h_t) ]  ->  decoder block  ->  norm_out  ->  lm_head

Its cross-entropy joins the next-token loss over the same normaliser with weight ``mtp_loss_weight``. Under the
``detached`` objective the head reads detached trunk states and embeddings, so the trunk fits the next-token loss
alone and the head fits the trunk. On packed rows nothing is re-packed: embeddings and targets are the row shifted
by one, and the last position of every document (whose shifted neighbours belong to the next document) is not
scored. :func:`draft_acceptance` reports how often the head's greedy draft equals the target - the figure
speculative decoding with the head depends on.

Checkpoint names follow the DeepSeek-V3 release: the head is layer ``num_hidden_layers`` with ``enorm``, ``hnorm``,
``eh_proj`` and ``shared_head.norm`` beside the block's own tensors. The role of the reference's released-head
training (halo/models/mtp/head.py:36-120, halo/models/mtp/acceptance.py).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from halo_b200.ops import gemm
from halo_b200.ops.norm import rms_norm

IGNORE = -100


def shifted_targets(labels: torch.Tensor, cu_seqlens: torch.Tensor) -> torch.Tensor:
    """Targets two tokens ahead, aligned with positions: ``labels`` shifted left by one, with every document's last
    position (and the row's last) set to "not scored"."""
    flat = labels.reshape(-1)
    out = torch.full_like(flat, IGNORE)
    out[:-1] = flat[1:]
    ends = (torch.as_tensor(cu_seqlens, device=flat.device)[1:].long() - 1).clamp(min=0)
    out[ends[ends < out.numel()]] = IGNORE
    return out


class MTPHead(nn.Module):
    def __init__(self, cfg, dtype, device, n_local_experts: int, router_dtype=None):
        super().__init__()
        from .qwen3 import DecoderLayer

        H = cfg.hidden_size
        self.cfg = cfg
        self.embedding_norm = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.hidden_norm = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.projection = nn.Parameter(torch.empty(H, 2 * H, dtype=dtype, device=device))
        self.layer = DecoderLayer(cfg, cfg.num_hidden_layers, dtype, device, n_local_experts, router_dtype)
        self.output_norm = nn.Parameter(torch.ones(H, dtype=dtype, device=device))

    def forward(self, trunk_hidden: torch.Tensor, next_embeddings: torch.Tensor, ctx, recompute_layer: bool) -> torch.Tensor:
        """``trunk_hidden [T, H]`` (before the final norm), ``next_embeddings [T, H]`` (embedding of the following
        token) -> normed hidden states ``[T, H]`` for the shared head."""
        from .recompute import recompute

        eps = self.cfg.rms_norm_eps
        joined = torch.cat([rms_norm(next_embeddings, self.embedding_norm, eps), rms_norm(trunk_hidden, self.hidden_norm, eps)], dim=-1)
        x = gemm.linear(joined, self.projection)
        x = recompute(self.layer, x, ctx) if recompute_layer else self.layer(x, ctx)
        return rms_norm(x, self.output_norm, eps)


@torch.no_grad()
def draft_acceptance(hidden: torch.Tensor, head_weight: torch.Tensor, targets: torch.Tensor, chunk_rows: int = 8192):
    """``(accepted, scored)``: positions whose greedy draft (argmax of the head's logits) equals the target, and the
    number of scored positions; the vocabulary-sized logits exist one chunk of rows at a time."""
    targets = targets.reshape(-1)
    accepted = torch.zeros((), dtype=torch.int64, device=hidden.device)
    for lo in range(0, hidden.shape[0], chunk_rows):
        t = targets[lo:lo + chunk_rows]
        scored = t != IGNORE
        if not bool(scored.any()) and not hidden.is_cuda:
            continue
        h = hidden[lo:lo + chunk_rows]
        logits = gemm.matmul(h, head_weight) if h.is_cuda else h.float() @ head_weight.float().t()
        accepted += ((logits.argmax(-1) == t) & scored).sum()
    return accepted, (targets != IGNORE).sum()
