"""What a family does to its logits around ``lm_head``: a constant scale, a tanh soft-cap, a cut of the
vocabulary to the rows the tokenizer can emit (halo/models/head_transform.py:1-252).

The fused linear + cross-entropy path takes the scale as the GEMM's ``alpha`` and the vocabulary cut as a
narrower weight view, both for free; a soft-cap needs the element-wise pass below on each logits chunk
(forward ``cap * tanh(z / cap)``, backward ``1 - tanh^2``), which the chunked PyTorch path applies."""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class HeadTransform:
    logit_scale: float = 1.0
    softcap: float = 0.0
    vocab_cut: int = 0           # 0 = keep every row of lm_head

    @property
    def is_identity(self) -> bool:
        return self.logit_scale == 1.0 and not self.softcap and not self.vocab_cut

    @property
    def fusable(self) -> bool:
        """True when the fused kernel path can apply it without an extra pass over the logits."""
        return not self.softcap

    def weight_view(self, lm_head: torch.Tensor) -> torch.Tensor:
        return lm_head[: self.vocab_cut] if self.vocab_cut else lm_head

    def apply(self, logits: torch.Tensor) -> torch.Tensor:
        z = logits.float() * self.logit_scale
        if self.softcap:
            z = self.softcap * torch.tanh(z / self.softcap)
        return z


def from_config(cfg_dict: dict) -> HeadTransform:
    """Read the family's fields from a Hugging Face config dictionary."""
    scale = float(cfg_dict.get("logit_scale", 1.0) or 1.0)
    if cfg_dict.get("logits_scaling"):            # granite-style divisor
        scale = 1.0 / float(cfg_dict["logits_scaling"])
    cap = float(cfg_dict.get("final_logit_softcapping", 0.0) or 0.0)
    return HeadTransform(scale, cap, int(cfg_dict.get("vocab_cut", 0) or 0))


def chunked_cross_entropy(hidden, lm_head, labels, transform: HeadTransform, chunk_rows: int = 4096, ignore_index: int = -100,
                          normalizer: float | None = None):
    """Reference / soft-cap path: row chunks of logits, transformed, fp32 cross-entropy; differentiable."""
    w = transform.weight_view(lm_head)
    total = hidden.new_zeros((), dtype=torch.float32)
    count = (labels != ignore_index).sum().clamp_min(1) if normalizer is None else normalizer
    for lo in range(0, hidden.shape[0], chunk_rows):
        h = hidden[lo:lo + chunk_rows]
        z = transform.apply(h.float() @ w.float().t())
        total = total + torch.nn.functional.cross_entropy(z, labels[lo:lo + chunk_rows], ignore_index=ignore_index, reduction="sum")
    return total / count
