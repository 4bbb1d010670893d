"""What a run does with the attention sinks of a gpt-oss checkpoint (one learned logit per head that joins every
softmax): ``neutralized`` sets them to (almost) the most negative finite bf16 value, so they take no softmax mass and get no
gradient - fine-tuning then behaves like a model without sinks; ``live`` keeps the pretrained values and freezes
them (the on-policy setting: the policy must predict like the sampler); ``trainable`` keeps and trains them.
(The role of halo/models/attention/gpt_oss_sinks.py:1-344: ``SinksPolicy`` and ``apply_sinks_policy``.)"""

from __future__ import annotations

import torch

POLICIES = ("neutralized", "live", "trainable")
POLICY_ATTR = "sinks_policy"


def policy_from_flags(reset_sinks: bool, train_sinks: bool = False) -> str:
    if reset_sinks and train_sinks:
        raise ValueError("train_sinks: true contradicts reset_sinks: true - a neutralized sink has zero softmax mass and zero "
                         "gradient, so nothing could train; set reset_sinks: false alongside train_sinks")
    if reset_sinks:
        return "neutralized"
    return "trainable" if train_sinks else "live"


def sink_parameters(model) -> list[tuple[str, torch.nn.Parameter]]:
    return [(n, p) for n, p in model.named_parameters() if n.endswith(".sinks")]


def is_sink_name(name: str) -> bool:
    return name.endswith(".sinks") or ".sinks." in name


@torch.no_grad()
def apply_sinks_policy(model, policy: str, pretrained: bool = True) -> int:
    """Apply ``policy`` to every sink of ``model`` once, after loading; returns how many tensors it touched. A model
    initialised from scratch has nothing pretrained to protect: ``neutralized`` leaves its (zero) sinks live there."""
    if policy not in POLICIES:
        raise ValueError(f"sinks policy {policy!r}: choose from {', '.join(POLICIES)}")
    sinks = sink_parameters(model)
    if not sinks:
        if policy == "trainable":
            raise ValueError("train_sinks: this model has no attention sinks")
        return 0
    if policy == "trainable" and any(".lora_" in n for n, _ in model.named_parameters()):
        raise ValueError("train_sinks with low-rank adapters: the adapter file has no place for sinks; keep them live and "
                         "frozen (reset_sinks: false without train_sinks) or train full weights")
    if policy == "neutralized" and not pretrained:
        policy = "live"
    for _, p in sinks:
        if policy == "neutralized":
            # just inside the bf16 range, so that a save in bf16 (or a reload in fp32) keeps it finite
            p.fill_(0.99 * torch.finfo(torch.bfloat16).min)
        p.requires_grad_(policy == "trainable")
    setattr(model, POLICY_ATTR, policy)
    return len(sinks)
