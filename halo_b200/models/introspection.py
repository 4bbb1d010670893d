"""Structural queries on a model object that callbacks, loaders and trainers share
(halo/models/introspection/*.py): the decoder layers, the backbone without the head, parameter roles."""

from __future__ import annotations

from collections import Counter


def decoder_layers(model) -> list:
    layers = getattr(model, "layers", None)
    if layers is None:
        raise TypeError(f"{type(model).__name__} exposes no decoder layer list")
    return list(layers)


def moe_layer_indices(model) -> list[int]:
    return [i for i, layer in enumerate(decoder_layers(model)) if hasattr(layer.mlp, "experts_gate_up")]


def parameter_role(name: str, param) -> str:
    """One of: embedding, head, norm, attention, router, expert, shared_expert, dense_ffn."""
    if name.startswith("embed_tokens"):
        return "embedding"
    if name.startswith("lm_head"):
        return "head"
    if param.dim() == 1 or name.endswith(("layernorm", "norm", "q_norm", "k_norm")):
        return "norm"
    if ".self_attn." in name:
        return "attention"
    if name.endswith("mlp.gate") or name.endswith("shared_gate"):
        return "router"
    if getattr(param, "is_expert", False):
        return "expert"
    if ".shared_expert." in name:
        return "shared_expert"
    return "dense_ffn"


def parameter_roles(model) -> dict[str, int]:
    """Number of parameters per role (a quick check of what a freeze pattern or a learning-rate group covers)."""
    c: Counter = Counter()
    for n, p in model.named_parameters():
        c[parameter_role(n, p)] += p.numel()
    return dict(c)
