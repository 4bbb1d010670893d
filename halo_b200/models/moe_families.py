"""Facts about mixture-of-experts families and their on-disk expert layouts.

One frozen ``MoEFamilySpec`` per ``model_type`` says how the family routes (softmax or sigmoid scores, whether
the top-k weights are renormalised, a selection bias, a routed scaling factor, grouped top-k), whether it has
shared experts, which GLU it applies, and how its expert weights are laid out in a hub checkpoint. The five
layout kinds and the conversion of every kind to the run-time banks ``gate_up [E, 2F, H]`` / ``down [E, H, F]``
are the content of the reference's ``ExpertLayout`` (halo/models/moe/expert_layout.py:63-163) and
``MoEFamilySpec`` registry (halo/models/moe/family_specs.py:66-426).

``runnable`` marks the families whose whole decoder this package implements (the Qwen line, Mixtral, OLMoE, GLM-4-MoE, gpt-oss). The others are
registered so that loading one fails with a sentence that names what is missing instead of a shape error.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

FUSED = "FUSED"                                      # gate_up_proj [E, H, 2F] (+ down_proj [E, F, H]): one tensor per bank
FUSED_SPLIT_PER_EXPERT = "FUSED_SPLIT_PER_EXPERT"    # experts.{e}.gate_up_proj [2F, H], experts.{e}.down_proj
SEPARATE_GLU = "SEPARATE_GLU"                        # experts.{e}.gate_proj / up_proj / down_proj
SEPARATE_MLP = "SEPARATE_MLP"                        # experts.{e}.w1 / w3 / w2 (Mixtral naming)
INTERLEAVED_GLU = "INTERLEAVED_GLU"                  # gate_up_proj [E, H, 2F] with gate/up interleaved column-wise
LAYOUT_KINDS = (FUSED, FUSED_SPLIT_PER_EXPERT, SEPARATE_GLU, SEPARATE_MLP, INTERLEAVED_GLU)


@dataclass(frozen=True)
class MoEFamilySpec:
    model_type: str
    layout: str
    score_function: str = "softmax"          # "softmax" | "sigmoid"
    norm_topk_prob: bool = True
    selection_bias: bool = False             # e_score_correction_bias ranks experts (aux-loss-free balancing)
    routed_scaling_factor: float = 1.0
    grouped_topk: bool = False               # group-limited routing (n_group / topk_group)
    shared_experts: bool = False
    activation: str = "silu"                 # "silu" | "gelu_tanh" | "clamped_silu" | "gptoss"
    expert_bias: bool = False                # per-expert bias vectors (gpt-oss)
    router_name: str = "mlp.gate"
    experts_prefix: str = "mlp.experts"
    runnable: bool = False
    missing: str = ""


_SPECS: dict[str, MoEFamilySpec] = {}


def register(spec: MoEFamilySpec) -> MoEFamilySpec:
    if spec.layout not in LAYOUT_KINDS:
        raise ValueError(f"unknown expert layout {spec.layout!r}")
    _SPECS[spec.model_type] = spec
    return spec


for _s in (
    MoEFamilySpec("qwen3_moe", SEPARATE_GLU, runnable=True),
    MoEFamilySpec("qwen2_moe", SEPARATE_GLU, norm_topk_prob=False, shared_experts=True, runnable=True),
    MoEFamilySpec("qwen3_5_moe", SEPARATE_GLU, shared_experts=True, runnable=True),      # its text tower: model_type qwen3_5_moe_text
    MoEFamilySpec("qwen3_next", SEPARATE_GLU, shared_experts=True, runnable=True),
    MoEFamilySpec("qwen4_exp", FUSED, shared_experts=True, missing="block-sparse attention"),
    MoEFamilySpec("gpt_oss", INTERLEAVED_GLU, activation="gptoss", expert_bias=True, router_name="mlp.router", runnable=True),
    MoEFamilySpec("deepseek_v3", SEPARATE_GLU, score_function="sigmoid", selection_bias=True, routed_scaling_factor=2.5,
                  grouped_topk=True, shared_experts=True, runnable=True),
    MoEFamilySpec("deepseek_v4", SEPARATE_GLU, score_function="sigmoid", selection_bias=True, routed_scaling_factor=2.5,
                  grouped_topk=True, shared_experts=True, missing="its compressed sparse attention (latent attention and hyper-connections are built: see deepseek_v3)"),
    MoEFamilySpec("glm4_moe", SEPARATE_GLU, score_function="sigmoid", selection_bias=True, grouped_topk=True,
                  shared_experts=True, runnable=True),
    MoEFamilySpec("glm4_moe_lite", SEPARATE_GLU, score_function="sigmoid", selection_bias=True, grouped_topk=True, routed_scaling_factor=1.8,
                  shared_experts=True, runnable=True),
    MoEFamilySpec("glm_moe_dsa", SEPARATE_GLU, score_function="sigmoid", selection_bias=True, grouped_topk=True, routed_scaling_factor=2.5,
                  shared_experts=True, runnable=True),
    MoEFamilySpec("glm5_next", SEPARATE_GLU, score_function="sigmoid", selection_bias=True, shared_experts=True,
                  missing="its checkpoint names (sparse attention behind an indexer and hyper-connections are built: see glm_moe_dsa and hc_mult)"),
    MoEFamilySpec("gemma4", FUSED, activation="gelu_tanh", missing="per-layer head widths, keys / values shared between layers, per-layer input embeddings and the dense block beside the experts (the sliding / full mix and soft-capping are built: see gemma3_text)"),
    MoEFamilySpec("bailing_moe", SEPARATE_GLU, score_function="sigmoid", selection_bias=True, grouped_topk=True,
                  shared_experts=True, missing="its checkpoint names (group-limited sigmoid routing with a stored bias and shared experts are built: see glm4_moe)"),
    MoEFamilySpec("cohere2_moe", SEPARATE_GLU, missing="parallel attention/FFN block, layer norm"),
    MoEFamilySpec("inkling", SEPARATE_GLU, missing="family decoder"),
    MoEFamilySpec("laguna", SEPARATE_GLU, missing="family decoder"),
    MoEFamilySpec("lfm2_moe", SEPARATE_MLP, score_function="sigmoid", selection_bias=True, router_name="feed_forward.gate",
                  experts_prefix="feed_forward.experts", runnable=True),
    MoEFamilySpec("mistral4", FUSED, grouped_topk=True, shared_experts=True, runnable=True),
    MoEFamilySpec("olmoe", SEPARATE_GLU, norm_topk_prob=False, runnable=True),
    MoEFamilySpec("mixtral", SEPARATE_MLP, router_name="block_sparse_moe.gate", experts_prefix="block_sparse_moe.experts",
                  runnable=True),
    MoEFamilySpec("nemotron_h", SEPARATE_MLP, score_function="sigmoid", shared_experts=True, activation="relu2",
                  missing="Mamba-2 mixer layers, one block per layer, non-gated experts (document-bounded convolutions and a chunked state recurrence are built: see qwen3_next)"),
    MoEFamilySpec("step3p7", SEPARATE_GLU, shared_experts=True, missing="family decoder"),
    MoEFamilySpec("zaya", SEPARATE_GLU, missing="compressed-convolution attention"),
):
    register(_s)


def family_spec(model_type: str) -> MoEFamilySpec:
    try:
        return _SPECS[model_type]
    except KeyError:
        raise KeyError(f"no MoE family facts registered for model_type {model_type!r}; known: {sorted(_SPECS)}") from None


def families() -> list[str]:
    return sorted(_SPECS)


def require_runnable(model_type: str) -> MoEFamilySpec:
    spec = family_spec(model_type)
    if not spec.runnable:
        raise NotImplementedError(f"model_type {model_type!r} is registered but its decoder is not built here: "
                                  f"missing {spec.missing}")
    return spec


# ---- layout conversion -------------------------------------------------------------------------
def to_runtime_banks(kind: str, tensors: dict, num_experts: int, prefix: str = "") -> tuple[torch.Tensor, torch.Tensor]:
    """Hub tensors of one MoE layer (names relative to ``prefix``) -> (gate_up [E, 2F, H], down [E, H, F])."""
    g = lambda name: tensors[prefix + name]  # noqa: E731
    if kind == SEPARATE_GLU or kind == SEPARATE_MLP:
        a, b, c = ("gate_proj", "up_proj", "down_proj") if kind == SEPARATE_GLU else ("w1", "w3", "w2")
        gate_up = torch.stack([torch.cat([g(f"{e}.{a}.weight"), g(f"{e}.{b}.weight")], dim=0) for e in range(num_experts)])
        down = torch.stack([g(f"{e}.{c}.weight") for e in range(num_experts)])
        return gate_up, down
    if kind == FUSED_SPLIT_PER_EXPERT:
        gate_up = torch.stack([g(f"{e}.gate_up_proj.weight") for e in range(num_experts)])
        down = torch.stack([g(f"{e}.down_proj.weight") for e in range(num_experts)])
        return gate_up, down
    if kind == FUSED:
        return g("gate_up_proj").transpose(1, 2).contiguous(), g("down_proj").transpose(1, 2).contiguous()
    if kind == INTERLEAVED_GLU:
        gu = g("gate_up_proj")                                   # [E, H, 2F], columns g0 u0 g1 u1 ...
        gate, up = gu[..., 0::2], gu[..., 1::2]
        return torch.cat([gate, up], dim=-1).transpose(1, 2).contiguous(), g("down_proj").transpose(1, 2).contiguous()
    raise ValueError(f"unknown expert layout {kind!r}")


def from_runtime_banks(kind: str, gate_up: torch.Tensor, down: torch.Tensor, prefix: str = "", expert_offset: int = 0) -> dict:
    """Inverse of :func:`to_runtime_banks` (expert ids start at ``expert_offset`` for per-expert kinds)."""
    E, F2, H = gate_up.shape
    F = F2 // 2
    out = {}
    if kind in (SEPARATE_GLU, SEPARATE_MLP):
        a, b, c = ("gate_proj", "up_proj", "down_proj") if kind == SEPARATE_GLU else ("w1", "w3", "w2")
        for e in range(E):
            out[f"{prefix}{e + expert_offset}.{a}.weight"] = gate_up[e, :F]
            out[f"{prefix}{e + expert_offset}.{b}.weight"] = gate_up[e, F:]
            out[f"{prefix}{e + expert_offset}.{c}.weight"] = down[e]
        return out
    if kind == FUSED_SPLIT_PER_EXPERT:
        for e in range(E):
            out[f"{prefix}{e + expert_offset}.gate_up_proj.weight"] = gate_up[e]
            out[f"{prefix}{e + expert_offset}.down_proj.weight"] = down[e]
        return out
    if kind == FUSED:
        return {prefix + "gate_up_proj": gate_up.transpose(1, 2).contiguous(), prefix + "down_proj": down.transpose(1, 2).contiguous()}
    if kind == INTERLEAVED_GLU:
        gu = torch.empty((E, H, F2), dtype=gate_up.dtype, device=gate_up.device)
        gu[..., 0::2] = gate_up[:, :F].transpose(1, 2)
        gu[..., 1::2] = gate_up[:, F:].transpose(1, 2)
        return {prefix + "gate_up_proj": gu, prefix + "down_proj": down.transpose(1, 2).contiguous()}
    raise ValueError(f"unknown expert layout {kind!r}")
