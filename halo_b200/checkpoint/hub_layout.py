"""Runtime parameter names <-> Hugging Face hub tensor names.

At run time attention holds one fused ``qkv_proj``, the dense FFN one ``gate_up_proj`` and the
routed experts two stacked banks; on disk a checkpoint uses the hub names of its family
(``q_proj`` / ``k_proj`` / ``v_proj``, ``gate_proj`` / ``up_proj``, ``experts.{e}.gate_proj`` ..., or Mixtral's
``block_sparse_moe.experts.{e}.w1`` / ``w3`` / ``w2``) so ``transformers`` loads it without custom code. The expert bank layouts are the kinds of the
reference's ``ExpertLayout`` (halo/models/moe/expert_layout.py:63-163): this family is
``SEPARATE_GLU`` on the hub and ``FUSED`` at run time.
"""

from __future__ import annotations

import re

import torch

EXPERT_LAYOUT_KINDS = ("FUSED", "FUSED_SPLIT_PER_EXPERT", "SEPARATE_GLU", "SEPARATE_MLP", "INTERLEAVED_GLU")
_LAYER = re.compile(r"^layers\.(\d+)\.(.+)$")
# family -> (feed-forward block, gate / up / down projection names of one expert) as the hub stores them
MOE_HUB_NAMES = {
    "qwen3_moe": ("mlp", "gate_proj", "up_proj", "down_proj"),
    "qwen2_moe": ("mlp", "gate_proj", "up_proj", "down_proj"),
    "mixtral": ("block_sparse_moe", "w1", "w3", "w2"),
    "glm4_moe": ("mlp", "gate_proj", "up_proj", "down_proj"),
    "deepseek_v3": ("mlp", "gate_proj", "up_proj", "down_proj"),
    "mistral4": ("mlp", "gate_proj", "up_proj", "down_proj"),
    "glm4_moe_lite": ("mlp", "gate_proj", "up_proj", "down_proj"),
    "glm_moe_dsa": ("mlp", "gate_proj", "up_proj", "down_proj"),
    "lfm2_moe": ("feed_forward", "w1", "w3", "w2"),
    "qwen3_5_moe_text": ("mlp", "gate_proj", "up_proj", "down_proj"),
    "olmoe": ("mlp", "gate_proj", "up_proj", "down_proj"),
}
# gpt-oss stores each bank as ONE tensor, transposed, with gate and up columns interleaved (``INTERLEAVED_GLU``);
# Mistral 4 stores each bank as one tensor in the runtime's own layout (``FUSED``: gate rows, then up rows)
WHOLE_BANK_FAMILIES = ("gpt_oss", "mistral4")


def _interleave(gate_then_up: torch.Tensor, dim: int) -> torch.Tensor:
    """``[.., 2F, ..]`` gate rows then up rows -> gate and up alternating along ``dim``."""
    g, u = gate_then_up.chunk(2, dim=dim)
    return torch.stack([g, u], dim=dim + 1).flatten(dim, dim + 1)


def _deinterleave(alternating: torch.Tensor, dim: int) -> torch.Tensor:
    index = [slice(None)] * alternating.dim()
    even, odd = list(index), list(index)
    even[dim], odd[dim] = slice(0, None, 2), slice(1, None, 2)
    return torch.cat([alternating[tuple(even)], alternating[tuple(odd)]], dim=dim)


def whole_bank_source(name: str, cfg, first_layer: int = 0):
    """For a parameter that the hub stores as one transformed tensor: ``(hub name, function hub tensor -> runtime
    tensor)``; ``None`` for every other parameter."""
    m = _LAYER.match(name)
    if not m or getattr(cfg, "family", "") not in WHOLE_BANK_FAMILIES:
        return None
    pre = f"model.layers.{int(m.group(1)) + first_layer}.mlp.experts."
    if cfg.family == "mistral4":
        return {"mlp.experts_gate_up": (pre + "gate_up_proj", lambda t: t),
                "mlp.experts_down": (pre + "down_proj", lambda t: t)}.get(m.group(2))
    return {
        "mlp.experts_gate_up": (pre + "gate_up_proj", lambda t: _deinterleave(t.transpose(1, 2), 1).contiguous()),
        "mlp.experts_gate_up_bias": (pre + "gate_up_proj_bias", lambda t: _deinterleave(t, 1).contiguous()),
        "mlp.experts_down": (pre + "down_proj", lambda t: t.transpose(1, 2).contiguous()),
        "mlp.experts_down_bias": (pre + "down_proj_bias", lambda t: t),
    }.get(m.group(2))
# how a family names its always-on shared feed-forward block
SHARED_EXPERT_NAMES = {"glm4_moe": "shared_experts", "deepseek_v3": "shared_experts", "mistral4": "shared_experts",
                       "glm4_moe_lite": "shared_experts", "glm_moe_dsa": "shared_experts"}


LAYER_NORMS = ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm")


def stored_with_unit_offset(name: str, cfg) -> bool:
    """Gemma stores every RMSNorm weight as ``w - 1`` (the module multiplies by ``1 + weight``); at run time the norms
    are plain, so the loader adds the one back and the writer takes it off."""
    if not getattr(cfg, "norm_unit_offset", False):
        return False
    m = _LAYER.match(name)
    return name == "norm" or bool(m and m.group(2) in LAYER_NORMS + ("self_attn.q_norm", "self_attn.k_norm"))


# families whose hub names differ from the common ones only by substitution: (common fragment, family's fragment), applied
# in order to every hub name the common rules produce
_FAMILY_RENAMES = {
    "qwen3_5_moe_text": (("model.", "model.language_model."),),
    "lfm2_moe": (("model.norm.weight", "model.embedding_norm.weight"), (".input_layernorm.", ".operator_norm."),
                 (".post_attention_layernorm.", ".ffn_norm."), (".self_attn.o_proj.", ".self_attn.out_proj."),
                 (".self_attn.q_norm.", ".self_attn.q_layernorm."), (".self_attn.k_norm.", ".self_attn.k_layernorm."),
                 (".mlp.gate_proj.", ".feed_forward.w1."), (".mlp.up_proj.", ".feed_forward.w3."),
                 (".mlp.down_proj.", ".feed_forward.w2."), (".feed_forward.gate.e_score_correction_bias", ".feed_forward.expert_bias")),
}


def runtime_to_hub(name: str, tensor: torch.Tensor, cfg, first_layer: int = 0, expert_offset: int = 0) -> dict:
    """One runtime tensor -> {hub name: tensor}. ``first_layer``: global index of ``layers.0`` (pipeline
    stages); ``expert_offset``: global index of local expert 0 (expert-parallel shards)."""
    out = _common_runtime_to_hub(name, tensor, cfg, first_layer, expert_offset)
    renames = _FAMILY_RENAMES.get(getattr(cfg, "family", ""))
    if not renames:
        return out
    renamed = {}
    for hub, t in out.items():
        for old, new in renames:
            hub = hub.replace(old, new)
        renamed[hub] = t
    return renamed


def _common_runtime_to_hub(name: str, tensor: torch.Tensor, cfg, first_layer: int = 0, expert_offset: int = 0) -> dict:
    if stored_with_unit_offset(name, cfg):
        tensor = tensor - 1
    if name == "embed_tokens":
        return {"model.embed_tokens.weight": tensor}
    if name == "norm":
        return {"model.norm.weight": tensor}
    if name == "lm_head":
        return {"lm_head.weight": tensor}
    if name == "score_head.score.weight":          # the sequence-level head of reward / classification models
        return {"score.weight": tensor}
    if name.startswith("hc_head."):
        return {"model." + name: tensor}
    if name.startswith("mtp."):
        # the head is stored as layer ``num_hidden_layers``, with the names of the DeepSeek-V3 release beside the block's
        own = {"mtp.embedding_norm": "enorm.weight", "mtp.hidden_norm": "hnorm.weight", "mtp.projection": "eh_proj.weight",
               "mtp.output_norm": "shared_head.norm.weight"}
        if name in own:
            return {f"model.layers.{cfg.num_hidden_layers}.{own[name]}": tensor}
        return _common_runtime_to_hub(f"layers.{cfg.num_hidden_layers - first_layer}." + name[len("mtp.layer."):], tensor, cfg,
                                      first_layer, expert_offset)
    m = _LAYER.match(name)
    if not m:
        raise KeyError(f"no hub name for runtime parameter {name!r}")
    li, rest = int(m.group(1)) + first_layer, m.group(2)
    pre = f"model.layers.{li}."
    D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    if rest in LAYER_NORMS:
        return {pre + rest + ".weight": tensor}
    if rest.startswith(("attn_hc.", "ffn_hc.")):       # hyper-connection parameters keep their names
        return {pre + rest: tensor}
    if rest == "self_attn.qkv_proj":
        # an output gate rides in the query projection (per head: query rows, then gate rows), so that block is twice as tall
        q, k, v = tensor.split([Hq * D * (2 if getattr(cfg, "attn_output_gate", False) else 1), Hkv * D, Hkv * D], dim=0)
        return {pre + "self_attn.q_proj.weight": q, pre + "self_attn.k_proj.weight": k,
                pre + "self_attn.v_proj.weight": v}
    if rest == "self_attn.qkv_bias":
        q, k, v = tensor.split([Hq * D, Hkv * D, Hkv * D], dim=0)
        return {pre + "self_attn.q_proj.bias": q, pre + "self_attn.k_proj.bias": k, pre + "self_attn.v_proj.bias": v}
    if rest == "self_attn.o_proj":
        return {pre + "self_attn.o_proj.weight": tensor}
    latent = {"self_attn.q_a_proj": "q_a_proj.weight", "self_attn.q_a_norm": "q_a_layernorm.weight", "self_attn.q_b_proj": "q_b_proj.weight",
              "self_attn.q_proj": "q_proj.weight", "self_attn.kv_a_proj": "kv_a_proj_with_mqa.weight",
              "self_attn.kv_a_norm": "kv_a_layernorm.weight", "self_attn.kv_b_proj": "kv_b_proj.weight",
              # the key-selecting indexer of sparse latent attention
              "self_attn.indexer_wq_b": "indexer.wq_b.weight", "self_attn.indexer_wk": "indexer.wk.weight",
              "self_attn.indexer_k_norm": "indexer.k_norm.weight", "self_attn.indexer_k_norm_bias": "indexer.k_norm.bias",
              "self_attn.indexer_weights_proj": "indexer.weights_proj.weight"}
    if rest in latent:          # multi-head latent attention (DeepSeek)
        return {pre + "self_attn." + latent[rest]: tensor}
    conv = {"self_attn.conv_in_proj": "conv.in_proj.weight", "self_attn.conv_taps": "conv.conv.weight",
            "self_attn.conv_out_proj": "conv.out_proj.weight"}
    if rest in conv:            # gated short-convolution mixer (LFM2)
        return {pre + conv[rest]: tensor}
    delta = {"self_attn.gdn_in_proj_qkvz": "in_proj_qkvz.weight", "self_attn.gdn_in_proj_ba": "in_proj_ba.weight",
             "self_attn.gdn_conv": "conv1d.weight", "self_attn.gdn_time_step": "dt_bias", "self_attn.gdn_A_log": "A_log",
             "self_attn.gdn_norm": "norm.weight", "self_attn.gdn_out_proj": "out_proj.weight",
             # Qwen3.5 stores one projection per role, each in flat head order
             "self_attn.gdn_in_proj_qkv": "in_proj_qkv.weight", "self_attn.gdn_in_proj_z": "in_proj_z.weight",
             "self_attn.gdn_in_proj_b": "in_proj_b.weight", "self_attn.gdn_in_proj_a": "in_proj_a.weight"}
    if rest in delta:           # gated delta-rule linear attention (Qwen3-Next)
        return {pre + "linear_attn." + delta[rest]: tensor}
    if rest == "self_attn.o_bias":
        return {pre + "self_attn.o_proj.bias": tensor}
    if rest == "self_attn.sinks":
        return {pre + "self_attn.sinks": tensor}
    if rest in ("self_attn.q_norm", "self_attn.k_norm"):
        return {pre + rest + ".weight": tensor}
    if rest == "mlp.gate_up_proj":
        g, u = tensor.chunk(2, dim=0)
        return {pre + "mlp.gate_proj.weight": g, pre + "mlp.up_proj.weight": u}
    if rest == "mlp.down_proj":
        return {pre + "mlp.down_proj.weight": tensor}
    if getattr(cfg, "family", "") in WHOLE_BANK_FAMILIES and rest.startswith("mlp."):
        if rest.startswith("mlp.experts_") and (expert_offset or tensor.shape[0] != cfg.num_experts):
            raise ValueError("this family's banks are stored whole: a shard of the experts has no hub form")
        whole = {"mlp.experts_gate_up": ("experts.gate_up_proj", lambda t: t),
                 "mlp.experts_down": ("experts.down_proj", lambda t: t)} if cfg.family == "mistral4" else {"mlp.gate": ("router.weight", lambda t: t), "mlp.gate_bias": ("router.bias", lambda t: t),
                 "mlp.experts_gate_up": ("experts.gate_up_proj", lambda t: _interleave(t, 1).transpose(1, 2)),
                 "mlp.experts_gate_up_bias": ("experts.gate_up_proj_bias", lambda t: _interleave(t, 1)),
                 "mlp.experts_down": ("experts.down_proj", lambda t: t.transpose(1, 2)),
                 "mlp.experts_down_bias": ("experts.down_proj_bias", lambda t: t)}
        if rest in whole:
            hub, to_hub = whole[rest]
            return {pre + "mlp." + hub: to_hub(tensor)}
    block, gate_name, up_name, down_name = MOE_HUB_NAMES.get(getattr(cfg, "family", ""), MOE_HUB_NAMES["qwen3_moe"])
    if rest == "mlp.gate":
        return {pre + f"{block}.gate.weight": tensor}
    if rest == "mlp.experts_gate_up":
        out = {}
        for le in range(tensor.shape[0]):
            g, u = tensor[le].chunk(2, dim=0)
            out[pre + f"{block}.experts.{le + expert_offset}.{gate_name}.weight"] = g
            out[pre + f"{block}.experts.{le + expert_offset}.{up_name}.weight"] = u
        return out
    if rest == "mlp.experts_down":
        return {pre + f"{block}.experts.{le + expert_offset}.{down_name}.weight": tensor[le] for le in range(tensor.shape[0])}
    shared = SHARED_EXPERT_NAMES.get(getattr(cfg, "family", ""), "shared_expert")
    if rest == "mlp.shared_expert.gate_up_proj":
        g, u = tensor.chunk(2, dim=0)
        return {pre + f"mlp.{shared}.gate_proj.weight": g, pre + f"mlp.{shared}.up_proj.weight": u}
    if rest == "mlp.shared_expert.down_proj":
        return {pre + f"mlp.{shared}.down_proj.weight": tensor}
    if rest == "mlp.e_score_correction_bias":
        return {pre + f"{block}.gate.e_score_correction_bias": tensor}
    if rest == "mlp.shared_gate":
        return {pre + "mlp.shared_expert_gate.weight": tensor}
    raise KeyError(f"no hub name for runtime parameter {name!r}")


def hub_sources(name: str, shape, cfg, first_layer: int = 0, expert_offset: int = 0) -> list[tuple[str, tuple]]:
    """Inverse view used by the loader: the hub tensors a runtime parameter is assembled from, each
    with the index of the destination slice ``(dim0 start, dim0 stop[, expert])``."""
    probe = torch.empty(shape, device="meta")
    pieces = runtime_to_hub(name, probe, cfg, first_layer, expert_offset)
    out, row = [], 0
    m = _LAYER.match(name)
    rest = m.group(2) if m else (name[len("mtp.layer."):] if name.startswith("mtp.layer.") else name)
    if rest in ("mlp.experts_gate_up", "mlp.experts_down"):
        _, gate_name, up_name, _ = MOE_HUB_NAMES.get(getattr(cfg, "family", ""), MOE_HUB_NAMES["qwen3_moe"])
        F = shape[1] // 2          # gate rows, then up rows, of the fused bank (unused for the down bank)
        for hub in pieces:
            e = int(re.search(r"experts\.(\d+)\.", hub).group(1)) - expert_offset
            if hub.endswith(f"{gate_name}.weight"):
                out.append((hub, (e, 0, F)))
            elif hub.endswith(f"{up_name}.weight"):
                out.append((hub, (e, F, 2 * F)))
            else:
                out.append((hub, (e, 0, shape[1])))
        return out
    for hub, t in pieces.items():
        n = t.shape[0]
        out.append((hub, (None, row, row + n)))
        row += n
    return out
