"""Architecture description of the decoder families built here, convertible to and from a Hugging Face
``config.json``: Qwen3 and Qwen3-MoE (per-head q/k norm), Qwen2 (biased q/k/v projections), Qwen2-MoE (gated
shared expert), Llama and Mistral (plain pre-norm decoder, optional rotary scaling), Mixtral (top-k of
softmax, ``block_sparse_moe`` names on the hub), OLMoE, GLM-4-MoE, gpt-oss (sinks, biased clamped-GLU experts),
DeepSeek-V3 (latent attention) and Gemma 3 (windowed / full layer mix, four norms per layer).

The named presets are the shapes of the benchmark configurations: a tiny MoE for CPU plumbing
tests, the dense 9B class, the 30B-A3B MoE and the ~120B-total shared-expert MoE.
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path


# Per family: the Hugging Face architecture, whether q / k carry a per-head RMSNorm, whether the q / k / v bias is a
# config key (Llama, Qwen3) or fixed by the family (Qwen2: always on), whether the config has a sliding window, and
# how the hub names the feed-forward block and its experts.
FAMILIES = {
    "qwen3": dict(architecture="Qwen3ForCausalLM", moe=False, qk_norm=True, bias_key=True, bias_default=False, has_window=False),
    "qwen3_moe": dict(architecture="Qwen3MoeForCausalLM", moe=True, qk_norm=True, bias_key=True, bias_default=False, has_window=False),
    "qwen2": dict(architecture="Qwen2ForCausalLM", moe=False, qk_norm=False, bias_key=False, bias_default=True, has_window=True),
    "qwen2_moe": dict(architecture="Qwen2MoeForCausalLM", moe=True, qk_norm=False, bias_key=False, bias_default=True, has_window=True),
    "llama": dict(architecture="LlamaForCausalLM", moe=False, qk_norm=False, bias_key=True, bias_default=False, has_window=False),
    "mistral": dict(architecture="MistralForCausalLM", moe=False, qk_norm=False, bias_key=False, bias_default=False, has_window=True),
    "mixtral": dict(architecture="MixtralForCausalLM", moe=True, qk_norm=False, bias_key=False, bias_default=False, has_window=True),
    # sigmoid scores with a selection bias and group-limited top-k, always-on shared experts, leading dense layers,
    # rotary embedding on the first half of every head
    # one RMSNorm over the whole q (and k) projection instead of one per head; top-k weights not renormalised
    "olmoe": dict(architecture="OlmoeForCausalLM", moe=True, qk_norm=True, bias_key=True, bias_default=False, has_window=False),
    "glm4_moe": dict(architecture="Glm4MoeForCausalLM", moe=True, qk_norm=True, bias_key=True, bias_default=False, has_window=False),
    # a learned sink logit per head, windowed and full layers in turn, biases on every projection and on the experts,
    # a clamped GLU in the experts, a biased router that takes the softmax of the top-k logits
    # multi-head latent attention (queries and keys / values through low-rank bottlenecks, rotary embedding on a separate
    # slice shared by all heads) in front of the sigmoid-routed, group-limited MoE with shared experts
    # Gemma 3 (text): five windowed layers per full one with their own rotary base, norms before AND after both blocks
    # with weights stored as (w - 1), tanh-GELU gating, embeddings scaled by sqrt(hidden), a configured softmax scale
    # Gemma 2: the same block as Gemma 3 without q / k norms and with one rotary base, plus tanh soft-capping of the
    # attention scores and of the output logits
    "gemma2": dict(architecture="Gemma2ForCausalLM", moe=False, qk_norm=False, bias_key=True, bias_default=False, has_window=True),
    "gemma3_text": dict(architecture="Gemma3ForCausalLM", moe=False, qk_norm=True, bias_key=True, bias_default=False, has_window=True),
    "deepseek_v3": dict(architecture="DeepseekV3ForCausalLM", moe=True, qk_norm=False, bias_key=True, bias_default=False, has_window=False),
    # GLM-4.7-Flash: the DeepSeek-V3 block with its dense layers named one by one (``mlp_layer_types``)
    "glm4_moe_lite": dict(architecture="Glm4MoeLiteForCausalLM", moe=True, qk_norm=False, bias_key=True, bias_default=False, has_window=False),
    # GLM-5 (DSA): the GLM-4.7-Flash block whose attention sees, per query, only the ``index_topk`` keys a small indexer
    # ranks highest; rotary pairs stored in halves, plain softmax scale
    "glm_moe_dsa": dict(architecture="GlmMoeDsaForCausalLM", moe=True, qk_norm=False, bias_key=True, bias_default=False, has_window=False),
    # Mistral 4: the DeepSeek-V3 block (latent attention, shared experts, group-limited routing) with softmax router
    # scores, expert banks stored whole, and queries scaled by 1 + beta * log(1 + floor(position / period))
    "mistral4": dict(architecture="Mistral4ForCausalLM", moe=True, qk_norm=False, bias_key=True, bias_default=False, has_window=False),
    # Qwen3-Next: gated delta-rule linear attention in the layers ``layer_types`` names ``linear_attention``, attention with
    # an output gate, a quarter of each head rotated and norms stored around zero in the others; Qwen2-MoE's gated shared expert
    "qwen3_next": dict(architecture="Qwen3NextForCausalLM", moe=True, qk_norm=True, bias_key=True, bias_default=False, has_window=False),
    # Qwen3.5-MoE (text tower): Qwen3-Next's layers with the linear-attention projections stored one per role, every layer
    # sparse, router weights always renormalised, and tensors named under ``model.language_model``
    "qwen3_5_moe_text": dict(architecture="Qwen3_5MoeForCausalLM", moe=True, qk_norm=True, bias_key=True, bias_default=False, has_window=False),
    # LFM2-MoE: gated short-convolution mixers in the layers ``layer_types`` names ``conv``, attention with per-head q / k
    # norms in the others; sigmoid router scores ranked with a stored per-expert bias; leading dense layers
    "lfm2_moe": dict(architecture="Lfm2MoeForCausalLM", moe=True, qk_norm=True, bias_key=False, bias_default=False, has_window=False),
    "gpt_oss": dict(architecture="GptOssForCausalLM", moe=True, qk_norm=False, bias_key=True, bias_default=True, has_window=True),
}


@dataclass
class ModelConfig:
    vocab_size: int = 151936
    hidden_size: int = 2048
    num_hidden_layers: int = 48
    num_attention_heads: int = 32
    num_key_value_heads: int = 4
    head_dim: int = 128
    intermediate_size: int = 6144          # dense FFN width (dense layers / dense models)
    moe_intermediate_size: int = 768       # width of one routed expert
    num_experts: int = 0                   # 0 = dense model
    num_experts_per_tok: int = 8
    norm_topk_prob: bool = True
    shared_expert_intermediate_size: int = 0
    shared_expert_gate: bool = False
    mlp_only_layers: list[int] = field(default_factory=list)
    decoder_sparse_step: int = 1
    rope_theta: float = 1e6
    rms_norm_eps: float = 1e-6
    use_qk_norm: bool = True
    qk_norm_whole_width: bool = False      # the q / k norm spans all heads of the projection (OLMoE) instead of one head
    attention_bias: bool = False           # bias on the q / k / v projections (Qwen2)
    partial_rotary_factor: float = 1.0     # share of every head's dims that the rotary embedding turns (the leading ones)
    score_function: str = "softmax"        # "softmax" | "sigmoid" (scores of the router)
    router_bias: bool = False              # a stored per-expert selection bias (``e_score_correction_bias``) ranks the experts
    n_group: int = 1                       # group-limited routing: experts in ``n_group`` groups, ``topk_group`` of them eligible
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    norm_topk_eps: float = 1e-20           # added to the sum the chosen weights are divided by (group-limited path)
    index_topk: int = 0                    # > 0: sparse attention - an indexer picks this many keys per query (GLM-5 / DeepSeek-V3.2 style)
    index_n_heads: int = 0
    index_head_dim: int = 0
    attn_output_gate: bool = False         # attention output times sigmoid(gate); the gate rides in the query projection (Qwen3-Next)
    linear_num_key_heads: int = 0          # gated delta-rule layers (``layer_types`` entry "linear_attention"): heads and widths
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 0
    linear_value_head_dim: int = 0
    linear_conv_kernel_dim: int = 4
    conv_kernel: int = 0                   # taps of the short-convolution mixer in the layers ``layer_types`` names "conv" (LFM2)
    query_scale_beta: float = 0.0          # > 0: queries times 1 + beta * log(1 + floor(position / query_scale_period)) (Mistral 4)
    query_scale_period: int = 0
    sliding_window: int = 0                # > 0: every query sees only its last ``sliding_window`` keys (Mistral-style)
    hidden_activation: str = "silu"        # gate activation of the dense feed-forward block: "silu" | "gelu_tanh"
    sandwich_norms: bool = False           # an RMSNorm on the output of each block too (Gemma): four norms per layer
    norm_unit_offset: bool = False         # the checkpoint stores norm weights as (w - 1); at run time they are plain weights
    embedding_multiplier: float = 1.0      # token embeddings are scaled by this (Gemma: sqrt(hidden_size))
    query_pre_attn_scalar: int = 0         # softmax scale = this ** -0.5 (0 = head_dim)
    attn_logit_softcapping: float = 0.0    # > 0: attention scores pass through cap * tanh(. / cap) before the mask (Gemma 2)
    final_logit_softcapping: float = 0.0   # > 0: the same on the output logits
    rope_local_theta: float = 0.0          # rotary base of the windowed layers when it differs from the full layers' (0 = the same)
    kv_lora_rank: int = 0                  # > 0: multi-head latent attention (DeepSeek); keys / values come from this many latent dims
    q_lora_rank: int = 0                   # latent dims of the query bottleneck (0 = one plain query projection)
    qk_nope_head_dim: int = 0              # per head: dims of q / k without rotary embedding ...
    qk_rope_head_dim: int = 0              # ... and with it (the key's rotary slice is shared by all heads); equals ``head_dim``
    v_head_dim: int = 0
    rope_interleave: bool = True           # the checkpoint stores rotary pairs interleaved (even, odd) instead of in halves
    layer_types: list[str] | None = None   # per layer "sliding_attention" | "full_attention"; None = the window on every layer
    attention_sinks: bool = False          # one learned logit per head joins every softmax (gpt-oss)
    output_bias: bool = False              # bias on the attention output projection too (gpt-oss)
    router_logit_bias: bool = False        # a trained bias on the router's logits (gpt-oss), unlike the selection bias
    expert_bias: bool = False              # per-expert bias vectors on both expert projections
    expert_activation: str = "swiglu"      # "swiglu" | "clamped_glu": gate * sigmoid(1.702 gate) * (up + 1), both clamped
    glu_limit: float = 7.0
    rope_scaling: dict | None = None       # Hugging Face ``rope_scaling`` / ``rope_parameters`` entry, None = plain
    num_nextn_predict_layers: int = 0      # 1 = a multi-token-prediction head trained beside the next-token loss
    mtp_loss_weight: float = 0.3
    mtp_objective: str = "joint"           # "joint": the head's loss also reaches the trunk; "detached": it does not
    hc_mult: int = 1                       # residual streams per token (1 = the plain residual; > 1 = hyper-connections)
    hc_kind: str = "mhc"                   # "mhc": Sinkhorn-projected mixing matrices; "gated": per-stream norm + gated mean + inject
    hc_sinkhorn_iters: int = 20
    hc_eps: float = 1e-6
    hc_mix_rank: int = 16                  # rank of the gated variant's gate projection
    tie_word_embeddings: bool = False
    router_aux_loss_coef: float = 0.0
    initializer_range: float = 0.02
    max_position_embeddings: int = 262144
    model_type: str = "qwen3_moe"

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def grouped_routing(self) -> bool:
        """The router ranks through the group-limited path (tensor ops) instead of the plain softmax top-k kernel."""
        return self.score_function == "sigmoid" or self.n_group > 1 or self.routed_scaling_factor != 1.0

    def layer_is_conv(self, i: int) -> bool:
        """The layer's mixer is a gated short convolution instead of attention."""
        return bool(self.layer_types) and i < len(self.layer_types) and self.layer_types[i] == "conv"

    def layer_is_linear_attention(self, i: int) -> bool:
        """The layer's mixer is the gated delta-rule recurrence instead of attention."""
        return bool(self.layer_types) and i < len(self.layer_types) and self.layer_types[i] == "linear_attention"

    def layer_is_moe(self, i: int) -> bool:
        return self.is_moe and i not in self.mlp_only_layers and (i + 1) % self.decoder_sparse_step == 0

    @property
    def qkv_dim(self) -> int:
        return (self.num_attention_heads + 2 * self.num_key_value_heads) * self.head_dim

    # ---- parameter counts (for MFU and memory planning) ---------------------------------
    def param_counts(self) -> dict[str, int]:
        H, D = self.hidden_size, self.head_dim
        norm_width = (self.num_attention_heads + self.num_key_value_heads) * D if self.qk_norm_whole_width else 2 * D
        if self.kv_lora_rank:
            Hq, dqk = self.num_attention_heads, self.qk_nope_head_dim + self.qk_rope_head_dim
            q_side = (H * self.q_lora_rank + self.q_lora_rank + self.q_lora_rank * Hq * dqk) if self.q_lora_rank else H * Hq * dqk
            attn = (q_side + H * (self.kv_lora_rank + self.qk_rope_head_dim) + self.kv_lora_rank
                    + self.kv_lora_rank * Hq * (self.qk_nope_head_dim + self.v_head_dim) + Hq * self.v_head_dim * H + 2 * H)
            if self.index_topk:
                attn += (self.q_lora_rank * self.index_n_heads * self.index_head_dim + H * self.index_head_dim + 2 * self.index_head_dim
                         + H * self.index_n_heads)
        else:
            attn = (H * self.qkv_dim + self.num_attention_heads * D * H + (norm_width if self.use_qk_norm else 0) + 2 * H
                    + (2 * H if self.sandwich_norms else 0) + (self.qkv_dim if self.attention_bias else 0) + (H if self.output_bias else 0)
                    + (self.num_attention_heads if self.attention_sinks else 0))
        dense_mlp = 3 * H * self.intermediate_size
        expert = 3 * H * self.moe_intermediate_size + ((2 * self.moe_intermediate_size + H) if self.expert_bias else 0)
        shared = 3 * H * self.shared_expert_intermediate_size + (H if self.shared_expert_gate else 0)
        shared += self.num_experts if self.router_bias else 0
        shared += self.num_experts if self.router_logit_bias else 0
        total = active = 0
        conv_mixer = 4 * H * H + H * self.conv_kernel + 2 * H        # in / out projections, taps, the layer's two norms
        key_dim, value_dim = self.linear_num_key_heads * self.linear_key_head_dim, self.linear_num_value_heads * self.linear_value_head_dim
        linear_mixer = (H * (2 * key_dim + 2 * value_dim) + H * 2 * self.linear_num_value_heads
                        + (2 * key_dim + value_dim) * self.linear_conv_kernel_dim + 2 * self.linear_num_value_heads
                        + self.linear_value_head_dim + value_dim * H + 2 * H)
        if self.attn_output_gate:
            attn += H * self.num_attention_heads * D
        for i in range(self.num_hidden_layers):
            mixer = conv_mixer if self.layer_is_conv(i) else linear_mixer if self.layer_is_linear_attention(i) else attn
            if self.layer_is_moe(i):
                total += mixer + self.num_experts * expert + self.num_experts * H + shared
                active += mixer + self.num_experts_per_tok * expert + self.num_experts * H + shared
            else:
                total += mixer + dense_mlp
                active += mixer + dense_mlp
        if self.num_nextn_predict_layers:
            L = self.num_hidden_layers
            moe = self.layer_is_moe(L)
            block = attn + (self.num_experts * expert + self.num_experts * H + shared if moe else dense_mlp)
            block_active = attn + (self.num_experts_per_tok * expert + self.num_experts * H + shared if moe else dense_mlp)
            total += block + 2 * H * H + 3 * H
            active += block_active + 2 * H * H + 3 * H
        if self.hc_mult > 1:
            n = self.hc_mult
            per_layer = (2 * ((2 * n + n * n) * (n * H + 1) + 3) if self.hc_kind == "mhc"
                         else 2 * (n * H + 2 * self.hc_mix_rank * n * H + n * n * H))
            head_collapse = n * n * H + n + 1 if self.hc_kind == "mhc" else 0
            total += self.num_hidden_layers * per_layer + head_collapse
            active += self.num_hidden_layers * per_layer + head_collapse
        emb = self.vocab_size * H
        head = 0 if self.tie_word_embeddings else emb
        return {"total": total + emb + head + H, "active": active + head + H, "embedding": emb,
                "expert_total": sum(self.num_experts * expert for i in range(self.num_hidden_layers) if self.layer_is_moe(i))}

    # ---- Hugging Face interchange -------------------------------------------------------
    def to_hf_dict(self) -> dict:
        fam = FAMILIES[self.family]
        rope = {"rope_type": "default", "rope_theta": self.rope_theta}
        if self.rope_scaling:
            rope = {**self.rope_scaling, "rope_theta": self.rope_theta}
            rope.setdefault("rope_type", rope.pop("type", "default"))
        d = {
            "architectures": [fam["architecture"]],
            "model_type": self.family,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "hidden_act": "silu",
            "rope_theta": self.rope_theta,
            "rope_parameters": rope,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_dropout": 0.0,
            "initializer_range": self.initializer_range,
            "max_position_embeddings": self.max_position_embeddings,
            "torch_dtype": "bfloat16",
            "use_cache": False,
        }
        if self.rope_scaling:
            d["rope_scaling"] = {k: v for k, v in rope.items() if k != "rope_theta"}
        if self.num_nextn_predict_layers:
            d.update({"num_nextn_predict_layers": self.num_nextn_predict_layers, "mtp_loss_weight": self.mtp_loss_weight,
                      "mtp_objective": self.mtp_objective})
        if self.hc_mult > 1:
            d.update({"hc_mult": self.hc_mult, "hc_kind": self.hc_kind, "hc_sinkhorn_iters": self.hc_sinkhorn_iters,
                      "hc_eps": self.hc_eps, "hc_mix_rank": self.hc_mix_rank})
        if fam["bias_key"]:
            d["attention_bias"] = self.attention_bias
        elif self.family == "qwen2_moe":
            d["qkv_bias"] = self.attention_bias
        if fam["has_window"]:
            d["sliding_window"] = self.sliding_window or None
            if self.family.startswith("qwen2"):
                d["use_sliding_window"] = bool(self.sliding_window)
                first_windowed = (self.layer_types or ["sliding_attention"]).index("sliding_attention") if self.sliding_window else 0
                if self.layer_types and "full_attention" in self.layer_types[first_windowed:]:
                    raise ValueError("Qwen2 stores its full-attention layers as a leading run (max_window_layers)")
                d["max_window_layers"] = first_windowed if self.sliding_window else self.num_hidden_layers
                if self.sliding_window and self.layer_types:
                    d["layer_types"] = list(self.layer_types)
        if self.family in ("gemma2", "gemma3_text"):
            d.pop("hidden_act", None)
            d.update({"hidden_activation": "gelu_pytorch_tanh", "query_pre_attn_scalar": self.query_pre_attn_scalar or self.head_dim,
                      "attn_logit_softcapping": self.attn_logit_softcapping or None,
                      "final_logit_softcapping": self.final_logit_softcapping or None,
                      "layer_types": list(self.layer_types or ["sliding_attention" if self.sliding_window else "full_attention"]
                                          * self.num_hidden_layers)})
            if self.family == "gemma3_text":
                for key in ("rope_theta", "rope_scaling"):
                    d.pop(key, None)
                full = d.pop("rope_parameters")
                d["rope_parameters"] = {"full_attention": full, "sliding_attention": {
                    "rope_type": "default", "rope_theta": self.rope_local_theta or self.rope_theta}}
        elif self.family == "gpt_oss":
            d.update({"num_local_experts": self.num_experts, "num_experts_per_tok": self.num_experts_per_tok,
                      "intermediate_size": self.moe_intermediate_size, "router_aux_loss_coef": self.router_aux_loss_coef,
                      "output_router_logits": False, "swiglu_limit": self.glu_limit,
                      "layer_types": list(self.layer_types or ["sliding_attention" if self.sliding_window else "full_attention"]
                                          * self.num_hidden_layers)})
        elif self.family in ("glm4_moe", "deepseek_v3", "mistral4", "glm4_moe_lite", "glm_moe_dsa"):
            first_dense = 0
            while first_dense in self.mlp_only_layers:
                first_dense += 1
            if self.family not in ("glm4_moe_lite", "glm_moe_dsa") and sorted(self.mlp_only_layers) != list(range(first_dense)):
                raise ValueError("glm4_moe stores its dense layers as a leading run (first_k_dense_replace)")
            d.update({"moe_intermediate_size": self.moe_intermediate_size, "n_routed_experts": self.num_experts,
                      "num_experts_per_tok": self.num_experts_per_tok, "norm_topk_prob": self.norm_topk_prob,
                      "n_shared_experts": self.shared_expert_intermediate_size // max(self.moe_intermediate_size, 1),
                      "n_group": self.n_group, "topk_group": self.topk_group, "first_k_dense_replace": first_dense,
                      "routed_scaling_factor": self.routed_scaling_factor, "use_qk_norm": self.use_qk_norm,
                      "partial_rotary_factor": self.partial_rotary_factor})
            if self.family == "glm4_moe":
                d["rope_parameters"]["partial_rotary_factor"] = self.partial_rotary_factor
            else:
                for key in ("use_qk_norm", "partial_rotary_factor"):
                    d.pop(key)
                d.update({"kv_lora_rank": self.kv_lora_rank, "q_lora_rank": self.q_lora_rank or None,
                          "qk_nope_head_dim": self.qk_nope_head_dim, "qk_rope_head_dim": self.qk_rope_head_dim,
                          "v_head_dim": self.v_head_dim, "rope_interleave": self.rope_interleave,
                          "head_dim": self.qk_rope_head_dim})
                if self.family == "glm_moe_dsa":
                    if self.rope_interleave:
                        raise ValueError("glm_moe_dsa stores its rotary pairs in halves (rope_interleave False)")
                    d.pop("rope_interleave")
                    d.update({"index_topk": self.index_topk, "index_n_heads": self.index_n_heads, "index_head_dim": self.index_head_dim})
                if self.family in ("glm4_moe_lite", "glm_moe_dsa"):
                    d.pop("first_k_dense_replace")
                    d["mlp_layer_types"] = ["dense" if i in self.mlp_only_layers else "sparse" for i in range(self.num_hidden_layers)]
                if self.family == "mistral4":
                    # a head is the un-rotated and the rotated slice together; the rotary table covers the rotated share
                    whole = self.qk_nope_head_dim + self.qk_rope_head_dim
                    d["head_dim"] = whole
                    d.pop("rope_scaling", None)
                    d.pop("rope_theta", None)
                    d["rope_parameters"] = dict(d["rope_parameters"], partial_rotary_factor=self.qk_rope_head_dim / whole)
                    stored = d["rope_parameters"].get("original_max_position_embeddings")
                    if self.query_scale_beta and stored and int(stored) != self.query_scale_period:
                        raise ValueError("mistral4 stores ONE original_max_position_embeddings: the period of the query stretch "
                                         f"({self.query_scale_period}) must equal the rotary scaling's ({stored})")
                    # the release's code reads both keys unconditionally: a zero beta is written, not left out
                    d["rope_parameters"]["llama_4_scaling_beta"] = self.query_scale_beta
                    d["rope_parameters"].setdefault("original_max_position_embeddings",
                                                    self.query_scale_period or self.max_position_embeddings)
        elif self.family == "lfm2_moe":
            first_dense = 0
            while first_dense in self.mlp_only_layers:
                first_dense += 1
            if sorted(self.mlp_only_layers) != list(range(first_dense)):
                raise ValueError("lfm2_moe stores its dense layers as a leading run (num_dense_layers)")
            for key in ("rms_norm_eps", "rope_theta", "rope_scaling", "hidden_act", "attention_dropout"):
                d.pop(key, None)
            if self.head_dim * self.num_attention_heads == self.hidden_size:
                d.pop("head_dim")
            d.update({"norm_eps": self.rms_norm_eps, "num_dense_layers": first_dense, "num_experts": self.num_experts,
                      "num_experts_per_tok": self.num_experts_per_tok, "moe_intermediate_size": self.moe_intermediate_size,
                      "use_expert_bias": self.router_bias, "routed_scaling_factor": self.routed_scaling_factor,
                      "norm_topk_prob": self.norm_topk_prob, "conv_bias": False, "conv_L_cache": self.conv_kernel,
                      "layer_types": list(self.layer_types or ["full_attention"] * self.num_hidden_layers)})
        elif self.family == "olmoe":
            d.update({"num_experts": self.num_experts, "num_experts_per_tok": self.num_experts_per_tok,
                      "norm_topk_prob": self.norm_topk_prob, "intermediate_size": self.moe_intermediate_size, "clip_qkv": None,
                      "router_aux_loss_coef": self.router_aux_loss_coef, "output_router_logits": False})
        elif self.family == "mixtral":
            d.update({"num_local_experts": self.num_experts, "num_experts_per_tok": self.num_experts_per_tok,
                      "router_aux_loss_coef": self.router_aux_loss_coef, "output_router_logits": False,
                      "intermediate_size": self.moe_intermediate_size})
        elif self.is_moe:
            d.update({
                "moe_intermediate_size": self.moe_intermediate_size,
                "num_experts": self.num_experts,
                "num_experts_per_tok": self.num_experts_per_tok,
                "norm_topk_prob": self.norm_topk_prob,
                "decoder_sparse_step": self.decoder_sparse_step,
                "mlp_only_layers": list(self.mlp_only_layers),
                "router_aux_loss_coef": self.router_aux_loss_coef,
                "output_router_logits": False,
            })
            if self.shared_expert_intermediate_size:
                d["shared_expert_intermediate_size"] = self.shared_expert_intermediate_size
            if self.family == "qwen3_5_moe_text":
                if self.mlp_only_layers or self.decoder_sparse_step != 1 or not self.norm_topk_prob:
                    raise ValueError("qwen3_5_moe_text: every layer is sparse and the router always renormalises")
                for key in ("decoder_sparse_step", "mlp_only_layers", "norm_topk_prob"):
                    d.pop(key, None)
            if self.family in ("qwen3_next", "qwen3_5_moe_text"):
                d.update({"layer_types": list(self.layer_types or ["full_attention"] * self.num_hidden_layers),
                          "linear_num_key_heads": self.linear_num_key_heads, "linear_num_value_heads": self.linear_num_value_heads,
                          "linear_key_head_dim": self.linear_key_head_dim, "linear_value_head_dim": self.linear_value_head_dim,
                          "linear_conv_kernel_dim": self.linear_conv_kernel_dim, "partial_rotary_factor": self.partial_rotary_factor})
                d["rope_parameters"] = dict(d["rope_parameters"], partial_rotary_factor=self.partial_rotary_factor)
        return d

    @property
    def family(self) -> str:
        """The Hugging Face ``model_type`` this configuration is written as."""
        if self.model_type in FAMILIES and FAMILIES[self.model_type]["moe"] == self.is_moe:
            return self.model_type
        return "qwen3_moe" if self.is_moe else "qwen3"

    @classmethod
    def from_hf_dict(cls, d: dict) -> "ModelConfig":
        mt = d.get("model_type", "qwen3")
        if mt == "qwen3_5_moe" and "text_config" in d:
            # the multimodal release: its text tower is the model here (the tensors carry the same names either way)
            d = dict(d["text_config"], tie_word_embeddings=d.get("tie_word_embeddings", d["text_config"].get("tie_word_embeddings", False)))
            mt = d["model_type"] = "qwen3_5_moe_text"
        if mt not in FAMILIES:
            raise ValueError(f"model_type {mt!r} has no family registered here (known: {sorted(FAMILIES)})")
        fam = FAMILIES[mt]
        window = d.get("sliding_window") or 0
        if not (fam["has_window"] and window and d.get("use_sliding_window", True) and window < d.get("max_position_embeddings", 0)):
            window = 0
        kinds = None
        if window and mt.startswith("qwen2") and d.get("max_window_layers", 0) not in (0, None):
            # Qwen2 windows only the layers from ``max_window_layers`` on
            first = int(d["max_window_layers"])
            if first >= d["num_hidden_layers"]:
                window = 0
            else:
                kinds = ["full_attention"] * first + ["sliding_attention"] * (d["num_hidden_layers"] - first)
        rp = d.get("rope_parameters") or {}
        local_theta = 0.0
        if "full_attention" in rp:             # one entry per layer kind (Gemma 3)
            local_theta = float((rp.get("sliding_attention") or {}).get("rope_theta", 0.0))
            rp = rp["full_attention"]
        rope_theta = d.get("rope_theta") or rp.get("rope_theta", 1e6 if mt.startswith("qwen") else 1e4)
        scaling = d.get("rope_scaling") or ({k: v for k, v in rp.items() if k not in ("rope_theta", "partial_rotary_factor")} if rp else None)
        if scaling:
            scaling = dict(scaling)
            scaling.setdefault("rope_type", scaling.pop("type", "default"))
            if scaling["rope_type"] == "default":
                scaling = None
        hd = d.get("head_dim") or d["hidden_size"] // d["num_attention_heads"]
        extra = {}
        if mt in ("deepseek_v3", "mistral4", "glm4_moe_lite", "glm_moe_dsa"):
            n_exp, width, dense_width = d["n_routed_experts"], d["moe_intermediate_size"], d["intermediate_size"]
            topk, renorm = d.get("num_experts_per_tok", 8 if mt == "deepseek_v3" else 4), d.get("norm_topk_prob", True)
            hd = int(d.get("qk_rope_head_dim", 64))            # the rotary table is built for the rotary slice
            routing = dict(score_function="sigmoid", router_bias=True)
            if mt == "mistral4":
                routing = dict(score_function="softmax", router_bias=False)
                beta = float(rp.get("llama_4_scaling_beta") or 0.0)
                if beta:
                    routing.update(query_scale_beta=beta, query_scale_period=int(rp["original_max_position_embeddings"]))
                if scaling:
                    for key in ("llama_4_scaling_beta", "max_position_embeddings"):
                        scaling.pop(key, None)
            extra = dict(**routing, n_group=int(d.get("n_group", 1)),
                         topk_group=int(d.get("topk_group", 1)), routed_scaling_factor=float(d.get("routed_scaling_factor", 1.0)),
                         shared_expert_intermediate_size=int(d.get("n_shared_experts", 0) or 0) * width,
                         mlp_only_layers=([i for i, kind in enumerate(d.get("mlp_layer_types") or (["dense"] + ["sparse"] * (d["num_hidden_layers"] - 1) if mt == "glm4_moe_lite" else
                                                                                                   ["dense"] * min(3, d["num_hidden_layers"]) + ["sparse"] * max(d["num_hidden_layers"] - 3, 0)))
                                           if kind == "dense"] if mt in ("glm4_moe_lite", "glm_moe_dsa") else list(range(int(d.get("first_k_dense_replace", 0))))),
                         use_qk_norm=False, kv_lora_rank=int(d["kv_lora_rank"]), q_lora_rank=int(d.get("q_lora_rank") or 0),
                         qk_nope_head_dim=int(d["qk_nope_head_dim"]), qk_rope_head_dim=hd, v_head_dim=int(d["v_head_dim"]),
                         rope_interleave=bool(d.get("rope_interleave", mt != "glm_moe_dsa")))
            if mt == "glm_moe_dsa":
                extra.update(index_topk=int(d.get("index_topk", 2048)), index_n_heads=int(d.get("index_n_heads", 32)),
                             index_head_dim=int(d.get("index_head_dim", 128)))
        elif mt in ("qwen3_next", "qwen3_5_moe_text"):
            n_exp, width, dense_width = d.get("num_experts", 0), d.get("moe_intermediate_size", 0), d.get("intermediate_size", 0)
            topk, renorm = d.get("num_experts_per_tok", 10), d.get("norm_topk_prob", True)
            every = int(d.get("full_attention_interval", 4))
            extra = dict(layer_types=list(d.get("layer_types") or ["full_attention" if (i + 1) % every == 0 else "linear_attention"
                                                                    for i in range(d["num_hidden_layers"])]),
                         partial_rotary_factor=float(d.get("partial_rotary_factor", rp.get("partial_rotary_factor", 0.25))),
                         attn_output_gate=True, norm_unit_offset=True, shared_expert_gate=bool(d.get("shared_expert_intermediate_size", 0)),
                         linear_num_key_heads=int(d.get("linear_num_key_heads", 16)), linear_num_value_heads=int(d.get("linear_num_value_heads", 32)),
                         linear_key_head_dim=int(d.get("linear_key_head_dim", 128)), linear_value_head_dim=int(d.get("linear_value_head_dim", 128)),
                         linear_conv_kernel_dim=int(d.get("linear_conv_kernel_dim", 4)))
        elif mt == "lfm2_moe":
            if d.get("conv_bias"):
                raise ValueError("lfm2_moe with conv_bias: the biased convolution and projections are not built")
            n_exp, width, dense_width = d["num_experts"], d["moe_intermediate_size"], d["intermediate_size"]
            topk, renorm = d.get("num_experts_per_tok", 4), d.get("norm_topk_prob", True)
            extra = dict(score_function="sigmoid", router_bias=bool(d.get("use_expert_bias", True)), norm_topk_eps=1e-6,
                         routed_scaling_factor=float(d.get("routed_scaling_factor", 1.0)),
                         mlp_only_layers=list(range(int(d.get("num_dense_layers", 2)))), rms_norm_eps=float(d.get("norm_eps", 1e-5)),
                         conv_kernel=int(d.get("conv_L_cache", 3)), layer_types=list(d["layer_types"]),
                         tie_word_embeddings=bool(d.get("tie_word_embeddings", d.get("tie_embedding", True))))
        elif mt == "glm4_moe":
            n_exp, width, dense_width = d["n_routed_experts"], d["moe_intermediate_size"], d["intermediate_size"]
            topk, renorm = d.get("num_experts_per_tok", 8), d.get("norm_topk_prob", True)
            extra = dict(partial_rotary_factor=float(d.get("partial_rotary_factor", rp.get("partial_rotary_factor", 0.5))),
                         score_function="sigmoid", router_bias=True, n_group=int(d.get("n_group", 1)),
                         topk_group=int(d.get("topk_group", 1)), routed_scaling_factor=float(d.get("routed_scaling_factor", 1.0)),
                         shared_expert_intermediate_size=int(d.get("n_shared_experts", 0) or 0) * width,
                         mlp_only_layers=list(range(int(d.get("first_k_dense_replace", 0)))), use_qk_norm=bool(d.get("use_qk_norm", False)))
        elif mt in ("gemma2", "gemma3_text"):
            if d.get("use_bidirectional_attention"):
                raise ValueError("bidirectional attention is not built")
            n_exp, width, dense_width = 0, 0, d["intermediate_size"]
            topk, renorm = 8, True
            every = 6 if mt == "gemma3_text" else 2          # one full layer per this many
            kinds = list(d.get("layer_types") or ["full_attention" if (i + 1) % every == 0 else "sliding_attention"
                                                   for i in range(d["num_hidden_layers"])])
            if "sliding_attention" not in kinds:
                window = 0
            theta = float(rp.get("rope_theta", 1e6))
            extra = dict(layer_types=kinds if window else None, hidden_activation="gelu_tanh", sandwich_norms=True, norm_unit_offset=True,
                         embedding_multiplier=float(d["hidden_size"]) ** 0.5,
                         query_pre_attn_scalar=int(d.get("query_pre_attn_scalar", 256)),
                         rope_local_theta=local_theta if window and local_theta and local_theta != theta else 0.0,
                         attn_logit_softcapping=float(d.get("attn_logit_softcapping") or 0.0),
                         final_logit_softcapping=float(d.get("final_logit_softcapping") or 0.0),
                         tie_word_embeddings=d.get("tie_word_embeddings", True))
        elif mt == "gpt_oss":
            n_exp, width, dense_width = d.get("num_local_experts", 128), d["intermediate_size"], d["intermediate_size"]
            topk, renorm = d.get("num_experts_per_tok", 4), True
            kinds = list(d.get("layer_types") or ["sliding_attention" if i % 2 == 0 else "full_attention"
                                                   for i in range(d["num_hidden_layers"])])
            if "sliding_attention" not in kinds:
                window = 0
            extra = dict(layer_types=kinds if window else None, attention_sinks=True, output_bias=bool(d.get("attention_bias", True)),
                         router_logit_bias=True, expert_bias=True, expert_activation="clamped_glu",
                         glu_limit=float(d.get("swiglu_limit", 7.0)))
        elif mt == "olmoe":
            if d.get("clip_qkv"):
                raise ValueError("an OLMoE checkpoint with clip_qkv set: clamping the projections is not built")
            n_exp, width, dense_width = d.get("num_experts", 64), d["intermediate_size"], d["intermediate_size"]
            topk, renorm = d.get("num_experts_per_tok", 8), d.get("norm_topk_prob", False)
            extra = dict(qk_norm_whole_width=True)
        elif mt == "mixtral":
            n_exp, width, dense_width = d.get("num_local_experts", 8), d["intermediate_size"], d["intermediate_size"]
            topk, renorm = d.get("num_experts_per_tok", 2), True
        else:
            n_exp = d.get("num_experts", 0) if fam["moe"] else 0
            width, dense_width = d.get("moe_intermediate_size", 0), d.get("intermediate_size", 0)
            topk, renorm = d.get("num_experts_per_tok", 8), d.get("norm_topk_prob", mt != "qwen2_moe")
        fields = dict(
            vocab_size=d["vocab_size"], hidden_size=d["hidden_size"], num_hidden_layers=d["num_hidden_layers"],
            num_attention_heads=d["num_attention_heads"],
            num_key_value_heads=d.get("num_key_value_heads", d["num_attention_heads"]), head_dim=hd,
            intermediate_size=dense_width, moe_intermediate_size=width,
            num_experts=n_exp, num_experts_per_tok=topk, norm_topk_prob=renorm,
            shared_expert_intermediate_size=d.get("shared_expert_intermediate_size", 0) or 0,
            shared_expert_gate=(mt == "qwen2_moe"),
            mlp_only_layers=list(d.get("mlp_only_layers", []) or []), decoder_sparse_step=d.get("decoder_sparse_step", 1),
            rope_theta=float(rope_theta), rms_norm_eps=d.get("rms_norm_eps", 1e-6), use_qk_norm=fam["qk_norm"],
            sliding_window=int(window), layer_types=kinds,
            attention_bias=(bool(d.get("attention_bias", False)) if fam["bias_key"]
                            else bool(d.get("qkv_bias", fam["bias_default"]))),
            num_nextn_predict_layers=int(d.get("num_nextn_predict_layers", 0) or 0),
            mtp_loss_weight=float(d.get("mtp_loss_weight", 0.3)), mtp_objective=d.get("mtp_objective", "joint"),
            rope_scaling=scaling, hc_mult=int(d.get("hc_mult", 1)), hc_sinkhorn_iters=int(d.get("hc_sinkhorn_iters", 20)),
            hc_eps=float(d.get("hc_eps", 1e-6)), hc_kind=d.get("hc_kind", "mhc"), hc_mix_rank=int(d.get("hc_mix_rank", 16)),
            tie_word_embeddings=d.get("tie_word_embeddings", False),
            router_aux_loss_coef=d.get("router_aux_loss_coef", 0.0), initializer_range=d.get("initializer_range", 0.02),
            max_position_embeddings=d.get("max_position_embeddings", 262144), model_type=mt,
        )
        fields.update(extra)
        return cls(**fields)

    def save(self, directory: str | Path) -> None:
        Path(directory).mkdir(parents=True, exist_ok=True)
        (Path(directory) / "config.json").write_text(json.dumps(self.to_hf_dict(), indent=2))

    @classmethod
    def load(cls, directory: str | Path) -> "ModelConfig":
        return cls.from_hf_dict(json.loads((Path(directory) / "config.json").read_text()))

    def asdict(self) -> dict:
        return asdict(self)


def tiny_moe_config() -> ModelConfig:
    """4 layers, hidden 256, 4 query / 2 kv heads of 64, 8 experts of width 128, top-2, vocab 4096."""
    return ModelConfig(vocab_size=4096, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, intermediate_size=512, moe_intermediate_size=128,
                       num_experts=8, num_experts_per_tok=2, rope_theta=1e6, rms_norm_eps=1e-6)


def dense_9b_config() -> ModelConfig:
    """36 layers, hidden 4096, 32 query / 8 kv heads of 128, SwiGLU FFN 12288."""
    return ModelConfig(hidden_size=4096, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
                       head_dim=128, intermediate_size=12288, num_experts=0, model_type="qwen3")


def moe_30b_a3b_config() -> ModelConfig:
    """48 layers, hidden 2048, 32 query / 4 kv heads of 128, 128 experts of width 768, top-8."""
    return ModelConfig(hidden_size=2048, num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4,
                       head_dim=128, intermediate_size=6144, moe_intermediate_size=768, num_experts=128,
                       num_experts_per_tok=8)


def moe_120b_config() -> ModelConfig:
    """48 layers, hidden 3072, 24 query / 4 kv heads of 128, 256 experts of width 1024 + one shared expert, top-8."""
    return ModelConfig(hidden_size=3072, num_hidden_layers=48, num_attention_heads=24, num_key_value_heads=4,
                       head_dim=128, intermediate_size=8192, moe_intermediate_size=1024, num_experts=256,
                       num_experts_per_tok=8, shared_expert_intermediate_size=1024)


PRESETS = {
    "tiny-moe": tiny_moe_config,
    "dense-9b": dense_9b_config,
    "moe-30b-a3b": moe_30b_a3b_config,
    "moe-120b": moe_120b_config,
}
