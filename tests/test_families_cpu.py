"""Decoder families beyond Qwen3: a model of each family, saved in hub layout, loads in ``transformers`` (which
converts the hub names itself) and gives our logits; a checkpoint written by ``transformers`` loads here; rotary
scaling follows the Hugging Face frequencies; windowed attention (Mistral-style) follows the Hugging Face mask."""

import numpy as np
import pytest
import torch

from halo_b200.checkpoint.load import from_pretrained
from halo_b200.checkpoint.save import save_model
from halo_b200.data.packing import pack_documents
from halo_b200.models.config import FAMILIES, ModelConfig
from halo_b200.models.qwen3 import build_model
from halo_b200.ops.rope import scaled_inverse_frequencies

LLAMA3 = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
YARN = {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32}


def family_config(family: str, **kw) -> ModelConfig:
    base = dict(vocab_size=512, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                head_dim=32, intermediate_size=192, moe_intermediate_size=0, num_experts=0, model_type=family, rope_theta=10000.0,
                max_position_embeddings=256, use_qk_norm=FAMILIES[family]["qk_norm"],
                attention_bias=FAMILIES[family]["bias_default"])
    if FAMILIES[family]["moe"]:
        base.update(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=96, norm_topk_prob=True)
    if family == "mixtral":
        base.update(intermediate_size=96)
    if family == "qwen2_moe":
        base.update(shared_expert_intermediate_size=64, shared_expert_gate=True, norm_topk_prob=False)
    if family == "olmoe":
        base.update(intermediate_size=96, norm_topk_prob=False, qk_norm_whole_width=True)
    if family == "glm4_moe":
        base.update(num_experts=8, partial_rotary_factor=0.5, score_function="sigmoid", router_bias=True, n_group=2, topk_group=1,
                    routed_scaling_factor=1.5, shared_expert_intermediate_size=96, mlp_only_layers=[0], use_qk_norm=True)
    if family == "gemma2":
        base.update(num_hidden_layers=2, sliding_window=16, layer_types=["sliding_attention", "full_attention"], use_qk_norm=False,
                    hidden_activation="gelu_tanh", sandwich_norms=True, norm_unit_offset=True, embedding_multiplier=128 ** 0.5,
                    query_pre_attn_scalar=24, attn_logit_softcapping=2.0, final_logit_softcapping=0.7, tie_word_embeddings=True)
    if family == "gemma3_text":
        base.update(num_hidden_layers=3, sliding_window=16, layer_types=["sliding_attention", "sliding_attention", "full_attention"],
                    hidden_activation="gelu_tanh", sandwich_norms=True, norm_unit_offset=True, embedding_multiplier=128 ** 0.5,
                    query_pre_attn_scalar=24, rope_local_theta=500.0, tie_word_embeddings=True)
    if family == "glm_moe_dsa":
        # fewer keys selected (24) than the test's row holds (96): the indexer's choice decides the logits
        base.update(rope_interleave=False, index_topk=24, index_n_heads=3, index_head_dim=20, rms_norm_eps=1e-5)
    if family in ("deepseek_v3", "glm4_moe_lite", "glm_moe_dsa"):
        base.update(num_experts=8, score_function="sigmoid", router_bias=True, n_group=2, topk_group=1, routed_scaling_factor=2.5,
                    shared_expert_intermediate_size=96, mlp_only_layers=[0], use_qk_norm=False, num_key_value_heads=4, head_dim=16,
                    kv_lora_rank=32, q_lora_rank=48, qk_nope_head_dim=24, qk_rope_head_dim=16, v_head_dim=20)
    if family == "mistral4":
        # positions reach past the period (so the query stretch is visible), two of four groups eligible
        base.update(num_experts=8, n_group=4, topk_group=2, routed_scaling_factor=1.5, shared_expert_intermediate_size=96,
                    mlp_only_layers=[0], use_qk_norm=False, num_key_value_heads=4, head_dim=16, kv_lora_rank=32, q_lora_rank=48,
                    qk_nope_head_dim=24, qk_rope_head_dim=16, v_head_dim=20, query_scale_beta=0.3, query_scale_period=16,
                    rope_scaling={"rope_type": "yarn", "factor": 4.0, "beta_fast": 32.0, "beta_slow": 1.0, "mscale": 1.0,
                                  "mscale_all_dim": 1.0, "original_max_position_embeddings": 16})
    if family in ("qwen3_next", "qwen3_5_moe_text"):
        base.update(num_hidden_layers=4, layer_types=["linear_attention", "linear_attention", "full_attention", "linear_attention"],
                    partial_rotary_factor=0.25, attn_output_gate=True, norm_unit_offset=True, shared_expert_intermediate_size=64,
                    shared_expert_gate=True, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=8,
                    linear_value_head_dim=12, linear_conv_kernel_dim=4)
    if family == "lfm2_moe":
        base.update(num_hidden_layers=4, layer_types=["conv", "conv", "full_attention", "conv"], conv_kernel=3, num_experts=8,
                    score_function="sigmoid", router_bias=True, norm_topk_eps=1e-6, routed_scaling_factor=1.5, mlp_only_layers=[0],
                    rms_norm_eps=1e-5, tie_word_embeddings=True)
    if family == "gpt_oss":
        base.update(intermediate_size=96, sliding_window=16, layer_types=["sliding_attention", "full_attention"], attention_sinks=True,
                    output_bias=True, router_logit_bias=True, expert_bias=True, expert_activation="clamped_glu", rms_norm_eps=1e-5,
                    rope_scaling={"rope_type": "yarn", "factor": 4.0, "beta_fast": 32.0, "beta_slow": 1.0, "truncate": False,
                                  "original_max_position_embeddings": 64})
    base.update(kw)
    return ModelConfig(**base)


def logits_of(model, ids):
    b = pack_documents([ids])
    with torch.no_grad():
        h = model.hidden_states(b.input_ids, b.position_ids, b.cu_seqlens)
        return (model.capped_logits(h) if model.cfg.final_logit_softcapping else h @ model.head_weight().t()), b


CASES = [("mistral", {"sliding_window": 16}), ("qwen2", {"sliding_window": 24}),
         ("qwen2", {"sliding_window": 12, "layer_types": ["full_attention", "sliding_attention"]}), ("llama", {}), ("llama", {"rope_scaling": LLAMA3}), ("llama", {"attention_bias": True}), ("mistral", {}),
         ("qwen2", {}), ("qwen2", {"rope_scaling": YARN}), ("mixtral", {}), ("qwen2_moe", {}), ("olmoe", {}),
         ("glm4_moe", {}), ("glm4_moe", {"n_group": 4, "topk_group": 2, "use_qk_norm": False, "attention_bias": True}),
         ("gpt_oss", {}), ("gemma2", {}), ("gemma3_text", {}), ("gemma3_text", {"rope_scaling": {"rope_type": "linear", "factor": 8.0}, "tie_word_embeddings": False}),
         ("deepseek_v3", {}), ("deepseek_v3", {"q_lora_rank": 0, "rope_interleave": False}),
         ("deepseek_v3", {"rope_scaling": {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64, "mscale": 1.0,
                                           "mscale_all_dim": 1.0, "beta_fast": 32.0, "beta_slow": 1.0}}),
         ("glm4_moe_lite", {}), ("glm4_moe_lite", {"num_hidden_layers": 3, "mlp_only_layers": [0, 2], "n_group": 1, "topk_group": 1}),
         ("glm_moe_dsa", {}), ("glm_moe_dsa", {"index_topk": 512, "mlp_only_layers": [1]}),
         ("qwen3_next", {}), ("qwen3_next", {"linear_num_key_heads": 4, "linear_conv_kernel_dim": 3, "shared_expert_intermediate_size": 48,
                                             "mlp_only_layers": [1]}),
         ("qwen3_5_moe_text", {}),
         ("lfm2_moe", {}), ("lfm2_moe", {"conv_kernel": 4, "router_bias": False, "tie_word_embeddings": False,
                                         "layer_types": ["full_attention", "conv", "conv", "conv"]}),
         ("mistral4", {}), ("mistral4", {"q_lora_rank": 0, "rope_interleave": False, "n_group": 1, "topk_group": 1,
                                         "routed_scaling_factor": 1.0, "query_scale_beta": 0.0, "query_scale_period": 0})]


@pytest.mark.parametrize("family,extra", CASES, ids=[f"{f}-{'-'.join(e) or 'plain'}" for f, e in CASES])
def test_family_round_trip_through_transformers(tmp_path, family, extra):
    transformers = pytest.importorskip("transformers")
    cfg = family_config(family, **extra)
    model = build_model(cfg, device="cpu", seed=5, gradient_checkpointing=False)
    if cfg.sandwich_norms:
        with torch.no_grad():
            g = torch.Generator().manual_seed(37)
            for layer in model.layers:       # all-ones norm weights would hide a misplaced norm or a forgotten offset
                for name in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
                    getattr(layer, name).normal_(1.0, 0.3, generator=g)
            model.norm.normal_(1.0, 0.3, generator=g)
    if cfg.kv_lora_rank:
        with torch.no_grad():
            for layer in model.layers:       # all-ones norm weights would hide a misplaced norm
                layer.self_attn.kv_a_norm.normal_(1.0, 0.2, generator=torch.Generator().manual_seed(29))
                if cfg.q_lora_rank:
                    layer.self_attn.q_a_norm.normal_(1.0, 0.2, generator=torch.Generator().manual_seed(31))
    if cfg.linear_num_value_heads:
        with torch.no_grad():
            g = torch.Generator().manual_seed(43)
            for layer in model.layers:       # small taps, unit decay rates and a unit norm would hide a wrong order or a dropped term
                if hasattr(layer.self_attn, "gdn_conv"):
                    a = layer.self_attn
                    a.gdn_conv.normal_(0.0, 0.5, generator=g)
                    for name, std in (("gdn_in_proj_qkvz", 0.3), ("gdn_in_proj_ba", 0.5), ("gdn_in_proj_qkv", 0.3), ("gdn_in_proj_z", 0.3),
                                      ("gdn_in_proj_b", 0.5), ("gdn_in_proj_a", 0.5)):
                        if hasattr(a, name):
                            getattr(a, name).normal_(0.0, std, generator=g)
                    a.gdn_A_log.uniform_(-1.0, 1.5, generator=g)
                    a.gdn_time_step.normal_(0.5, 0.5, generator=g)
                    a.gdn_norm.normal_(1.0, 0.2, generator=g)
    if cfg.conv_kernel:
        with torch.no_grad():
            g = torch.Generator().manual_seed(41)
            for layer in model.layers:       # taps near zero would hide a reversed or shifted kernel
                if hasattr(layer.self_attn, "conv_taps"):
                    layer.self_attn.conv_taps.normal_(0.0, 0.6, generator=g)
                    layer.self_attn.conv_in_proj.normal_(0.0, 0.15, generator=g)
    if cfg.index_topk:
        with torch.no_grad():
            g = torch.Generator().manual_seed(47)
            for layer in model.layers:       # near-zero projections would rank the keys by noise; a plain norm would hide its bias
                a = layer.self_attn
                for t, std in ((a.indexer_wq_b, 0.3), (a.indexer_wk, 0.3), (a.indexer_weights_proj, 0.5)):
                    t.normal_(0.0, std, generator=g)
                a.indexer_k_norm.normal_(1.0, 0.2, generator=g)
                a.indexer_k_norm_bias.normal_(0.0, 0.2, generator=g)
    if cfg.use_qk_norm:
        with torch.no_grad():
            for layer in model.layers:       # all-ones norm weights would hide a wrong norm scope
                if not hasattr(layer.self_attn, "q_norm"):
                    continue
                layer.self_attn.q_norm.normal_(1.0, 0.2, generator=torch.Generator().manual_seed(17))
                layer.self_attn.k_norm.normal_(1.0, 0.2, generator=torch.Generator().manual_seed(19))
    if cfg.router_bias:
        with torch.no_grad():
            for layer in model.layers:       # a zero selection bias would hide a wrong ranking
                if hasattr(layer.mlp, "e_score_correction_bias"):
                    layer.mlp.e_score_correction_bias.normal_(0.0, 0.2, generator=torch.Generator().manual_seed(13))
    if cfg.attention_bias:
        with torch.no_grad():
            for layer in model.layers:       # a zero bias would hide a wrong split
                layer.self_attn.qkv_bias.normal_(0.0, 0.5, generator=torch.Generator().manual_seed(11))
    if family == "gpt_oss":
        with torch.no_grad():                # zero sinks and biases would hide a wrong softmax, split or interleave
            g = torch.Generator().manual_seed(23)
            for layer in model.layers:
                layer.self_attn.sinks.normal_(0.0, 1.0, generator=g)
                layer.self_attn.o_bias.normal_(0.0, 0.2, generator=g)
                layer.mlp.gate_bias.normal_(0.0, 0.5, generator=g)
                layer.mlp.experts_gate_up_bias.normal_(0.0, 4.0, generator=g)     # wide enough to reach the clamps
                layer.mlp.experts_down_bias.normal_(0.0, 0.2, generator=g)
    d = str(tmp_path / "hf")
    save_model(model, d, save_dtype=None)
    assert ModelConfig.load(d) == cfg
    # by the architecture's own class: not every text model is registered with the causal-LM auto class
    hf = getattr(transformers, FAMILIES[family]["architecture"]).from_pretrained(d, dtype=torch.float32, attn_implementation="eager")
    hf.eval()
    assert type(hf).__name__ == FAMILIES[family]["architecture"]
    ids = np.random.default_rng(2).integers(0, cfg.vocab_size, size=96)
    ours, b = logits_of(model, ids)
    with torch.no_grad():
        theirs = hf(input_ids=b.input_ids[None]).logits[0]
    if 0 < cfg.index_topk < len(ids):
        # a hard top-k: where a query's last chosen and first dropped key score within fp32 rounding of each other, the two
        # implementations may choose differently, and that token's logits then differ. Rare (about one query in 200
        # here), so: nearly every token must agree, instead of every one
        close = (ours - theirs).abs().max(dim=-1).values < 5e-2 * theirs.abs().max().item()
        assert close.float().mean().item() >= 0.97, close.float().mean().item()
    else:
        assert (ours - theirs).abs().max().item() < 5e-2 * theirs.abs().max().item()
    # and the other way: what transformers writes loads here, tensor for tensor
    d2 = str(tmp_path / "from_hf")
    hf.save_pretrained(d2, safe_serialization=True)
    back = from_pretrained(d2, device="cpu", dtype=torch.float32, gradient_checkpointing=False)
    for (n, a), (_, c) in zip(model.named_parameters(), back.named_parameters()):
        # norms stored as (w - 1) come back through one fp32 subtraction and addition
        assert torch.equal(a, c) or (cfg.norm_unit_offset and a.dim() == 1 and torch.allclose(a, c, atol=1e-6, rtol=0)), n


@pytest.mark.parametrize("scaling", [LLAMA3, YARN, {"rope_type": "linear", "factor": 2.0}])
def test_scaled_frequencies_match_transformers(scaling):
    pytest.importorskip("transformers")
    from transformers import LlamaConfig
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS

    hf_cfg = LlamaConfig(hidden_size=128, num_attention_heads=4, head_dim=32, max_position_embeddings=256,
                         rope_parameters={**scaling, "rope_theta": 10000.0})
    want, want_factor = ROPE_INIT_FUNCTIONS[scaling["rope_type"]](hf_cfg, "cpu")
    got, factor = scaled_inverse_frequencies(32, 10000.0, scaling, 256)
    assert torch.allclose(got, want, rtol=1e-6, atol=0)
    assert abs(factor - want_factor) < 1e-6


def test_window_and_family_gates():
    d = family_config("mistral").to_hf_dict()
    d["sliding_window"] = 64
    assert ModelConfig.from_hf_dict(d).sliding_window == 64
    d["sliding_window"] = 4096                      # as wide as the context: plain causal attention
    assert ModelConfig.from_hf_dict(d).sliding_window == 0
    q = family_config("qwen2", sliding_window=16).to_hf_dict()
    q["max_window_layers"] = 1                      # Qwen2 windows the layers from this one on
    assert ModelConfig.from_hf_dict(q).layer_types == ["full_attention", "sliding_attention"]
    q["max_window_layers"] = 2
    assert ModelConfig.from_hf_dict(q).sliding_window == 0
    text = family_config("qwen3_5_moe_text").to_hf_dict()
    wrapped = {"model_type": "qwen3_5_moe", "text_config": text, "vision_config": {"depth": 2}, "tie_word_embeddings": False}
    assert ModelConfig.from_hf_dict(wrapped) == family_config("qwen3_5_moe_text")     # a multimodal config reads as its text tower
    with pytest.raises(ValueError, match="no family registered"):
        ModelConfig.from_hf_dict({**d, "model_type": "mamba"})


def test_biased_clamped_glu_experts_match_the_dense_form():
    from halo_b200.ops.biased_glu_experts import biased_glu_experts, biased_glu_experts_reference

    g = torch.Generator().manual_seed(3)
    T, H, F, E, k = 40, 32, 24, 6, 2
    x = torch.randn(T, H, generator=g, requires_grad=True)
    banks = [torch.randn(E, 2 * F, H, generator=g) * 0.5, torch.randn(E, 2 * F, generator=g) * 4.0,       # biases reach both clamps
             torch.randn(E, H, F, generator=g) * 0.2, torch.randn(E, H, generator=g)]
    banks = [b.requires_grad_() for b in banks]
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    idx[:, 0] = idx[:, 0].clamp(max=E - 2)                  # the last expert is rarely hit; expert E-1 may get no token at all
    w = torch.rand(T, k, generator=g).requires_grad_()
    got = biased_glu_experts(x, idx, w, *banks)
    want = biased_glu_experts_reference(x, idx, w, *banks)
    assert torch.allclose(got, want, atol=1e-4)
    probe = torch.randn(T, H, generator=g)
    for a, b in zip(torch.autograd.grad((got * probe).sum(), (x, w, *banks)), torch.autograd.grad((want * probe).sum(), (x, w, *banks))):
        assert torch.allclose(a, b, atol=1e-4)


def test_gpt_oss_trains_and_sinks_follow_the_policy(tmp_path):
    """A tiny gpt-oss model takes optimizer steps (loss falls; sinks, router bias and expert biases all get gradients);
    the sinks policy neutralizes, freezes or trains the sinks; layouts that would cut the family are refused by name."""
    from halo_b200.config_validation import ConfigError
    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.attention_sinks import apply_sinks_policy, policy_from_flags
    from halo_b200.parallel.config import ParallelismConfig
    from halo_b200.parallel.rules import reject_model_layout
    from halo_b200.trainers.engine import TrainEngine

    cfg = family_config("gpt_oss")
    model = build_model(cfg, device="cpu", seed=1, gradient_checkpointing=True)
    assert [layer.self_attn.window for layer in model.layers] == [16, 0]
    assert sum(p.numel() for p in model.parameters()) == cfg.param_counts()["total"]
    assert apply_sinks_policy(model, policy_from_flags(False, True)) == 2 and model.sinks_policy == "trainable"
    engine = TrainEngine(model, torch.optim.AdamW(model.parameters(), lr=3e-3), "cpu", max_grad_norm=1.0)
    batch = synthetic_packed_batch(96, cfg.vocab_size, seed=0, lo=20, hi=50)
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    losses = [float(engine.train_step(batch).loss.reshape(-1)[0]) for _ in range(6)]
    assert losses[-1] < losses[0] - 0.3, losses
    moved = {n for n, p in model.named_parameters() if not torch.equal(p, before[n])}
    for name in ("layers.0.self_attn.sinks", "layers.1.self_attn.sinks", "layers.0.self_attn.o_bias", "layers.0.mlp.gate_bias",
                 "layers.0.mlp.experts_gate_up_bias", "layers.1.mlp.experts_down_bias"):
        assert name in moved, name
    # neutralized: no softmax mass, no gradient, the same function as a model without sinks
    apply_sinks_policy(model, "neutralized")
    assert all(not layer.self_attn.sinks.requires_grad and layer.self_attn.sinks.max() < -1e30 for layer in model.layers)
    ids = np.random.default_rng(4).integers(0, cfg.vocab_size, size=64)
    neutral, _ = logits_of(model, ids)
    saved = [layer.self_attn.sinks for layer in model.layers]
    for layer in model.layers:
        layer.self_attn.sinks = None
    plain, _ = logits_of(model, ids)
    for layer, s in zip(model.layers, saved):
        layer.self_attn.sinks = s
    assert torch.allclose(neutral, plain, atol=1e-5)
    fresh = build_model(cfg, device="cpu", seed=1, gradient_checkpointing=False)
    apply_sinks_policy(fresh, "neutralized", pretrained=False)         # nothing pretrained to protect: stays live
    assert fresh.sinks_policy == "live" and float(fresh.layers[0].self_attn.sinks.abs().max()) == 0.0
    with pytest.raises(ValueError, match="contradicts"):
        policy_from_flags(True, True)
    with pytest.raises(ValueError, match="no attention sinks"):
        apply_sinks_policy(build_model(family_config("llama"), device="cpu"), "trainable")
    for axis in ("tp_size", "cp_size"):
        with pytest.raises(ConfigError, match="not cut inside an expert, a head group or a row"):
            reject_model_layout(ParallelismConfig(world_size=2, **{axis: 2}), cfg)
    reject_model_layout(ParallelismConfig(world_size=4, pp_size=2), cfg)
    reject_model_layout(ParallelismConfig(world_size=2, ep_size=2), cfg)       # whole experts move, their bias rows with them
    # an expert-parallel rank holds its slice of the banks and of the two bias banks
    from halo_b200.models.qwen3 import SparseMoE

    sliced = SparseMoE(cfg, torch.float32, "meta", cfg.num_experts // 2)
    assert sliced.experts_gate_up_bias.shape[0] == sliced.experts_down_bias.shape[0] == cfg.num_experts // 2


def test_keys_visited_follow_each_layers_window():
    """The attention term of the model-FLOPs count, per layer: the mask the layer really applies has that many pairs."""
    from halo_b200.models.attention_cost import attention_flops, causal_pairs, keys_visited_per_layer, layer_windows
    from halo_b200.ops.masked_attention import window_mask

    cu = [0, 5, 45, 46, 96]
    cfg = family_config("gpt_oss")                  # layer 0 windowed (16), layer 1 full
    assert layer_windows(cfg) == [16, 0]
    windowed, full = keys_visited_per_layer(cfg, cu)
    assert windowed == float(window_mask(cu, 16).sum()) and full == float(window_mask(cu, 96).sum())
    assert causal_pairs([40], 16) == 16 * 17 / 2 + 24 * 16 and causal_pairs([5], 16) == 15.0
    assert attention_flops(cfg, cu) == 12.0 * cfg.head_dim * cfg.num_attention_heads * (windowed + full)
    plain = family_config("llama")
    assert keys_visited_per_layer(plain, cu) == [full] * 2


@pytest.mark.parametrize("family,streams", [("deepseek_v3", 1), ("deepseek_v3", 2), ("mistral4", 1)])
def test_latent_attention_model_trains(family, streams):
    """DeepSeek-V3 shape (latent attention, sigmoid group-limited routing, shared experts, a leading dense layer) takes
    optimizer steps under per-layer recomputation - also on two hyper-connected residual streams - and so does the
    Mistral 4 shape (softmax scores, position-stretched queries); layouts that would cut the attention block are refused
    by name."""
    from halo_b200.config_validation import ConfigError
    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.parallel.config import ParallelismConfig
    from halo_b200.parallel.rules import reject_model_layout
    from halo_b200.trainers.engine import TrainEngine

    cfg = family_config(family, hc_mult=streams)
    model = build_model(cfg, device="cpu", seed=2, gradient_checkpointing=True)
    assert sum(p.numel() for p in model.parameters()) == cfg.param_counts()["total"]
    engine = TrainEngine(model, torch.optim.AdamW(model.parameters(), lr=3e-3), "cpu", max_grad_norm=1.0)
    batch = synthetic_packed_batch(96, cfg.vocab_size, seed=0, lo=20, hi=50)
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    losses = [float(engine.train_step(batch).loss.reshape(-1)[0]) for _ in range(6)]
    assert losses[-1] < losses[0] - 0.3, losses
    moved = {n for n, p in model.named_parameters() if not torch.equal(p, before[n])}
    for name in ("q_a_proj", "q_a_norm", "q_b_proj", "kv_a_proj", "kv_a_norm", "kv_b_proj", "o_proj"):
        assert f"layers.1.self_attn.{name}" in moved, name
    for axis in ("tp_size", "cp_size"):
        with pytest.raises(ConfigError, match="latent attention"):
            reject_model_layout(ParallelismConfig(world_size=2, **{axis: 2}), cfg)
    reject_model_layout(ParallelismConfig(world_size=2, ep_size=2), cfg)


def test_short_convolution_family_trains_and_keeps_documents_apart():
    """LFM2-MoE shape: the taps of a conv layer never reach across a document's first token in a packed row (each
    document's logits equal the ones it gets alone), the model takes optimizer steps under per-layer recomputation, and
    layouts that would cut a row are refused by name."""
    from halo_b200.config_validation import ConfigError
    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.attention_cost import keys_visited_per_layer
    from halo_b200.parallel.config import ParallelismConfig
    from halo_b200.parallel.rules import reject_model_layout
    from halo_b200.trainers.engine import TrainEngine

    cfg = family_config("lfm2_moe")
    model = build_model(cfg, device="cpu", seed=2, gradient_checkpointing=True)
    assert sum(p.numel() for p in model.parameters()) == cfg.param_counts()["total"]
    with torch.no_grad():
        for layer in model.layers:
            if hasattr(layer.self_attn, "conv_taps"):
                layer.self_attn.conv_taps.normal_(0.0, 0.6, generator=torch.Generator().manual_seed(3))
    rng = np.random.default_rng(4)
    docs = [rng.integers(0, cfg.vocab_size, size=n) for n in (1, 2, 17, 5)]       # shorter than the kernel, too
    b = pack_documents(docs)
    with torch.no_grad():
        packed = model.hidden_states(b.input_ids, b.position_ids, b.cu_seqlens)
        start = 0
        for d in docs:
            alone, _ = logits_of(model, d)
            together = packed[start:start + len(d)] @ model.head_weight().t()
            assert torch.allclose(alone, together, atol=2e-5), float((alone - together).abs().max())
            start += len(d)
    visited = keys_visited_per_layer(cfg, [0, 40, 96])
    assert [v == 0.0 for v in visited] == [True, True, False, True]
    engine = TrainEngine(model, torch.optim.AdamW(model.parameters(), lr=3e-3), "cpu", max_grad_norm=1.0)
    batch = synthetic_packed_batch(96, cfg.vocab_size, seed=0, lo=20, hi=50)
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    losses = [float(engine.train_step(batch).loss.reshape(-1)[0]) for _ in range(6)]
    assert losses[-1] < losses[0] - 0.3, losses
    moved = {n for n, p in model.named_parameters() if not torch.equal(p, before[n])}
    for name in ("conv_in_proj", "conv_taps", "conv_out_proj"):
        assert f"layers.1.self_attn.{name}" in moved, name
    for axis in ("tp_size", "cp_size"):
        with pytest.raises(ConfigError, match="short-convolution"):
            reject_model_layout(ParallelismConfig(world_size=2, **{axis: 2}), cfg)
    reject_model_layout(ParallelismConfig(world_size=2, ep_size=2), cfg)


def test_chunked_delta_rule_equals_the_recurrence():
    """The chunked form (triangular solve per chunk, documents side by side) against the token-by-token recurrence: outputs,
    each document's final state and the gradients of every input, for chunk sizes that do and do not divide the documents."""
    from halo_b200.models.gated_delta_net import chunked_gated_delta_rule, recurrent_gated_delta_step

    g = torch.Generator().manual_seed(1)
    lengths, H, dk, dv = [5, 1, 23, 8], 3, 6, 4
    T = sum(lengths)
    leaves = [torch.randn(T, H, dk, generator=g), torch.randn(T, H, dk, generator=g), torch.randn(T, H, dv, generator=g),
              -torch.rand(T, H, generator=g) * 2.0, torch.rand(T, H, generator=g)]
    leaves = [t.double().requires_grad_() for t in leaves]

    def prepared():
        q, k, v, lg, beta = leaves
        return q / q.norm(dim=-1, keepdim=True), k / k.norm(dim=-1, keepdim=True), v, lg, beta

    def recurrent():
        q, k, v, lg, beta = prepared()
        outs, finals, start = [], [], 0
        for n in lengths:
            s = torch.zeros(1, H, dk, dv)
            for t in range(start, start + n):
                o, s = recurrent_gated_delta_step(s, q[t][None].float(), k[t][None].float(), v[t][None].float(), lg[t][None].float(),
                                                  beta[t][None].float())
                outs.append(o[0])
            finals.append(s[0])
            start += n
        return torch.stack(outs), torch.stack(finals)

    probe_o, probe_s = torch.randn(T, H, dv, generator=g), torch.randn(len(lengths), H, dk, dv, generator=g)
    want_o, want_s = recurrent()
    want = torch.autograd.grad((want_o * probe_o).sum() + (want_s * probe_s).sum(), leaves)
    for chunk in (4, 8, 64):
        got_o, got_s = chunked_gated_delta_rule(*prepared(), lengths, chunk=chunk)
        assert torch.allclose(got_o, want_o.float(), atol=2e-5), (chunk, float((got_o - want_o).abs().max()))
        assert torch.allclose(got_s, want_s.float(), atol=2e-5), chunk
        got = torch.autograd.grad((got_o * probe_o).sum() + (got_s * probe_s).sum(), leaves)
        for a, b, name in zip(got, want, "q k v log_g beta".split()):
            assert torch.allclose(a, b, atol=5e-5), (chunk, name, float((a - b).abs().max()))


def test_linear_attention_family_trains_and_keeps_documents_apart():
    """Qwen3-Next shape: neither the convolution nor the matrix state of a linear-attention layer crosses a document's first
    token in a packed row; the model takes optimizer steps under per-layer recomputation; row- and head-cutting layouts and an
    adapter on the gate-carrying query projection are refused by name."""
    from halo_b200.config_validation import ConfigError
    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.parallel.config import ParallelismConfig
    from halo_b200.parallel.rules import reject_model_layout
    from halo_b200.peft.lora import LoraSpec, apply_lora
    from halo_b200.trainers.engine import TrainEngine

    cfg = family_config("qwen3_next")
    model = build_model(cfg, device="cpu", seed=2, gradient_checkpointing=True)
    assert sum(p.numel() for p in model.parameters()) == cfg.param_counts()["total"]
    with torch.no_grad():
        for layer in model.layers:
            if hasattr(layer.self_attn, "gdn_conv"):
                layer.self_attn.gdn_conv.normal_(0.0, 0.5, generator=torch.Generator().manual_seed(3))
                layer.self_attn.gdn_in_proj_qkvz.normal_(0.0, 0.3, generator=torch.Generator().manual_seed(4))
    rng = np.random.default_rng(4)
    docs = [rng.integers(0, cfg.vocab_size, size=n) for n in (2, 70, 1, 9)]       # one longer than a chunk
    b = pack_documents(docs)
    with torch.no_grad():
        packed = model.hidden_states(b.input_ids, b.position_ids, b.cu_seqlens)
        start = 0
        for d in docs:
            alone, _ = logits_of(model, d)
            together = packed[start:start + len(d)] @ model.head_weight().t()
            assert torch.allclose(alone, together, atol=5e-5), float((alone - together).abs().max())
            start += len(d)
    engine = TrainEngine(model, torch.optim.AdamW(model.parameters(), lr=3e-3), "cpu", max_grad_norm=1.0)
    batch = synthetic_packed_batch(96, cfg.vocab_size, seed=0, lo=20, hi=50)
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    losses = [float(engine.train_step(batch).loss.reshape(-1)[0]) for _ in range(6)]
    assert losses[-1] < losses[0] - 0.3, losses
    moved = {n for n, p in model.named_parameters() if not torch.equal(p, before[n])}
    for name in ("gdn_in_proj_qkvz", "gdn_in_proj_ba", "gdn_conv", "gdn_time_step", "gdn_A_log", "gdn_norm", "gdn_out_proj"):
        assert f"layers.1.self_attn.{name}" in moved, name
    assert "layers.2.self_attn.qkv_proj" in moved
    for axis in ("tp_size", "cp_size"):
        with pytest.raises(ConfigError, match="delta-rule"):
            reject_model_layout(ParallelismConfig(world_size=2, **{axis: 2}), cfg)
    reject_model_layout(ParallelismConfig(world_size=2, ep_size=2), cfg)
    with pytest.raises(ValueError, match="output gate"):
        apply_lora(build_model(cfg, device="cpu", seed=2), LoraSpec(r=4, target_modules=["q_proj", "v_proj"]))
    counts = apply_lora(model, LoraSpec(r=4, target_modules=["k_proj", "v_proj", "o_proj", "down_proj"]))
    assert counts["trainable"] > 0
    assert model.layers[0].self_attn.lora is None and model.layers[2].self_attn.lora is not None
    out = model(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels)
    (out.loss if hasattr(out, "loss") else out).sum().backward()
    assert model.layers[2].self_attn.lora.B["v_proj"].grad is not None


def test_sparse_latent_attention_selects_within_documents_and_trains():
    """GLM-5 (DSA) shape: every query attends at most ``index_topk`` keys, all of its own document and none after it; the
    model trains with the indexer's tensors held fixed. (Logits of a packed document are not compared with the document
    alone: keys whose indexer score is exactly zero - every head's product negative, one key in eight here - tie, and which
    of them a top-k keeps depends on the row's length.)"""
    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.ops.masked_attention import window_mask
    from halo_b200.trainers.engine import TrainEngine

    cfg = family_config("glm_moe_dsa", index_topk=6)
    model = build_model(cfg, device="cpu", seed=2, gradient_checkpointing=True)
    assert sum(p.numel() for p in model.parameters()) == cfg.param_counts()["total"]
    with torch.no_grad():
        g = torch.Generator().manual_seed(3)
        for layer in model.layers:
            for t in (layer.self_attn.indexer_wq_b, layer.self_attn.indexer_wk, layer.self_attn.indexer_weights_proj):
                t.normal_(0.0, 0.4, generator=g)
    rng = np.random.default_rng(4)
    docs = [rng.integers(0, cfg.vocab_size, size=n) for n in (3, 30, 1, 14)]
    b = pack_documents(docs)
    T = int(b.cu_seqlens[-1])
    a = model.layers[0].self_attn
    ctx = model.make_context(b.position_ids.reshape(-1), b.cu_seqlens)
    visible = window_mask(b.cu_seqlens, T, device="cpu")
    h = torch.randn(T, cfg.hidden_size, generator=torch.Generator().manual_seed(5))
    chosen = a.selected_keys(h, torch.randn(T, cfg.q_lora_rank, generator=torch.Generator().manual_seed(6)), ctx.rope, visible)
    assert not (chosen & ~visible).any()
    assert torch.equal(chosen.sum(1), visible.sum(1).clamp(max=6))
    trainable = [p for p in model.parameters() if p.requires_grad]
    assert all("indexer" not in n for n, p in model.named_parameters() if p.requires_grad)
    engine = TrainEngine(model, torch.optim.AdamW(trainable, lr=3e-3), "cpu", max_grad_norm=1.0)
    batch = synthetic_packed_batch(96, cfg.vocab_size, seed=0, lo=20, hi=50)
    losses = [float(engine.train_step(batch).loss.reshape(-1)[0]) for _ in range(6)]
    assert losses[-1] < losses[0] - 0.3, losses


def test_gemma3_trains_under_every_recomputation_policy():
    """The four-norm layer gives the same loss and gradients whether it runs whole, in halves or under recomputation."""
    from halo_b200.data.packing import synthetic_packed_batch

    cfg = family_config("gemma3_text")
    batch = synthetic_packed_batch(96, cfg.vocab_size, seed=0, lo=20, hi=50)
    results = {}
    for policy in ("none", "mlp", "full"):
        model = build_model(cfg, device="cpu", seed=2, gradient_checkpointing=policy != "none")
        for layer in model.layers:
            layer.recompute_policy = policy
        out = model(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels)
        loss = out.loss if hasattr(out, "loss") else out
        loss.sum().backward()
        results[policy] = (loss.detach().sum(), {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None})
    base_loss, base_grads = results["none"]
    from halo_b200.config_validation import ConfigError
    from halo_b200.parallel.config import ParallelismConfig
    from halo_b200.parallel.rules import reject_model_layout

    for fam in ("gemma3_text", "mistral"):
        with pytest.raises(ConfigError, match="whole rows"):
            reject_model_layout(ParallelismConfig(world_size=2, tp_size=2), family_config(fam, sliding_window=16))
    reject_model_layout(ParallelismConfig(world_size=2, tp_size=2), family_config("mistral"))
    assert "layers.0.pre_feedforward_layernorm" in base_grads and "layers.2.post_feedforward_layernorm" in base_grads
    for policy in ("mlp", "full"):
        loss, grads = results[policy]
        assert torch.allclose(loss, base_loss, atol=1e-6)
        assert grads.keys() == base_grads.keys()
        for n in grads:
            assert torch.allclose(grads[n], base_grads[n], atol=1e-5), (policy, n)


def test_sft_entry_point_fine_tunes_a_gpt_oss_checkpoint(tmp_path):
    """From a hub-layout gpt-oss checkpoint: the default run neutralizes the sinks (and says so), ``reset_sinks: false`` with
    ``train_sinks: true`` trains them; the saved model reloads with the policy's sinks."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = family_config("gpt_oss")
    model = build_model(cfg, device="cpu", seed=4, gradient_checkpointing=False)
    with torch.no_grad():
        for layer in model.layers:
            layer.self_attn.sinks.fill_(0.5)
    base = str(tmp_path / "base")
    save_model(model, base, save_dtype=None)
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")

    def run(name, extra):
        y = tmp_path / f"{name}.yaml"
        y.write_text(f"model_name_or_path: {base}\ntorch_dtype: float32\ndataset_format: synthetic\npacked_row_length: 128\nmax_steps: 2\n"
                     f"save_steps: 2\noptim: adamw_torch\nlearning_rate: 1.0e-2\nlogging_steps: 1\noutput_dir: {tmp_path}/{name}\n" + extra)
        r = subprocess.run([sys.executable, "-m", "halo_b200.cli", "launch", "sft", str(y)], cwd=root, capture_output=True, text=True,
                           timeout=300, env=env)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
        return r.stdout + r.stderr, from_pretrained(str(tmp_path / name / "final"), device="cpu", dtype=torch.float32)

    log, tuned = run("neutral", "")
    assert "policy neutralized" in log
    assert all(float(layer.self_attn.sinks.detach().max()) < -1e30 for layer in tuned.layers)
    assert torch.isfinite(tuned.layers[0].self_attn.sinks.detach().bfloat16()).all()
    log, tuned = run("trained", "reset_sinks: false\ntrain_sinks: true\n")
    assert "policy trainable" in log
    sinks = torch.stack([layer.self_attn.sinks for layer in tuned.layers])
    assert torch.isfinite(sinks).all() and float((sinks - 0.5).abs().max()) > 1e-4 and float((sinks - 0.5).abs().max()) < 0.5


def test_soft_capped_logits_loss_and_logprobs_agree():
    """Gemma 2: the training loss, the per-token log-probabilities the preference / policy-gradient trainers use and the
    Hugging Face loss all describe the same soft-capped distribution; the model takes optimizer steps."""
    transformers = pytest.importorskip("transformers")
    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.trainers.engine import TrainEngine

    cfg = family_config("gemma2")
    model = build_model(cfg, device="cpu", seed=3, gradient_checkpointing=True)
    batch = synthetic_packed_batch(96, cfg.vocab_size, seed=0, lo=96, hi=97)       # one document: comparable with a padded-free HF call
    loss = model(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels)
    loss = (loss.loss if hasattr(loss, "loss") else loss).sum()
    logp, entropy = model.token_logprobs(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels, want_entropy=True)
    scored = batch.labels.reshape(-1) != -100
    assert torch.allclose(-logp[scored].mean(), loss, atol=1e-5) and float(logp[~scored].abs().sum()) == 0.0
    assert entropy.shape == logp.shape and float(entropy.min()) > 0
    import tempfile

    d = tempfile.mkdtemp()
    save_model(model, d, save_dtype=None)
    hf = transformers.AutoModelForCausalLM.from_pretrained(d, dtype=torch.float32, attn_implementation="eager").eval()
    with torch.no_grad():
        z = hf(input_ids=batch.input_ids.reshape(1, -1)).logits[0]
    want = torch.nn.functional.cross_entropy(z[scored], batch.labels.reshape(-1)[scored])
    assert torch.allclose(loss.detach(), want, atol=1e-5)
    engine = TrainEngine(model, torch.optim.AdamW(model.parameters(), lr=3e-3), "cpu", max_grad_norm=1.0)
    losses = [float(engine.train_step(batch).loss.reshape(-1)[0]) for _ in range(5)]
    assert losses[-1] < losses[0] - 0.05, losses


def test_reset_sinks_tool(tmp_path):
    from halo_b200.checkpoint.tools import reset_sinks

    cfg = family_config("gpt_oss")
    model = build_model(cfg, device="cpu", seed=4, gradient_checkpointing=False)
    with torch.no_grad():
        for layer in model.layers:
            layer.self_attn.sinks.fill_(0.25)
    src, dst, back = (str(tmp_path / n) for n in ("src", "dst", "back"))
    save_model(model, src, save_dtype=None)
    assert reset_sinks.main([src, dst]) == 0
    neutral = from_pretrained(dst, device="cpu", dtype=torch.float32)
    assert all(float(layer.self_attn.sinks.detach().max()) < -1e30 for layer in neutral.layers)
    for (n, a), (_, c) in zip(model.named_parameters(), neutral.named_parameters()):
        assert n.endswith(".sinks") or torch.equal(a, c), n
    assert reset_sinks.main([dst, back, "--from-checkpoint", src]) == 0
    restored = from_pretrained(back, device="cpu", dtype=torch.float32)
    assert all(torch.equal(a, c) for (_, a), (_, c) in zip(model.named_parameters(), restored.named_parameters()))
    plain = str(tmp_path / "plain")
    save_model(build_model(family_config("llama"), device="cpu"), plain, save_dtype=None)
    with pytest.raises(SystemExit, match="no attention sinks"):
        reset_sinks.main([plain, str(tmp_path / "nope")])
