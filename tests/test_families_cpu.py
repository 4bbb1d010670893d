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
    base.update(kw)
    return ModelConfig(**base)


def logits_of(model, ids):
    b = pack_documents([ids])
    with torch.no_grad():
        return model.hidden_states(b.input_ids, b.position_ids, b.cu_seqlens) @ model.head_weight().t(), b


CASES = [("mistral", {"sliding_window": 16}), ("qwen2", {"sliding_window": 24}), ("llama", {}), ("llama", {"rope_scaling": LLAMA3}), ("llama", {"attention_bias": True}), ("mistral", {}),
         ("qwen2", {}), ("qwen2", {"rope_scaling": YARN}), ("mixtral", {}), ("qwen2_moe", {}), ("olmoe", {}),
         ("glm4_moe", {}), ("glm4_moe", {"n_group": 4, "topk_group": 2, "use_qk_norm": False, "attention_bias": True})]


@pytest.mark.parametrize("family,extra", CASES, ids=[f"{f}-{'-'.join(e) or 'plain'}" for f, e in CASES])
def test_family_round_trip_through_transformers(tmp_path, family, extra):
    transformers = pytest.importorskip("transformers")
    cfg = family_config(family, **extra)
    model = build_model(cfg, device="cpu", seed=5, gradient_checkpointing=False)
    if cfg.use_qk_norm:
        with torch.no_grad():
            for layer in model.layers:       # all-ones norm weights would hide a wrong norm scope
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
    d = str(tmp_path / "hf")
    save_model(model, d, save_dtype=None)
    assert ModelConfig.load(d) == cfg
    hf = transformers.AutoModelForCausalLM.from_pretrained(d, torch_dtype=torch.float32, attn_implementation="eager")
    hf.eval()
    assert type(hf).__name__ == FAMILIES[family]["architecture"]
    ids = np.random.default_rng(2).integers(0, cfg.vocab_size, size=96)
    ours, b = logits_of(model, ids)
    with torch.no_grad():
        theirs = hf(input_ids=b.input_ids[None]).logits[0]
    assert (ours - theirs).abs().max().item() < 5e-2 * theirs.abs().max().item()
    # and the other way: what transformers writes loads here, tensor for tensor
    d2 = str(tmp_path / "from_hf")
    hf.save_pretrained(d2, safe_serialization=True)
    back = from_pretrained(d2, device="cpu", dtype=torch.float32, gradient_checkpointing=False)
    for (n, a), (_, c) in zip(model.named_parameters(), back.named_parameters()):
        assert torch.equal(a, c), n


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
    q["max_window_layers"] = 1
    with pytest.raises(ValueError, match="per-layer mix"):
        ModelConfig.from_hf_dict(q)
    with pytest.raises(ValueError, match="no family registered"):
        ModelConfig.from_hf_dict({**d, "model_type": "mamba"})
