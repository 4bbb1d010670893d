"""Generation with the key/value cache on CPU: cached decoding reproduces the full forward's next-token
distribution at every step, greedy decoding matches ``transformers.generate``, stop tokens and sampling controls
behave, and returned log-probabilities are the model's."""

import dataclasses

import numpy as np
import pytest
import torch

from halo_b200.data.packing import pack_documents
from halo_b200.inference.generate import Generator, SamplingParams, _sample
from halo_b200.models.config import ModelConfig, tiny_moe_config
from halo_b200.models.qwen3 import build_model


def dense_cfg():
    return ModelConfig(vocab_size=128, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=16, intermediate_size=96, moe_intermediate_size=0, num_experts=0, model_type="qwen3")


def full_forward_logits(model, ids):
    b = pack_documents([np.asarray(ids)])
    with torch.no_grad():
        h = model.hidden_states(b.input_ids, b.position_ids, b.cu_seqlens)
    return model.capped_logits(h)[-1]           # plain logits unless the family caps them


def windowed_cfg():
    """Mistral-style: every layer sees its last 6 keys (shorter than prompt + completion)."""
    return dataclasses.replace(dense_cfg(), model_type="mistral", use_qk_norm=False, sliding_window=6, max_position_embeddings=64)


def sink_cfg():
    """gpt-oss style: a windowed and a full layer, sink logits, biased clamped-GLU experts."""
    return ModelConfig(vocab_size=128, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                       intermediate_size=48, moe_intermediate_size=48, num_experts=4, num_experts_per_tok=2, model_type="gpt_oss",
                       use_qk_norm=False, attention_bias=True, sliding_window=6, layer_types=["sliding_attention", "full_attention"],
                       attention_sinks=True, output_bias=True, router_logit_bias=True, expert_bias=True,
                       expert_activation="clamped_glu", max_position_embeddings=64)


def latent_cfg():
    """DeepSeek-V3 style: latent attention (query width 24 + 16, value width 20), sigmoid routing, a shared expert."""
    return ModelConfig(vocab_size=128, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, head_dim=16,
                       intermediate_size=96, moe_intermediate_size=48, num_experts=4, num_experts_per_tok=2, model_type="deepseek_v3",
                       use_qk_norm=False, score_function="sigmoid", router_bias=True, shared_expert_intermediate_size=48,
                       mlp_only_layers=[0], kv_lora_rank=32, q_lora_rank=24, qk_nope_head_dim=24, qk_rope_head_dim=16, v_head_dim=20,
                       max_position_embeddings=64)


def stretched_cfg():
    """Mistral 4 style: latent attention with softmax group-limited routing and queries stretched by position; the period
    (4) is shorter than the prompts, so prefill and decode steps both cross it."""
    return dataclasses.replace(latent_cfg(), model_type="mistral4", score_function="softmax", router_bias=False, n_group=2, topk_group=1,
                               routed_scaling_factor=1.5, query_scale_beta=0.4, query_scale_period=4)


def conv_cfg():
    """LFM2-MoE style: short-convolution mixers (4 taps: longer than the shortest prompt) around one attention layer."""
    return ModelConfig(vocab_size=128, hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                       intermediate_size=96, moe_intermediate_size=48, num_experts=4, num_experts_per_tok=2, model_type="lfm2_moe",
                       use_qk_norm=True, score_function="sigmoid", router_bias=True, norm_topk_eps=1e-6, mlp_only_layers=[0],
                       layer_types=["conv", "full_attention", "conv"], conv_kernel=4, max_position_embeddings=64)


def linear_cfg():
    """Qwen3-Next style: gated delta-rule layers (conv of 4 taps in front) around one gated-attention layer with a quarter of
    each head rotated."""
    return ModelConfig(vocab_size=128, hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                       intermediate_size=96, moe_intermediate_size=48, num_experts=4, num_experts_per_tok=2, model_type="qwen3_next",
                       use_qk_norm=True, shared_expert_intermediate_size=48, shared_expert_gate=True, attn_output_gate=True,
                       norm_unit_offset=True, partial_rotary_factor=0.25, layer_types=["linear_attention", "full_attention", "linear_attention"],
                       linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=8, linear_value_head_dim=12,
                       linear_conv_kernel_dim=4, max_position_embeddings=64)


def sparse_cfg():
    """GLM-5 (DSA) style: latent attention behind a key-selecting indexer; up to ``index_topk`` keys every key is selected,
    so cached decoding is exact."""
    return dataclasses.replace(latent_cfg(), model_type="glm_moe_dsa", rope_interleave=False, index_topk=32, index_n_heads=2,
                               index_head_dim=20)


def gemma_cfg():
    """Gemma 3 style: windowed layers with their own rotary base, a full layer, output norms, tanh-GELU gate, scaled embeddings."""
    return dataclasses.replace(dense_cfg(), model_type="gemma3_text", num_hidden_layers=3, sliding_window=6, max_position_embeddings=64,
                               layer_types=["sliding_attention", "sliding_attention", "full_attention"], hidden_activation="gelu_tanh",
                               sandwich_norms=True, norm_unit_offset=True, embedding_multiplier=8.0, query_pre_attn_scalar=24,
                               rope_local_theta=500.0, tie_word_embeddings=True)


def capped_cfg():
    """Gemma 2 style: soft-capped attention scores and output logits (caps small enough to bend both)."""
    return dataclasses.replace(gemma_cfg(), model_type="gemma2", num_hidden_layers=2, layer_types=["sliding_attention", "full_attention"],
                               use_qk_norm=False, rope_local_theta=0.0, attn_logit_softcapping=1.0, final_logit_softcapping=0.5)


@pytest.mark.parametrize("kind", ["dense", "moe", "windowed", "sinks", "latent", "stretched", "sparse", "conv", "linear", "gemma", "capped"])
def test_cached_decoding_equals_the_full_forward(kind):
    cfg = {"dense": dense_cfg, "windowed": windowed_cfg, "sinks": sink_cfg, "latent": latent_cfg, "stretched": stretched_cfg, "sparse": sparse_cfg, "conv": conv_cfg, "linear": linear_cfg, "gemma": gemma_cfg, "capped": capped_cfg,
           "moe": lambda: dataclasses.replace(tiny_moe_config(), num_hidden_layers=2, vocab_size=128)}[kind]()
    model = build_model(cfg, device="cpu", seed=7, gradient_checkpointing=False)
    if kind == "conv":
        with torch.no_grad():
            for layer in model.layers:       # taps near zero would hide a stale or shifted cache
                if hasattr(layer.self_attn, "conv_taps"):
                    layer.self_attn.conv_taps.normal_(0.0, 0.6, generator=torch.Generator().manual_seed(5))
    if kind == "linear":
        with torch.no_grad():
            for layer in model.layers:       # taps and projections near zero would hide a stale convolution or matrix state
                if hasattr(layer.self_attn, "gdn_conv"):
                    layer.self_attn.gdn_conv.normal_(0.0, 0.5, generator=torch.Generator().manual_seed(5))
                    layer.self_attn.gdn_in_proj_qkvz.normal_(0.0, 0.3, generator=torch.Generator().manual_seed(6))
    if kind == "sinks":
        with torch.no_grad():
            for layer in model.layers:
                layer.self_attn.sinks.normal_(0.0, 1.0, generator=torch.Generator().manual_seed(5))
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg.vocab_size, size=n) for n in (5, 11, 3)]
    outs = Generator(model).generate(prompts, SamplingParams(max_new_tokens=6, temperature=0.0))
    for p, g in zip(prompts, outs):
        assert len(g.token_ids) == 6 and g.finish_reason == "length"
        seq = list(p)
        for tok, lp in zip(g.token_ids, g.logprobs):
            logits = full_forward_logits(model, seq)
            assert int(logits.argmax()) == int(tok)
            assert abs(float(torch.log_softmax(logits.detach(), -1)[tok]) - float(lp)) < 1e-4
            seq.append(int(tok))


def test_greedy_matches_transformers_generate(tmp_path):
    transformers = pytest.importorskip("transformers")
    from halo_b200.checkpoint.save import save_model

    cfg = dense_cfg()
    model = build_model(cfg, device="cpu", seed=3, gradient_checkpointing=False)
    d = str(tmp_path / "hf")
    save_model(model, d, save_dtype=None)
    hf = transformers.AutoModelForCausalLM.from_pretrained(d, dtype=torch.float32, attn_implementation="eager").eval()
    prompt = np.arange(7) * 3 % cfg.vocab_size
    ours = Generator(model).generate([prompt], SamplingParams(max_new_tokens=12, temperature=0.0))[0]
    # the oracle is the other implementation's full forward at every step (no cache on that side)
    seq = torch.from_numpy(prompt)[None]
    for tok in ours.token_ids:
        with torch.no_grad():
            want = int(hf(input_ids=seq).logits[0, -1].argmax())
        assert want == int(tok)
        seq = torch.cat([seq, torch.tensor([[want]])], dim=1)


def test_stop_tokens_and_seeds():
    cfg = dense_cfg()
    model = build_model(cfg, device="cpu", seed=1, gradient_checkpointing=False)
    prompts = [np.array([1, 2, 3]), np.array([4, 5])]
    greedy = Generator(model).generate(prompts, SamplingParams(max_new_tokens=8, temperature=0.0))
    stop = int(greedy[0].token_ids[2])
    first = greedy[0].token_ids.tolist().index(stop)
    stopped = Generator(model, eos_token_id=stop).generate(prompts, SamplingParams(max_new_tokens=8, temperature=0.0))
    assert stopped[0].finish_reason == "stop" and stopped[0].token_ids.tolist() == greedy[0].token_ids[:first + 1].tolist()
    if stop not in greedy[1].token_ids:
        assert stopped[1].token_ids.tolist() == greedy[1].token_ids.tolist()      # the other sequence ran on
    a = Generator(model).generate(prompts, SamplingParams(max_new_tokens=8, temperature=1.0, seed=5))
    b = Generator(model).generate(prompts, SamplingParams(max_new_tokens=8, temperature=1.0, seed=5))
    c = Generator(model).generate(prompts, SamplingParams(max_new_tokens=8, temperature=1.0, seed=6))
    assert [x.token_ids.tolist() for x in a] == [x.token_ids.tolist() for x in b]
    assert [x.token_ids.tolist() for x in a] != [x.token_ids.tolist() for x in c]


def test_sampling_filters():
    logits = torch.log(torch.tensor([[0.5, 0.3, 0.15, 0.05]]))
    g = torch.Generator().manual_seed(0)
    seen_k = {int(_sample(logits, SamplingParams(top_k=2), g)[0]) for _ in range(200)}
    assert seen_k == {0, 1}
    seen_p = {int(_sample(logits, SamplingParams(top_p=0.6), g)[0]) for _ in range(200)}
    assert seen_p == {0, 1}                       # 0.5 alone is short of 0.6: the next token joins the nucleus
    tok, lp = _sample(logits, SamplingParams(temperature=0.0), g)
    assert int(tok) == 0 and abs(float(lp) - np.log(0.5)) < 1e-6
    tok, lp = _sample(logits, SamplingParams(temperature=5.0, top_k=2), g)
    assert abs(float(lp) - float(torch.log_softmax(logits, -1)[0, tok])) < 1e-6   # reported under the unmodified distribution


def test_generation_and_evaluation_clis(tmp_path, capsys):
    import json

    from halo_b200.checkpoint.save import save_model
    from halo_b200.entrypoints import evaluation, generation

    cfg = dataclasses.replace(dense_cfg(), num_nextn_predict_layers=1)
    model = build_model(cfg, device="cpu", seed=2, gradient_checkpointing=False)
    ckpt = str(tmp_path / "ckpt")
    save_model(model, ckpt, save_dtype=None)
    prompts = tmp_path / "prompts.jsonl"
    prompts.write_text("\n".join(json.dumps({"id": i, "prompt_ids": [1 + i, 2, 3]}) for i in range(3)))
    out = tmp_path / "out.jsonl"
    assert generation.main([ckpt, "--prompts", str(prompts), "--out", str(out), "--n", "2", "--batch", "4", "--max-new-tokens", "5",
                            "--device", "cpu", "--temperature", "0"]) == 0
    recs = [json.loads(l) for l in open(out)]
    assert len(recs) == 6 and all(len(r["completion_ids"]) == 5 for r in recs)
    assert recs[0]["completion_ids"] == recs[1]["completion_ids"] and recs[0]["id"] == 0       # greedy samples agree
    data = tmp_path / "eval.jsonl"
    rng = np.random.default_rng(0)
    data.write_text("\n".join(json.dumps({"input_ids": rng.integers(0, 128, size=n).tolist()}) for n in (30, 50, 20)))
    capsys.readouterr()
    assert evaluation.main([ckpt, "--data", str(data), "--device", "cpu", "--row-length", "64", "--mtp"]) == 0
    report = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    b = pack_documents([np.asarray(json.loads(l)["input_ids"]) for l in open(data)])
    with torch.no_grad():
        want = model.__class__.forward(build_model(dense_cfg(), device="cpu", seed=2, gradient_checkpointing=False), b.input_ids,
                                       b.position_ids, b.cu_seqlens, b.labels).item()
    assert report["tokens"] == 97 and abs(report["loss"] - want) < 1e-4
    assert 0.0 <= report["mtp_acceptance"] <= 1.0 and report["mtp_loss"] > 0


def test_generation_callbacks(tmp_path):
    from halo_b200.callbacks.generation import GenerateExamplesCallback, MtpAcceptanceGate, MtpGateFailed, PhaseTimerCallback
    from halo_b200.configs.arguments import TrainingArguments
    from halo_b200.diagnostics.phase_timers import PhaseTimers
    from halo_b200.trainers.sft import SFTTrainer

    cfg = dataclasses.replace(dense_cfg(), num_nextn_predict_layers=1)
    rng = np.random.default_rng(0)
    train = [pack_documents([rng.integers(0, 128, size=40)]) for _ in range(2)]

    def run(lr, gate):
        model = build_model(cfg, device="cpu", seed=1, gradient_checkpointing=False)
        args = TrainingArguments(output_dir=str(tmp_path / f"run{lr}"), max_steps=30, learning_rate=lr, optim="adamw_torch",
                                 lr_scheduler_type="constant", weight_decay=0.0, logging_steps=10)
        timers = PhaseTimers(device="cpu")
        examples = GenerateExamplesCallback([[1, 2, 3]], every=10, max_new_tokens=4)
        trainer = SFTTrainer(model, args, iter(train * 100), device=torch.device("cpu"),
                             callbacks=[examples, gate, PhaseTimerCallback(timers)])
        with timers.span("whole"):
            pass
        trainer.train()
        return trainer, examples

    gate = MtpAcceptanceGate(train, min_gain=0.2)
    trainer, examples = run(3e-3, gate)                      # the held-out rows are the training rows: acceptance rises
    assert gate.final > gate.baseline + 0.2
    assert [h["step"] for h in examples.history] == [10, 20, 30] and len(examples.history[0]["examples"][0]["completion_ids"]) == 4
    assert any("phase/whole" in rec for rec in trainer.log_history)
    with pytest.raises(MtpGateFailed, match="rejected"):
        run(0.0 + 1e-12, MtpAcceptanceGate(train, min_gain=0.2))     # nothing learned: the gate fails the run
