"""QLoRA on CPU: the 4-bit block formats keep their error bound and pack two codes per byte; a model whose base
matrices are stored in 4 bits computes what the same model with the rounded matrices computes, under every
recomputation policy; only adapters remain as parameters; the SFT entry point trains and saves adapters."""

import dataclasses
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

from halo_b200.data.packing import pack_documents
from halo_b200.models.config import ModelConfig, tiny_moe_config
from halo_b200.models.qwen3 import build_model
from halo_b200.ops.nf4 import NF4_LEVELS, dequantize_4bit, levels, quantization_error_bound, quantize_4bit
from halo_b200.peft.lora import LoraSpec, apply_lora
from halo_b200.peft.qlora import dequantized_base_state, is_quantized, quantize_base_weights


@pytest.mark.parametrize("kind", ["nf4", "fp4"])
@pytest.mark.parametrize("nested", [False, True])
def test_block_format_error_bound_and_size(kind, nested):
    g = torch.Generator().manual_seed(0)
    w = torch.randn(128, 256, generator=g) * torch.logspace(-2, 1, 128)[:, None]       # rows of very different size
    p = quantize_4bit(w, kind, nested)
    back = dequantize_4bit(p)
    assert back.shape == w.shape and back.dtype == w.dtype and p.codes.numel() == w.numel() // 2
    maxima = w.reshape(-1, 64).abs().amax(1, keepdim=True)
    err = ((back - w).reshape(-1, 64).abs() / maxima).max()
    # nested: the maxima themselves are rounded (below 1.4 % here), which moves every value of the block by that share
    assert float(err) <= quantization_error_bound(kind) + (0.015 if nested else 1e-6)
    bits = 8.0 * p.nbytes / w.numel()
    assert bits == pytest.approx(4.5 if not nested else 4.0 + 8 / 64 + 64 / (64 * 256), abs=1e-6)
    # every level is a fixed point, zero included
    table = levels(kind)
    exact = (table[torch.randint(0, 16, (4, 64), generator=g)] * 3.0)
    exact[:, 0] = 3.0                                  # the block maximum is present
    assert torch.equal(dequantize_4bit(quantize_4bit(exact, kind)), exact)
    assert len(set(NF4_LEVELS)) == 16 and 0.0 in NF4_LEVELS and NF4_LEVELS[0] == -1.0 and NF4_LEVELS[-1] == 1.0
    with pytest.raises(ValueError, match="blocks of 64"):
        quantize_4bit(torch.zeros(10, 10), kind)


def test_int8_storage():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(64, 256, generator=g) * torch.logspace(-2, 1, 64)[:, None]
    p = quantize_4bit(w, "int8")
    back = dequantize_4bit(p)
    assert p.codes.numel() == w.numel() and 8.0 * p.nbytes / w.numel() == 8.5
    err = ((back - w).reshape(-1, 64).abs() / w.reshape(-1, 64).abs().amax(1, keepdim=True)).max()
    assert float(err) <= quantization_error_bound("int8") + 1e-6
    with pytest.raises(ValueError, match="4-bit option"):
        quantize_4bit(w, "int8", nested=True)


def _moe_cfg():
    return dataclasses.replace(tiny_moe_config(), num_hidden_layers=2, shared_expert_intermediate_size=64, vocab_size=512)


def _dense_cfg():
    return ModelConfig(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=16, intermediate_size=128, moe_intermediate_size=0, num_experts=0, model_type="qwen3")


@pytest.mark.parametrize("kind", ["dense", "moe"])
@pytest.mark.parametrize("policy", ["full", "mlp", "none"])
def test_quantized_base_equals_the_rounded_model(kind, policy):
    cfg = _dense_cfg() if kind == "dense" else _moe_cfg()
    spec = LoraSpec(r=4, alpha=8.0, target_modules=["q_proj", "v_proj", "down_proj"] + (["experts.gate_proj"] if kind == "moe" else []))
    rng = np.random.default_rng(0)
    b = pack_documents([rng.integers(0, cfg.vocab_size, size=n) for n in (40, 24)])

    def make():
        m = build_model(cfg, device="cpu", seed=3, gradient_checkpointing=policy != "none")
        for layer in m.layers:
            layer.recompute_policy = policy
        apply_lora(m, spec, seed=0)
        with torch.no_grad():
            for n, p in m.named_parameters():
                if re.search(r"\.B[._]", n):
                    p.normal_(0.0, 0.05, generator=torch.Generator().manual_seed(len(n)))     # a zero B hides the adapters
        return m

    q, plain = make(), make()
    assert sum(float(p.abs().sum()) > 0 for n, p in q.named_parameters() if re.search(r"\.B[._]", n)) >= 2 * cfg.num_hidden_layers
    before = {n for n, _ in q.named_parameters()}
    stats = quantize_base_weights(q, "nf4")
    assert is_quantized(q) and stats["matrices"] == (4 if kind == "dense" else 6) * cfg.num_hidden_layers
    gone = before - {n for n, _ in q.named_parameters()}
    assert gone == set(dequantized_base_state(q)) and all(p.requires_grad or "lora" not in n for n, p in q.named_parameters())
    with pytest.raises(AttributeError):
        q.layers[0].self_attn.qkv_proj                      # exists only while the layer runs
    with torch.no_grad():
        for name, rounded in dequantized_base_state(q).items():
            plain.get_parameter(name).copy_(rounded)
    loss_q, loss_p = (m(b.input_ids, b.position_ids, b.cu_seqlens, b.labels) for m in (q, plain))
    loss_q = loss_q.loss if hasattr(loss_q, "loss") else loss_q
    loss_p = loss_p.loss if hasattr(loss_p, "loss") else loss_p
    assert torch.allclose(loss_q, loss_p, atol=1e-6)
    loss_q.sum().backward()
    loss_p.sum().backward()
    grads = {n: p.grad for n, p in plain.named_parameters() if p.grad is not None}
    seen = 0
    for n, p in q.named_parameters():
        if p.requires_grad:
            assert torch.allclose(p.grad, grads[n], atol=1e-6), n
            seen += 1
    assert seen >= 6
    with pytest.raises(AttributeError):
        q.layers[1].mlp.down_proj if kind == "dense" else q.layers[1].mlp.experts_down
    with pytest.raises(ValueError, match="already stored"):
        quantize_base_weights(q)


def test_trainable_base_is_refused():
    m = build_model(_dense_cfg(), device="cpu", seed=0)
    with pytest.raises(ValueError, match="only frozen base weights"):
        quantize_base_weights(m)


def test_sft_entry_point_trains_a_quantized_base(tmp_path):
    from safetensors import safe_open

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = tmp_path / "sft.yaml"
    cfg.write_text("model_preset: tiny-moe\ninit_from_scratch: true\ndataset_format: synthetic\npacked_row_length: 256\n"
                   "max_steps: 3\nsave_steps: 3\noptim: adamw_torch\nlearning_rate: 2.0e-3\nlogging_steps: 1\n"
                   f"output_dir: {tmp_path}/run\nuse_peft: true\nlora_r: 4\nlora_alpha: 8\nload_in_4bit: true\n"
                   "use_bnb_nested_quant: true\nlora_target_modules: [q_proj, v_proj, experts.gate_proj, experts.down_proj]\n")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, "-m", "halo_b200.cli", "launch", "sft", str(cfg)], cwd=root, capture_output=True, text=True,
                       timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "quantised base (nf4):" in r.stdout + r.stderr
    final = tmp_path / "run" / "final"
    assert os.path.isfile(final / "adapter_config.json")
    with safe_open(str(final / "adapter_model.safetensors"), "pt") as f:
        assert any("lora_A" in k for k in f.keys())
    eight = tmp_path / "eight.yaml"
    eight.write_text(cfg.read_text().replace("load_in_4bit: true\n", "load_in_8bit: true\n").replace("use_bnb_nested_quant: true\n", "")
                     .replace(f"{tmp_path}/run", f"{tmp_path}/run8"))
    r = subprocess.run([sys.executable, "-m", "halo_b200.cli", "launch", "sft", str(eight)], cwd=root, capture_output=True, text=True,
                       timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "quantised base (int8):" in r.stdout + r.stderr and os.path.isfile(tmp_path / "run8" / "final" / "adapter_config.json")
    bad = tmp_path / "bad.yaml"
    bad.write_text(cfg.read_text().replace("use_peft: true\n", ""))
    r = subprocess.run([sys.executable, "-m", "halo_b200.cli", "launch", "sft", str(bad)], cwd=root, capture_output=True, text=True,
                       timeout=300, env=env)
    assert r.returncode != 0 and "need use_peft" in r.stdout + r.stderr
