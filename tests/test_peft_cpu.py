"""Low-rank adapters on CPU: the adapted model starts as the base model, only the pairs train, the low-rank path
and the effective-bank path give the gradients of the plain formula, adapters round-trip through the PEFT layout
(and load in ``peft`` when it is installed), and the three merge routes (in memory, merged save, offline tool)
agree."""

import dataclasses

import numpy as np
import pytest
import torch

from halo_b200.checkpoint.load import from_pretrained
from halo_b200.checkpoint.save import save_model
from halo_b200.checkpoint.tools import merge_adapter
from halo_b200.data.packing import pack_documents
from halo_b200.models.config import ModelConfig, tiny_moe_config
from halo_b200.models.qwen3 import build_model
from halo_b200.peft.lora import (LoraSpec, adapter_state_dict, apply_lora, load_adapters, merge_adapters_into_weights,
                                 read_adapter_spec)


def dense_cfg():
    return ModelConfig(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=16, intermediate_size=96, moe_intermediate_size=0, num_experts=0, model_type="qwen3")


def moe_cfg():
    return dataclasses.replace(tiny_moe_config(), num_hidden_layers=2, shared_expert_intermediate_size=64)


def batch(cfg, seed=0):
    rng = np.random.default_rng(seed)
    return pack_documents([rng.integers(0, cfg.vocab_size, size=n) for n in (40, 24)])


def loss_of(model, b):
    return model(b.input_ids, b.position_ids, b.cu_seqlens, b.labels)


def randomize_b(model, seed=1):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if ".lora.B." in name or ".expert_lora.B_" in name:
                p.normal_(0.0, 0.05, generator=g)


@pytest.mark.parametrize("kind", ["dense", "moe"])
def test_adapted_model_starts_as_base_and_trains_only_pairs(kind):
    cfg = dense_cfg() if kind == "dense" else moe_cfg()
    model = build_model(cfg, device="cpu", seed=3, gradient_checkpointing=(kind == "moe"))
    b = batch(cfg)
    base_loss = loss_of(model, b).item()
    stats = apply_lora(model, LoraSpec(r=4, alpha=8, target_modules="all-linear" if kind == "moe" else
                                       ["q_proj", "v_proj", "o_proj", "gate_proj", "down_proj"]))
    assert stats["trainable"] < stats["frozen"] // 4
    assert abs(loss_of(model, b).item() - base_loss) < 1e-6            # B = 0
    randomize_b(model)
    loss = loss_of(model, b)
    assert abs(loss.item() - base_loss) > 1e-5
    loss.backward()
    for name, p in model.named_parameters():
        is_pair = ".lora." in name or ".expert_lora." in name
        assert p.requires_grad == is_pair, name
        assert (p.grad is not None and p.grad.abs().sum() > 0) == is_pair, name


def test_gradients_match_the_folded_weights():
    """d loss / d (B A) through the low-rank path and through the effective banks equals what autograd gives when
    the same pairs are folded into the weights by hand."""
    cfg = moe_cfg()
    model = build_model(cfg, device="cpu", seed=5, gradient_checkpointing=False)
    apply_lora(model, LoraSpec(r=4, alpha=4, target_modules="all-linear"))
    randomize_b(model, 7)
    b = batch(cfg, 2)
    loss_of(model, b).backward()
    twin = build_model(cfg, device="cpu", seed=5, gradient_checkpointing=False)
    apply_lora(twin, LoraSpec(r=4, alpha=4, target_modules="all-linear"))
    twin.load_state_dict(model.state_dict())
    # the twin computes with explicitly folded weights: W + scale * B A as differentiable expressions
    layer, tl = model.layers[0], twin.layers[0]
    lora = tl.self_attn.lora
    q = cfg.num_attention_heads * cfg.head_dim
    folded_q = tl.self_attn.qkv_proj[:q] + lora.scale * lora.B["q_proj"] @ lora.A["q_proj"]
    x = torch.randn(5, cfg.hidden_size, generator=torch.Generator().manual_seed(0))
    want = x @ folded_q.t()
    got = layer.self_attn._qkv(x)[:, :q]
    assert torch.allclose(got, want, atol=1e-5)
    ex = tl.mlp.expert_lora
    gu, dn = ex.effective_banks(tl.mlp.experts_gate_up, tl.mlp.experts_down)
    width = cfg.moe_intermediate_size
    assert torch.allclose(gu[1, :width], tl.mlp.experts_gate_up[1, :width] + ex.scale * ex.B_gate_proj[1] @ ex.A_gate_proj[1], atol=1e-6)
    assert torch.allclose(dn[2], tl.mlp.experts_down[2] + ex.scale * ex.B_down_proj[2] @ ex.A_down_proj[2], atol=1e-6)


@pytest.mark.parametrize("kind", ["dense", "moe"])
def test_adapter_round_trip_and_three_merge_routes_agree(tmp_path, kind):
    cfg = dense_cfg() if kind == "dense" else moe_cfg()
    base = build_model(cfg, device="cpu", seed=3, gradient_checkpointing=False)
    base_dir, adapter_dir = str(tmp_path / "base"), str(tmp_path / "adapter")
    save_model(base, base_dir, save_dtype=None)
    model = from_pretrained(base_dir, device="cpu", dtype=torch.float32, gradient_checkpointing=False)
    spec = LoraSpec(r=4, alpha=8, target_modules="all-linear" if kind == "moe" else ["q_proj", "k_proj", "up_proj", "down_proj"])
    apply_lora(model, spec)
    randomize_b(model, 3)
    b = batch(cfg, 4)
    want = loss_of(model, b).item()
    save_model(model, adapter_dir)                       # adapters only
    assert read_adapter_spec(adapter_dir).target_modules == spec.target_modules
    fresh = from_pretrained(base_dir, device="cpu", dtype=torch.float32, gradient_checkpointing=False)
    apply_lora(fresh, read_adapter_spec(adapter_dir), seed=99)
    assert load_adapters(fresh, adapter_dir) == len(adapter_state_dict(model))
    assert abs(loss_of(fresh, b).item() - want) < 1e-6
    # route 1: offline tool
    merged_dir = str(tmp_path / "merged")
    merge_adapter.merge(base_dir, adapter_dir, merged_dir)
    plain = from_pretrained(merged_dir, device="cpu", dtype=torch.float32, gradient_checkpointing=False)
    assert abs(loss_of(plain, b).item() - want) < 1e-5
    # route 2: merged save
    merged_save = str(tmp_path / "merged_save")
    save_model(model, merged_save, save_dtype=None, adapters="merge")
    plain2 = from_pretrained(merged_save, device="cpu", dtype=torch.float32, gradient_checkpointing=False)
    for (n, a), (_, c) in zip(plain.named_parameters(), plain2.named_parameters()):
        assert torch.allclose(a, c, atol=1e-6), n
    # route 3: in memory
    merge_adapters_into_weights(model)
    assert abs(loss_of(model, b).item() - want) < 1e-5
    assert all(p.abs().sum() == 0 for n, p in model.named_parameters() if ".lora.B." in n or ".expert_lora.B_" in n)


def test_peft_reads_the_dense_adapters(tmp_path):
    peft = pytest.importorskip("peft")
    transformers = pytest.importorskip("transformers")
    cfg = dense_cfg()
    base_dir, adapter_dir = str(tmp_path / "base"), str(tmp_path / "adapter")
    model = build_model(cfg, device="cpu", seed=3, gradient_checkpointing=False)
    save_model(model, base_dir, save_dtype=None)
    apply_lora(model, LoraSpec(r=4, alpha=8, target_modules=["q_proj", "v_proj", "down_proj"]))
    randomize_b(model, 3)
    model.base_model_path = base_dir
    save_model(model, adapter_dir)
    hf = transformers.AutoModelForCausalLM.from_pretrained(base_dir, torch_dtype=torch.float32, attn_implementation="eager")
    hf = peft.PeftModel.from_pretrained(hf, adapter_dir).eval()
    b = batch(cfg, 1)
    with torch.no_grad():
        ours = model.hidden_states(b.input_ids[:40], b.position_ids[:40], torch.tensor([0, 40], dtype=torch.int32)) @ model.head_weight().t()
        theirs = hf(input_ids=b.input_ids[None, :40]).logits[0]
    assert (ours - theirs).abs().max().item() < 5e-2 * theirs.abs().max().item()


def test_adapters_on_the_other_families():
    """Expert pairs on gpt-oss' biased clamped-GLU banks and dense pairs on Gemma's tanh-GELU block change the function and
    get gradients; attention targets on a latent-attention model are refused by name (nothing would read them)."""
    from tests.test_families_cpu import family_config

    for family, targets in (("gpt_oss", ["q_proj", "o_proj", "experts.gate_proj", "experts.down_proj"]),
                            ("gemma3_text", ["v_proj", "gate_proj", "down_proj"]), ("deepseek_v3", ["experts.up_proj", "down_proj"])):
        cfg = family_config(family)
        model = build_model(cfg, device="cpu", seed=0, gradient_checkpointing=False)
        b = batch(cfg)
        base = float(loss_of(model, b))
        apply_lora(model, LoraSpec(r=4, alpha=8.0, target_modules=targets), seed=0)
        assert abs(float(loss_of(model, b)) - base) < 1e-6          # B starts at zero
        randomize_b(model)
        loss = loss_of(model, b)
        assert abs(float(loss) - base) > 1e-5, family
        loss.backward()
        pairs = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        assert pairs and all(p.grad is not None and float(p.grad.abs().sum()) > 0 for _, p in pairs), family
    with pytest.raises(ValueError, match="latent attention has no such projections"):
        apply_lora(build_model(family_config("deepseek_v3"), device="cpu"), LoraSpec(target_modules=["q_proj", "v_proj"]))


def test_bad_targets_are_refused():
    with pytest.raises(ValueError, match="unknown LoRA targets"):
        LoraSpec(target_modules=["qkv_proj"])
    model = build_model(dense_cfg(), device="cpu", seed=0)
    with pytest.raises(ValueError, match="name routed experts"):
        apply_lora(model, LoraSpec(target_modules=["experts.gate_proj"]))


def test_sft_entry_point_trains_and_saves_adapters_under_expert_parallelism(tmp_path):
    """Two gloo ranks, experts split over them: the run writes adapter-only checkpoints whose expert pairs cover
    every global expert, and a second run resumes from them."""
    import os
    import subprocess
    import sys

    from safetensors import safe_open

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = tmp_path / "sft.yaml"
    cfg.write_text("model_preset: tiny-moe\ninit_from_scratch: true\ndataset_format: synthetic\npacked_row_length: 256\n"
                   "max_steps: 2\nsave_steps: 2\noptim: adamw_torch\nlearning_rate: 1.0e-3\nexpert_parallel_size: 2\n"
                   f"output_dir: {tmp_path}/run\nuse_peft: true\nlora_r: 4\nlora_alpha: 8\n"
                   "lora_target_modules: [q_proj, v_proj, experts.gate_proj, experts.down_proj]\n")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "halo_b200.cli", "launch", "sft", str(cfg), "-n", "2", "--port", "29691"]
    r = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    final = tmp_path / "run" / "final"
    assert os.path.isfile(final / "adapter_config.json") and not os.path.exists(final / "config.json")
    with safe_open(str(final / "adapter_model.safetensors"), "pt") as f:
        keys = set(f.keys())
    experts = {int(k.split(".experts.")[1].split(".")[0]) for k in keys if ".experts." in k}
    assert experts == set(range(8))
    assert any("self_attn.q_proj.lora_A" in k for k in keys) and not any("k_proj" in k for k in keys)
    r = subprocess.run(cmd + ["--max_steps=3", "--resume_from_checkpoint=auto"], cwd=root, capture_output=True, text=True,
                       timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    out = r.stdout + r.stderr
    assert "step 3 " in out and "step 1 " not in out         # picked up after step 2
