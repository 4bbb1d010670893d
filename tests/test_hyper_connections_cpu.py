"""Hyper-connected decoder on CPU: a fresh model computes the plain residual model's function, every
hyper-connection parameter receives a gradient, recompute policies agree, checkpoints round-trip, and a few
optimizer steps lower the loss."""

import dataclasses

import numpy as np
import pytest
import torch

from halo_b200.checkpoint.load import from_pretrained
from halo_b200.checkpoint.save import save_model
from halo_b200.data.packing import pack_documents
from halo_b200.models.config import ModelConfig, tiny_moe_config
from halo_b200.models.qwen3 import build_model


def cfgs(kind):
    if kind == "dense":
        plain = ModelConfig(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                            head_dim=16, intermediate_size=96, moe_intermediate_size=0, num_experts=0, model_type="qwen3")
    else:
        plain = dataclasses.replace(tiny_moe_config(), num_hidden_layers=2)
    return plain, dataclasses.replace(plain, hc_mult=4, hc_sinkhorn_iters=5)


def batch(cfg):
    rng = np.random.default_rng(0)
    return pack_documents([rng.integers(0, cfg.vocab_size, size=n) for n in (33, 31)])


def loss_of(model, b):
    return model(b.input_ids, b.position_ids, b.cu_seqlens, b.labels)


@pytest.mark.parametrize("kind", ["dense", "moe"])
def test_fresh_model_is_the_plain_residual_model(kind):
    plain_cfg, hc_cfg = cfgs(kind)
    b = batch(plain_cfg)
    plain = build_model(plain_cfg, device="cpu", seed=2, gradient_checkpointing=False)
    hc = build_model(hc_cfg, device="cpu", seed=2, gradient_checkpointing=False)
    assert abs(loss_of(plain, b).item() - loss_of(hc, b).item()) < 2e-4
    loss = loss_of(hc, b)
    loss.backward()
    for name, p in hc.named_parameters():
        if "_hc." in name or name.startswith("hc_head."):
            assert p.dtype == torch.float32 and p.grad is not None, name
            if not name.endswith("scale"):         # the scales multiply a projection that is still zero
                assert p.grad.abs().sum() > 0, name
    assert hc_cfg.param_counts()["total"] == sum(p.numel() for p in hc.parameters())


def test_recompute_policies_agree_and_training_moves():
    _, hc_cfg = cfgs("moe")
    b = batch(hc_cfg)
    ref = build_model(hc_cfg, device="cpu", seed=4, gradient_checkpointing=False)
    loss_of(ref, b).backward()
    for policy in ("full", "mlp"):
        m = build_model(hc_cfg, device="cpu", seed=4, gradient_checkpointing=True)
        for layer in m.layers:
            layer.recompute_policy = policy
        loss_of(m, b).backward()
        for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
            assert torch.allclose(p.grad, q.grad, atol=1e-6, rtol=1e-4), (policy, n)
    opt = torch.optim.AdamW(ref.parameters(), lr=3e-3)
    first = None
    for _ in range(8):
        opt.zero_grad()
        loss = loss_of(ref, b)
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
    assert loss.item() < first - 0.3
    assert ref.layers[0].attn_hc.fn.abs().sum() > 0            # the projection left zero


def test_checkpoint_round_trip(tmp_path):
    _, hc_cfg = cfgs("dense")
    m = build_model(hc_cfg, device="cpu", seed=1)
    with torch.no_grad():
        for name, p in m.named_parameters():
            if "_hc." in name or name.startswith("hc_head."):
                p.add_(torch.randn(p.shape, generator=torch.Generator().manual_seed(3)) * 0.01)
    d = str(tmp_path / "ckpt")
    save_model(m, d, save_dtype=None)
    assert ModelConfig.load(d) == hc_cfg
    back = from_pretrained(d, device="cpu", dtype=torch.float32)
    for (n, a), (_, c) in zip(m.named_parameters(), back.named_parameters()):
        assert torch.equal(a, c), n


def test_layouts_that_are_not_built_are_refused():
    _, hc_cfg = cfgs("dense")
    with pytest.raises(ValueError, match="hyper-connected"):
        build_model(hc_cfg, device="cpu", layer_range=(0, 1), has_head=False)


def test_gated_variant_trains_and_round_trips(tmp_path):
    plain_cfg, _ = cfgs("dense")
    cfg = dataclasses.replace(plain_cfg, hc_mult=2, hc_kind="gated", hc_mix_rank=8)
    m = build_model(cfg, device="cpu", seed=6)
    assert cfg.param_counts()["total"] == sum(p.numel() for p in m.parameters())
    b = batch(cfg)
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    losses = []
    for _ in range(8):
        opt.zero_grad()
        loss = loss_of(m, b)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0] - 0.3
    assert all(p.grad is not None and p.grad.abs().sum() > 0 for n, p in m.named_parameters() if "_hc." in n)
    d = str(tmp_path / "ckpt")
    save_model(m, d, save_dtype=None)
    back = from_pretrained(d, device="cpu", dtype=torch.float32)
    assert abs(loss_of(back, b).item() - loss_of(m, b).item()) < 1e-6
