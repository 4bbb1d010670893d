"""Multi-token-prediction head on CPU: shifted targets on packed rows, the two objectives (detached leaves the
trunk's gradients those of the plain model), acceptance counting, parameter counts and checkpoint names."""

import dataclasses

import numpy as np
import pytest
import torch

from halo_b200.checkpoint.load import from_pretrained
from halo_b200.checkpoint.save import save_model
from halo_b200.data.packing import pack_documents
from halo_b200.models.config import ModelConfig, tiny_moe_config
from halo_b200.models.mtp import IGNORE, draft_acceptance, shifted_targets
from halo_b200.models.qwen3 import build_model


def dense_cfg(**kw):
    return ModelConfig(vocab_size=256, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=16, intermediate_size=96, moe_intermediate_size=0, num_experts=0, model_type="qwen3", **kw)


def batch(cfg, seed=0):
    rng = np.random.default_rng(seed)
    return pack_documents([rng.integers(0, cfg.vocab_size, size=n) for n in (20, 13, 31)])


def test_shifted_targets_stop_at_document_ends():
    b = batch(dense_cfg())
    got = shifted_targets(b.labels, b.cu_seqlens)
    ids, cu = b.input_ids.reshape(-1), list(map(int, b.cu_seqlens))
    for d in range(len(cu) - 1):
        lo, hi = cu[d], cu[d + 1]
        for t in range(lo, hi):
            want = ids[t + 2].item() if t + 2 < hi else IGNORE
            assert got[t].item() == want, (d, t)


@pytest.mark.parametrize("kind", ["dense", "moe"])
def test_objectives(kind):
    base = dense_cfg() if kind == "dense" else dataclasses.replace(tiny_moe_config(), num_hidden_layers=2)
    b = batch(base)
    plain = build_model(base, device="cpu", seed=3, gradient_checkpointing=False)
    plain(b.input_ids, b.position_ids, b.cu_seqlens, b.labels).backward()
    grads = {}
    for objective in ("detached", "joint"):
        cfg = dataclasses.replace(base, num_nextn_predict_layers=1, mtp_objective=objective, mtp_loss_weight=0.5)
        m = build_model(cfg, device="cpu", seed=3, gradient_checkpointing=(objective == "joint"))
        assert cfg.param_counts()["total"] == sum(p.numel() for p in m.parameters())
        loss = m(b.input_ids, b.position_ids, b.cu_seqlens, b.labels)
        with torch.no_grad():
            next_only = plain(b.input_ids, b.position_ids, b.cu_seqlens, b.labels)
        assert torch.allclose(loss.detach(), next_only + 0.5 * m.last_mtp_loss, atol=1e-5)
        loss.backward()
        grads[objective] = {n: p.grad.clone() for n, p in m.named_parameters()}
        assert all(g.abs().sum() > 0 for n, g in grads[objective].items() if n.startswith("mtp.")), objective
    for n, p in plain.named_parameters():
        assert torch.allclose(grads["detached"][n], p.grad, atol=1e-6, rtol=1e-4), n      # the trunk never sees the head
    assert any(not torch.allclose(grads["joint"][n], p.grad, atol=1e-6) for n, p in plain.named_parameters())


def test_acceptance_and_training():
    cfg = dense_cfg(num_nextn_predict_layers=1)
    m = build_model(cfg, device="cpu", seed=1, gradient_checkpointing=False)
    b = batch(cfg, 5)
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    for _ in range(30):
        opt.zero_grad()
        m(b.input_ids, b.position_ids, b.cu_seqlens, b.labels).backward()
        opt.step()
    with torch.no_grad():
        ctx = m.make_context(b.position_ids.reshape(-1), b.cu_seqlens)
        states = m.mtp_states(m.trunk_states(b.input_ids, ctx), b.input_ids, ctx)
        targets = shifted_targets(b.labels, b.cu_seqlens)
        accepted, scored = draft_acceptance(states, m.head_weight(), targets, chunk_rows=16)
    assert int(scored) == int((targets != IGNORE).sum()) == 64 - 2 * 3
    assert int(accepted) > int(scored) // 2          # the batch is memorised


def test_checkpoint_names_and_round_trip(tmp_path):
    import json

    cfg = dataclasses.replace(tiny_moe_config(), num_hidden_layers=2, num_nextn_predict_layers=1)
    m = build_model(cfg, device="cpu", seed=2)
    d = str(tmp_path / "ckpt")
    save_model(m, d, save_dtype=None)
    names = set(json.load(open(f"{d}/model.safetensors.index.json"))["weight_map"]) if (tmp_path / "ckpt" / "model.safetensors.index.json").exists() else None
    if names is None:
        from safetensors import safe_open

        with safe_open(f"{d}/model.safetensors", "pt") as f:
            names = set(f.keys())
    assert {"model.layers.2.enorm.weight", "model.layers.2.hnorm.weight", "model.layers.2.eh_proj.weight",
            "model.layers.2.shared_head.norm.weight", "model.layers.2.self_attn.q_proj.weight",
            "model.layers.2.mlp.experts.7.down_proj.weight"} <= names
    back = from_pretrained(d, device="cpu", dtype=torch.float32)
    for (n, a), (_, c) in zip(m.named_parameters(), back.named_parameters()):
        assert torch.equal(a, c), n
