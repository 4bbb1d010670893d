"""CPU checks of the pieces that need no GPU: packing, configs, the optimizer's CPU twin, the
model's CPU path (which doubles as the oracle of the GPU tests)."""

import numpy as np
import torch

from halo_b200.data.packing import pack_documents, synthetic_packed_batch
from halo_b200.models.config import PRESETS, ModelConfig, tiny_moe_config
from halo_b200.models.qwen3 import build_model
from halo_b200.optim.adamw_bf16 import (AdamWBF16, adamw_bf16_step_reference, param_name_hash, philox4x32_10,
                                         sr_key_pair)


def test_pack_documents_labels_stay_inside_documents():
    b = pack_documents([[1, 2, 3], [4, 5], [6]], row_len=8)
    assert b.input_ids.tolist() == [1, 2, 3, 4, 5, 6, 0, 0]
    assert b.position_ids.tolist() == [0, 1, 2, 0, 1, 0, 0, 1]
    assert b.labels.tolist() == [2, 3, -100, 5, -100, -100, -100, -100]
    assert b.cu_seqlens.tolist() == [0, 3, 5, 6, 8]
    assert b.n_scored == 3


def test_synthetic_batch_fills_row():
    b = synthetic_packed_batch(4096, 1000, seed=1, lo=32, hi=256)
    assert b.n_tokens == 4096 and b.cu_seqlens[-1] == 4096
    assert int(b.input_ids.max()) < 1000


def test_config_round_trip_and_counts():
    for name, make in PRESETS.items():
        cfg = make()
        back = ModelConfig.from_hf_dict(cfg.to_hf_dict())
        assert back.hidden_size == cfg.hidden_size and back.num_experts == cfg.num_experts, name
    c = PRESETS["moe-30b-a3b"]().param_counts()
    assert 30.0e9 < c["total"] < 31.0e9
    assert 3.0e9 < c["active"] < 3.6e9


def test_philox_known_answer():
    # Random123 known-answer vector for philox4x32-10 with zero key / counter
    out = philox4x32_10(0, 0, np.zeros(1, dtype=np.uint64))[0]
    assert [hex(int(x)) for x in out] == ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]


def test_sr_keys_depend_on_step_and_name():
    a = sr_key_pair(0xB165EED, 1, param_name_hash("a.weight"))
    assert a != sr_key_pair(0xB165EED, 2, param_name_hash("a.weight"))
    assert a != sr_key_pair(0xB165EED, 1, param_name_hash("b.weight"))
    assert a == sr_key_pair(0xB165EED, 1, param_name_hash("a.weight"))


def test_adamw_reference_tracks_fp32_adam_and_is_unbiased():
    torch.manual_seed(0)
    n = 4096
    p32 = torch.randn(n)
    p = p32.bfloat16().clone()
    m = torch.zeros(n, dtype=torch.bfloat16)
    v = torch.zeros(n, dtype=torch.bfloat16)
    ref = torch.nn.Parameter(p.float().clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, weight_decay=0.0, eps=1e-8)
    for step in range(1, 6):
        g = torch.randn(n) * 0.1
        ref.grad = g.bfloat16().float()
        opt.step()
        bc1 = 1 - 0.9**step
        adamw_bf16_step_reference(p, g.bfloat16(), m, v, beta1=0.9, beta2=0.999, step_size=1e-2 / bc1,
                                  bc2_sqrt=(1 - 0.999**step) ** 0.5, eps=1e-8, wd_factor=1.0, key=1, step=step,
                                  name_hash=7)
    assert (p.float() - ref.data).abs().max().item() < 0.05
    assert abs((p.float() - ref.data).mean().item()) < 2e-3  # stochastic rounding: no systematic drift


def test_optimizer_requires_names_and_steps_on_cpu():
    w = torch.nn.Parameter(torch.randn(10).bfloat16())
    try:
        AdamWBF16([{"params": [w]}])
        raise AssertionError("expected a refusal")
    except ValueError:
        pass
    opt = AdamWBF16([("w", w)], lr=1e-2)
    w.grad = torch.ones(10, dtype=torch.bfloat16)
    before = w.detach().clone()
    opt.step()
    assert not torch.equal(before, w.detach())


def test_tiny_moe_cpu_forward_backward_and_checkpointing_agree():
    cfg = tiny_moe_config()
    b = synthetic_packed_batch(384, cfg.vocab_size, seed=0, lo=32, hi=200)
    losses, grads = [], []
    for gc in (False, True):
        model = build_model(cfg, device="cpu", seed=0, gradient_checkpointing=gc)
        loss = model(b.input_ids, b.position_ids, b.cu_seqlens, b.labels)
        loss.backward()
        losses.append(loss.item())
        grads.append(model.layers[0].mlp.experts_gate_up.grad.clone())
    assert abs(losses[0] - np.log(cfg.vocab_size)) < 0.2
    assert abs(losses[0] - losses[1]) < 1e-6
    assert torch.allclose(grads[0], grads[1], atol=1e-7)


def test_documents_do_not_attend_across_boundaries():
    cfg = tiny_moe_config()
    model = build_model(cfg, device="cpu", seed=0, gradient_checkpointing=False)
    rng = np.random.default_rng(0)
    d1, d2, d3 = (rng.integers(0, cfg.vocab_size, size=n) for n in (40, 50, 60))
    a = pack_documents([d1, d2])
    b = pack_documents([d3, d2])
    with torch.no_grad():
        ha = model.hidden_states(a.input_ids, a.position_ids, a.cu_seqlens)
        hb = model.hidden_states(b.input_ids, b.position_ids, b.cu_seqlens)
    same = (ha[40:] - hb[60:]).abs().max().item()
    other = (ha[:40] - hb[:40]).abs().max().item()
    assert same < 2e-2, same          # fp32 reduction-order noise only
    assert other > 20 * same, (same, other)  # negative control: different documents do differ


def test_recompute_policies_give_the_same_gradients():
    """full / mlp-half / no recomputation differ only in what is kept alive, never in the result."""
    import dataclasses

    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.config import PRESETS
    from halo_b200.models.qwen3 import build_model, plan_recompute

    cfg = dataclasses.replace(PRESETS["tiny-moe"](), num_hidden_layers=3)
    b = synthetic_packed_batch(128, cfg.vocab_size, seed=0, lo=8, hi=64)
    grads = {}
    for policy in ("full", "mlp", "none"):
        m = build_model(cfg, device="cpu", dtype=torch.float32, seed=2)
        for layer in m.layers:
            layer.recompute_policy = policy
        loss = m(b.input_ids, b.position_ids, b.cu_seqlens, b.labels)
        loss.backward()
        grads[policy] = (loss.detach(), {n: p.grad.clone() for n, p in m.named_parameters()})
    for policy in ("mlp", "none"):
        assert torch.allclose(grads[policy][0], grads["full"][0], atol=1e-6)
        for n, g in grads["full"][1].items():
            assert torch.allclose(grads[policy][1][n], g, rtol=1e-5, atol=1e-7), (policy, n)
    m = build_model(cfg, device="cpu", dtype=torch.float32, seed=2)
    per_layer = 128 * 4 * (3 * cfg.hidden_size + 2 * cfg.qkv_dim + cfg.num_attention_heads * cfg.head_dim) + 128 * 4 * cfg.num_attention_heads
    assert plan_recompute(m, 128, free_bytes=2 * per_layer + 10, reserve_bytes=0) == 2
    assert [l.recompute_policy for l in m.layers] == ["full", "mlp", "mlp"]
