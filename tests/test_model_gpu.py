"""The whole decoder on the CUDA kernels against its own CPU/PyTorch path, and a few training steps."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg():
    from halo_b200.models.config import ModelConfig

    return ModelConfig(vocab_size=4096, hidden_size=256, num_hidden_layers=2, num_attention_heads=2,
                       num_key_value_heads=1, head_dim=128, moe_intermediate_size=128, num_experts=32,
                       num_experts_per_tok=4, intermediate_size=512)


def test_moe_model_loss_and_grads_match_cpu_path():
    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.qwen3 import build_model
    from halo_b200.ops import _lib

    cfg = _cfg()
    gpu = build_model(cfg, device="cuda", seed=0, gradient_checkpointing=True)
    cpu = build_model(cfg, device="cpu", seed=0, gradient_checkpointing=False)
    with torch.no_grad():
        for (n, pc), (_, pg) in zip(cpu.named_parameters(), gpu.named_parameters()):
            pc.copy_(pg.float().cpu())
    b = synthetic_packed_batch(700, cfg.vocab_size, seed=1, lo=50, hi=300)
    d = b.to("cuda")
    loss_g = gpu(d.input_ids, d.position_ids, d.cu_seqlens, d.labels)
    loss_g.backward()
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    loss_c = cpu(b.input_ids, b.position_ids, b.cu_seqlens, b.labels)
    loss_c.backward()
    assert abs(loss_g.item() - loss_c.item()) <= 0.05, (loss_g.item(), loss_c.item())
    checked = 0
    for (n, pc), (_, pg) in zip(cpu.named_parameters(), gpu.named_parameters()):
        gc, gg = pc.grad.float().flatten(), pg.grad.float().cpu().flatten()
        if gc.norm() < 1e-6:
            continue
        cos = torch.dot(gc, gg) / (gc.norm() * gg.norm() + 1e-12)
        ratio = gg.norm() / gc.norm()
        assert cos > 0.97, f"{n}: grad cosine {cos.item():.4f}"
        assert 0.8 < ratio < 1.25, f"{n}: grad norm ratio {ratio.item():.3f}"
        checked += 1
    assert checked >= 10


def test_dense_model_trains():
    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.config import ModelConfig
    from halo_b200.models.qwen3 import build_model
    from halo_b200.optim.adamw_bf16 import AdamWBF16
    from halo_b200.trainers.engine import TrainEngine

    cfg = ModelConfig(vocab_size=2048, hidden_size=256, num_hidden_layers=2, num_attention_heads=2,
                      num_key_value_heads=2, head_dim=128, intermediate_size=512, num_experts=0, model_type="qwen3")
    model = build_model(cfg, device="cuda", seed=0)
    opt = AdamWBF16(list(model.named_parameters()), lr=3e-3, weight_decay=0.0)
    eng = TrainEngine(model, opt, "cuda", max_grad_norm=1.0)
    batch = synthetic_packed_batch(1024, cfg.vocab_size, seed=0, lo=64, hi=400).pin()
    losses = [eng.train_step(batch).loss.item() for _ in range(12)]
    assert losses[0] > 7.0 and losses[-1] < losses[0] - 1.0, losses


def test_graft_smoke():
    import __graft_entry__ as entry

    entry.smoke()
