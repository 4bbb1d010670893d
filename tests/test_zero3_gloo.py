"""ZeRO-3 for the decoder layers on gloo ranks: a model whose layer matrices live as 1 / N slices trains exactly like the
replicated model (same losses, same weights after several steps, with gradient accumulation and clipping), saves one
ordinary checkpoint, and a dense and a MoE (expert-parallel) model both work."""

import pytest
import torch

from tests.common.gloo import run_gloo_ranks


def _train(rank, world, sharded, moe, out_dir=None, light_layers=0):
    import dataclasses

    import torch.distributed as dist

    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.config import PRESETS
    from halo_b200.models.qwen3 import build_model
    from halo_b200.optim.factory import build_optimizer
    from halo_b200.parallel.runtime import ParallelRuntime
    from halo_b200.trainers.engine import TrainEngine

    cfg = dataclasses.replace(PRESETS["tiny-moe"](), num_hidden_layers=3)
    if not moe:
        cfg = dataclasses.replace(cfg, num_experts=0, intermediate_size=96)
    transport, ep_group = None, None
    if moe:
        from halo_b200.parallel.expert_parallel import CollectiveTransport

        transport, ep_group = CollectiveTransport(dist.group.WORLD), dist.group.WORLD
    model = build_model(cfg, device="cpu", dtype=torch.float32, seed=11, transport=transport, gradient_checkpointing=True)
    for layer in model.layers[len(model.layers) - light_layers:]:
        layer.recompute_policy = "mlp"           # the lighter policy: attention keeps its graph, the feed-forward half is re-run
    parallel = ParallelRuntime("cpu", dp_group=dist.group.WORLD, ep_group=ep_group, transport=transport)
    zero3 = None
    if sharded:
        from halo_b200.parallel.zero3 import shard_layers

        zero3 = shard_layers(model, dist.group.WORLD, "cpu", ep_world=world if moe else 1)
        assert all(p.numel() == 0 for items in zero3.params for _, p, *_ in items)       # the full copies are gone
    opt = build_optimizer(model, "adamw_bf16", lr=3e-3, weight_decay=0.05)               # fp32 parameters: plain AdamW arithmetic
    if sharded:
        names = [n for g in opt.param_groups for n in g["param_names"]]
        assert "zero3_shard" in names and not any(n in zero3.managed_names() for n in names)
        decay = next(g for g in opt.param_groups if "zero3_shard" in g["param_names"])
        assert decay["weight_decay"] == 0.05
    eng = TrainEngine(model, opt, "cpu", max_grad_norm=0.7, parallel=parallel)
    losses = []
    for step in range(3):
        for micro in range(2):                                 # two micro-batches per step: the gradient shard accumulates
            b = synthetic_packed_batch(256, cfg.vocab_size, seed=100 * rank + 10 * step + micro)
            out = eng.train_step(b, accumulate=micro == 0)
            losses.append(float(out.loss))
        losses.append(float(out.grad_norm))
    weights = {}
    if sharded:
        for li in range(len(model.layers)):
            weights.update(zero3.full_tensors(li))
        for n, p in model.named_parameters():
            if not getattr(p, "zero3_managed", False) and n != "zero3_shard" and not getattr(p, "is_expert", False):
                weights[n] = p.detach().clone()
        if out_dir is not None:
            from halo_b200.checkpoint.load import load_model_weights
            from halo_b200.checkpoint.save import save_model

            save_model(model, out_dir, save_dtype=None)
            dist.barrier()
            # the saved directory loads back into the sharded model: every rank keeps its slices of the full tensors
            before = zero3.shard.detach().clone()
            with torch.no_grad():
                zero3.shard.zero_()
            load_model_weights(model, out_dir)
            assert torch.equal(zero3.shard.detach(), before)
    else:
        weights = {n: p.detach().clone() for n, p in model.named_parameters() if not getattr(p, "is_expert", False)}
    return losses, weights


def _worker(rank, world, moe, out_dir, light_layers=0):
    want_l, want_w = _train(rank, world, False, moe, light_layers=light_layers)
    got_l, got_w = _train(rank, world, True, moe, out_dir, light_layers=light_layers)
    assert len(want_l) == len(got_l)
    for a, b in zip(want_l, got_l):
        assert abs(a - b) <= 1e-5 * max(1.0, abs(a)), (want_l, got_l)
    assert set(got_w) == set(want_w), set(got_w) ^ set(want_w)
    for n in want_w:
        # Adam turns a rounding-level difference of a near-zero gradient into a difference of up to the step size for that
        # element; anything systematic would move whole tensors
        diff = (got_w[n] - want_w[n]).abs()
        assert float(diff.max()) < 2e-3 and float(diff.mean()) < 2e-6, (n, float(diff.max()), float(diff.mean()))
    if rank == 0 and out_dir is not None:
        from halo_b200.checkpoint.load import CheckpointIndex

        idx = CheckpointIndex(out_dir)
        assert "model.layers.1.self_attn.o_proj.weight" in idx.weight_map
        assert not any("zero3" in k for k in idx.weight_map)
        assert torch.allclose(idx.get("model.layers.1.self_attn.o_proj.weight").float(), got_w["layers.1.self_attn.o_proj"], atol=1e-6)


@pytest.mark.parametrize("moe", [False, True])
def test_sharded_layers_train_like_the_replicated_model(moe, tmp_path):
    run_gloo_ranks(_worker, 2, args=(moe, str(tmp_path / "ckpt")), timeout=240.0)


def test_three_ranks_pad_the_layer_to_a_multiple_of_the_world():
    run_gloo_ranks(_worker, 3, args=(False, None), timeout=240.0)


@pytest.mark.parametrize("moe", [False, True])
def test_sharded_layers_under_the_lighter_recomputation_policy(moe):
    """Two of three layers keep the graph of their attention half and re-run only the feed-forward half: the layer's
    parameters are gathered for the first pass, and again from the re-run of the second half until the backward of the
    first; what the attention half saved is read through the parameters bound in that second window."""
    run_gloo_ranks(_worker, 2, args=(moe, None, 2), timeout=240.0)


def _family_worker(rank, world, family, out_dir):
    import dataclasses

    import halo_b200.models.config as config_module
    from tests.test_families_cpu import family_config

    # the training helper builds the "tiny-moe" preset: stand the family's small configuration in its place
    config_module.PRESETS["tiny-moe"] = lambda: dataclasses.replace(family_config(family), vocab_size=256)
    want_l, want_w = _train(rank, world, False, True)
    got_l, got_w = _train(rank, world, True, True, out_dir)
    for a, b in zip(want_l, got_l):
        assert abs(a - b) <= 1e-4 * max(1.0, abs(a)), (want_l, got_l)
    assert set(got_w) == set(want_w), set(got_w) ^ set(want_w)
    for n in want_w:
        assert float((got_w[n] - want_w[n]).abs().max()) < 2e-3, n


@pytest.mark.parametrize("family", ["qwen3_next", "lfm2_moe"])
def test_sharded_layers_of_mixer_families(family, tmp_path):
    """Layers whose mixer is a convolution or a linear-attention block (three-dimensional tap tensors, per-head vectors)
    shard, train, save and reload like attention layers, with the experts cut over the same two ranks."""
    run_gloo_ranks(_family_worker, 2, args=(family, str(tmp_path / "ckpt")), timeout=400.0)
