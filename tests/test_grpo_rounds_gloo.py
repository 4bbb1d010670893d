"""GRPO rounds on two gloo ranks whose row counts differ: the rank with fewer rows than the world has micro-steps must
still enter every collective of the round (it runs filler micro-batches that score nothing), both ranks take exactly
one optimizer step per round, end with identical weights, and the result equals a single process that trains on the
union of the two ranks' rollouts: the round denominator is global, so neither the cut into micro-batches nor the
data-parallel width changes the update."""

import dataclasses

import numpy as np
import torch

from halo_b200.models.config import PRESETS
from tests.common.gloo import run_gloo_ranks

ROUNDS = 3


def _rollouts(round_index: int, rank: int, world: int):
    """Rank 0 of two holds 8 rows (several micro-batches at the budget below), rank 1 holds 4 short ones (one)."""
    from halo_b200.trainers.grpo.trainer import Rollout

    rng = np.random.default_rng(1000 * round_index + 17)
    rows = []
    for g in range(3):                                # three groups of four
        prompt = rng.integers(0, 512, size=int(rng.integers(4, 8)))
        for _ in range(4):
            n = int(rng.integers(10, 16)) if g < 2 else int(rng.integers(3, 5))
            comp = rng.integers(0, 512, size=n)
            rows.append(Rollout(prompt, comp, (-rng.random(n) - 0.05).astype(np.float32), float(rng.normal())))
    if world == 1:
        return rows
    return rows[:8] if rank == 0 else rows[8:]


def _train(rank: int, world: int, out_path: str, loss_type: str):
    import torch.distributed as dist

    from halo_b200.configs.arguments import GRPOArguments, TrainingArguments
    from halo_b200.models.qwen3 import build_model
    from halo_b200.trainers.grpo.trainer import GRPOTrainer

    cfg = dataclasses.replace(PRESETS["tiny-moe"](), num_hidden_layers=2, vocab_size=512)
    model = build_model(cfg, device="cpu", dtype=torch.float32, seed=0)
    parallel = None
    if world > 1:
        from halo_b200.parallel.runtime import ParallelRuntime

        parallel = ParallelRuntime("cpu", dp_group=dist.group.WORLD)
    micro_steps = []
    args = TrainingArguments(output_dir="unused", learning_rate=1e-3, optim="adamw_torch", logging_steps=1, max_grad_norm=0.0)
    t = GRPOTrainer(model, args, lambda i: _rollouts(i, rank, world) if i < ROUNDS else None, device="cpu", parallel=parallel,
                    grpo_args=GRPOArguments(num_generations=4, token_budget=26, loss_type=loss_type, max_completion_length=16,
                                            is_geo_band_min=0.01, is_geo_band_max=100.0, is_veto_min=1e-9, opsm_delta=50.0))
    orig = t.engine.train_step

    def counting(batch, accumulate=False):
        micro_steps.append(batch.n_scored)
        return orig(batch, accumulate=accumulate)

    t.engine.train_step = counting
    out = t.train()
    assert out["global_step"] == ROUNDS, out["global_step"]
    if world > 1:
        n = torch.tensor([len(micro_steps)])
        lo, hi = n.clone(), n.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        assert int(lo) == int(hi), (int(lo), int(hi))             # every rank ran the same number of micro-steps
        if rank == 1:
            assert 0 in micro_steps                               # ... and the short rank filled slots with fillers
        for p in model.parameters():
            ref = p.detach().clone()
            dist.broadcast(ref, 0)
            assert torch.equal(ref, p.detach())
    if rank == 0:
        torch.save({n: p.detach().clone() for n, p in model.named_parameters()}, out_path)


def test_unequal_ranks_run_equal_micro_steps_and_match_one_process(tmp_path):
    for loss_type in ("dapo", "grpo"):
        single, multi = str(tmp_path / f"s_{loss_type}.pt"), str(tmp_path / f"m_{loss_type}.pt")
        _train(0, 1, single, loss_type)
        run_gloo_ranks(_train, 2, args=(multi, loss_type), timeout=300)
        a, b = torch.load(single), torch.load(multi)
        for n in a:
            assert torch.allclose(a[n], b[n], atol=3e-5), (loss_type, n, (a[n] - b[n]).abs().max())
