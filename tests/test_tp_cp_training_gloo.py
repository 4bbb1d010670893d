"""Training steps under tensor and context parallelism on two gloo ranks follow the loss curve of a single process:
batch slicing, the global token normaliser, gradient reductions (replicated over all ranks, slices not at all) and
the global gradient norm all have to be right for that."""

import dataclasses

import numpy as np
import pytest
import torch

from halo_b200.data.packing import pack_documents
from halo_b200.models.config import PRESETS
from tests.common.gloo import run_gloo_ranks

STEPS = 6
ROW_LEN = 256


def _row(step: int):
    rng = np.random.default_rng(77 + step)
    docs, left = [], ROW_LEN
    while left > 0:
        n = min(left, int(rng.integers(20, 120)))
        docs.append(rng.integers(0, 4096, size=n))
        left -= n
    return pack_documents(docs)


def _train(rank: int, world: int, mode: str, out_path: str):
    import torch.distributed as dist

    from halo_b200.models.qwen3 import build_model
    from halo_b200.trainers.engine import TrainEngine

    cfg = dataclasses.replace(PRESETS["tiny-moe"](), num_hidden_layers=2)
    parallel = tp = cp = None
    if world > 1:
        from halo_b200.parallel.context_parallel import ContextParallel
        from halo_b200.parallel.runtime import ParallelRuntime
        from halo_b200.parallel.tensor_parallel import TensorParallel

        if mode == "tp":
            tp = TensorParallel(dist.group.WORLD, "cpu")
        else:
            cp = ContextParallel(dist.group.WORLD, "cpu", cfg, ROW_LEN)
        parallel = ParallelRuntime("cpu", dp_group=dist.group.WORLD, tensor_parallel=tp, context_parallel=cp)
    model = build_model(cfg, device="cpu", dtype=torch.float32, seed=0, gradient_checkpointing=True, tensor_parallel=tp)
    model.context_parallel = cp
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4)
    eng = TrainEngine(model, opt, "cpu", max_grad_norm=0.5, parallel=parallel)
    losses, norms = [], []
    for step in range(STEPS):
        out = eng.train_step(_row(step))          # every rank is handed the whole row and keeps its part
        loss = out.loss.reshape(-1)[0].clone()
        if world > 1:
            dist.all_reduce(loss)
        losses.append(float(loss))
        norms.append(float(out.grad_norm))
    if rank == 0:
        np.save(out_path, np.asarray([losses, norms]))


@pytest.mark.parametrize("mode", ["tp", "cp"])
def test_two_ranks_follow_the_single_process_curve(tmp_path, mode):
    single, multi = str(tmp_path / "single.npy"), str(tmp_path / f"{mode}.npy")
    _train(0, 1, mode, single)
    run_gloo_ranks(_train, 2, args=(mode, multi), timeout=300)
    a, b = np.load(single), np.load(multi)
    assert np.max(np.abs(a[0] - b[0])) < 2e-3, (a[0], b[0])          # losses
    assert np.max(np.abs(a[1] - b[1]) / a[1]) < 5e-3, (a[1], b[1])     # global gradient norms (clipping is active)
    assert a[1].min() > 0.5                                           # ... so the clip really scaled the updates
