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

        transport = None
        if mode == "ep_tp":
            # four ranks: tensor-parallel pairs (0, 1) and (2, 3), the experts sharded over all four; both pairs are handed
            # the same row, so the curve is the single process's (every sum and the token normaliser double together)
            from halo_b200.parallel.expert_parallel import CollectiveTransport

            pairs = [dist.new_group([0, 1]), dist.new_group([2, 3])]
            replicas = [dist.new_group([0, 2]), dist.new_group([1, 3])]
            tp = TensorParallel(pairs[rank // 2], "cpu")
            transport = CollectiveTransport(dist.group.WORLD)
            parallel = ParallelRuntime("cpu", dp_group=dist.group.WORLD, ep_group=dist.group.WORLD, transport=transport,
                                       tensor_parallel=tp, tp_replica_group=replicas[rank % 2])
        elif mode == "tp":
            tp = TensorParallel(dist.group.WORLD, "cpu")
        else:
            cp = ContextParallel(dist.group.WORLD, "cpu", cfg, ROW_LEN)
        if parallel is None:
            parallel = ParallelRuntime("cpu", dp_group=dist.group.WORLD, tensor_parallel=tp, context_parallel=cp)
    model = build_model(cfg, device="cpu", dtype=torch.float32, seed=0, gradient_checkpointing=True, tensor_parallel=tp,
                        **({"transport": parallel.transport} if world > 1 and mode == "ep_tp" else {}))
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


@pytest.mark.parametrize("mode", ["tp", "cp", "ep_tp"])
def test_two_ranks_follow_the_single_process_curve(tmp_path, mode):
    single, multi = str(tmp_path / "single.npy"), str(tmp_path / f"{mode}.npy")
    _train(0, 1, mode, single)
    run_gloo_ranks(_train, 4 if mode == "ep_tp" else 2, args=(mode, multi), timeout=300)
    a, b = np.load(single), np.load(multi)
    assert np.max(np.abs(a[0] - b[0])) < 2e-3, (a[0], b[0])          # losses
    assert np.max(np.abs(a[1] - b[1]) / a[1]) < 5e-3, (a[1], b[1])     # global gradient norms (clipping is active)
    assert a[1].min() > 0.5                                           # ... so the clip really scaled the updates


def test_expert_parallel_times_tensor_parallel_through_the_entry_point(tmp_path):
    """``expert_parallel_size: 4`` with ``tensor_parallel_size: 2`` on four CPU ranks through the launcher: two pairs of
    ranks each slice the attention of one row and hold half of its tokens between the blocks, all four shard the experts;
    the loss curve is the one of two expert-parallel ranks that each hold a whole row."""
    import os
    import re
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def run(name, extra, n):
        cfg = tmp_path / f"{name}.yaml"
        cfg.write_text("model_preset: tiny-moe\ninit_from_scratch: true\ndataset_format: synthetic\npacked_row_length: 1024\n"
                       "doc_length_min: 200\ndoc_length_max: 700\n"
                       "max_steps: 5\nlearning_rate: 3.0e-3\nlr_scheduler_type: constant\noptim: adamw_torch\nweight_decay: 0.0\n"
                       f"max_grad_norm: 0.0\noutput_dir: {tmp_path}/{name}\nlogging_steps: 1\n" + extra)
        r = subprocess.run([sys.executable, "-m", "halo_b200.cli", "launch", "sft", str(cfg), "-n", str(n), "--port", "29743"],
                           cwd=root, capture_output=True, text=True, timeout=600,
                           env=dict(os.environ, CUDA_VISIBLE_DEVICES="", NVLINK_DOMAIN_SIZE="4"))
        out = r.stdout + r.stderr
        assert r.returncode == 0, out[-4000:]
        return [float(x) for x in re.findall(r"step \d+ loss ([0-9.]+)", out)], out

    both, out = run("ep4tp2", "expert_parallel_size: 4\ntensor_parallel_size: 2\n", 4)
    assert len(both) >= 5, out[-3000:]
    flat, _ = run("ep2", "expert_parallel_size: 2\n", 2)
    assert abs(both[0] - flat[0]) < 4e-4, (both[:2], flat[:2])
    assert max(abs(a - b) / b for a, b in zip(both[:5], flat[:5])) < 5e-3, (both, flat)
