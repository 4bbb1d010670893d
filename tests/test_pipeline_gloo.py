"""Pipeline parallelism on two gloo ranks: the 1F1B and GPipe schedules give the loss and the gradients of the
unsplit model, micro-batch for micro-batch."""

import pytest
import torch

from halo_b200.parallel.pipeline import partition_layers
from tests.common.gloo import run_gloo_ranks


def test_partition_balances_head_cost():
    assert partition_layers(8, 2, head_weight=2.0) == [(0, 5), (5, 8)]
    assert partition_layers(48, 4, head_weight=0.0) == [(0, 12), (12, 24), (24, 36), (36, 48)]
    assert partition_layers(6, 3, split=[1, 3]) == [(0, 1), (1, 3), (3, 6)]
    with pytest.raises(ValueError):
        partition_layers(2, 3)
    with pytest.raises(ValueError):
        partition_layers(6, 3, split=[3, 3])
    ranges = partition_layers(48, 8, head_weight=3.0)
    assert ranges[0][0] == 0 and ranges[-1][1] == 48 and all(b > a for a, b in ranges)
    assert ranges[-1][1] - ranges[-1][0] < ranges[0][1] - ranges[0][0]


def _worker(rank, world, schedule, family="tiny-moe"):
    import dataclasses

    import torch.distributed as dist

    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.config import PRESETS
    from halo_b200.models.qwen3 import build_model
    from halo_b200.parallel.pipeline import PipelineStage, broadcast_loss, build_stage_model, run_schedule

    if family == "tiny-moe":
        cfg = dataclasses.replace(PRESETS["tiny-moe"](), num_hidden_layers=4)
    else:
        # a family whose layers differ by their GLOBAL index (windowed / full mix) and whose loss is soft-capped
        from tests.test_families_cpu import family_config

        cfg = family_config(family, num_hidden_layers=4, tie_word_embeddings=False,
                            layer_types=["sliding_attention", "sliding_attention", "full_attention", "sliding_attention"])
    row = 96
    micro = [synthetic_packed_batch(row, cfg.vocab_size, seed=i, lo=8, hi=48) for i in range(3)]
    norm = float(sum(b.n_scored for b in micro))
    stage_model = build_stage_model(cfg, rank, world, "cpu", dtype=torch.float32, seed=5, split=[2])
    stage = PipelineStage(stage_model, dist.group.WORLD, row)
    loss = broadcast_loss(stage, run_schedule(stage, micro, norm, schedule))

    full = build_model(cfg, device="cpu", dtype=torch.float32, seed=5)
    ref = sum(full(b.input_ids, b.position_ids, b.cu_seqlens, b.labels, norm) for b in micro)
    ref.backward()
    assert torch.allclose(loss, ref.detach(), rtol=1e-5, atol=1e-6), (float(loss), float(ref))
    lo = stage_model.layer_range[0]
    full_params = dict(full.named_parameters())
    checked = 0
    for name, p in stage_model.named_parameters():
        if name.startswith("layers."):
            _, li, rest = name.split(".", 2)
            name = f"layers.{int(li) + lo}.{rest}"
        q = full_params[name]
        assert torch.equal(p.detach(), q.detach()), name              # same initial weights as the unsplit model
        assert torch.allclose(p.grad, q.grad, rtol=1e-4, atol=1e-6), name
        checked += 1
    assert checked > 5


@pytest.mark.parametrize("schedule", ["1f1b", "gpipe"])
def test_pipeline_matches_unsplit_model(schedule):
    run_gloo_ranks(_worker, 2, args=(schedule,), timeout=90.0)


def test_pipeline_stages_keep_each_layers_own_attention_kind():
    run_gloo_ranks(_worker, 2, args=("1f1b", "gemma2"), timeout=120.0)


def _train_worker(rank, world, out_path):
    import dataclasses

    import numpy as np
    import torch.distributed as dist

    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.config import PRESETS
    from halo_b200.models.qwen3 import build_model
    from halo_b200.parallel.pipeline import PipelineStage, build_stage_model
    from halo_b200.trainers.engine import TrainEngine
    from halo_b200.trainers.pipeline_engine import PipelineEngine

    cfg = dataclasses.replace(PRESETS["tiny-moe"](), num_hidden_layers=4)
    row, steps, n_micro = 96, 4, 3
    batches = [[synthetic_packed_batch(row, cfg.vocab_size, seed=10 * s + i, lo=8, hi=48) for i in range(n_micro)]
               for s in range(steps)]
    if world > 1:
        model = build_stage_model(cfg, rank, world, "cpu", dtype=torch.float32, seed=9, split=[2])
        eng = PipelineEngine(PipelineStage(model, dist.group.WORLD, row), torch.optim.AdamW(model.parameters(), lr=3e-4),
                             max_grad_norm=0.5)
        curve = []
        for mb in batches:
            o = eng.train_step(mb)
            curve.append([float(o.loss), float(o.grad_norm)])     # read now: the norm tensor is reused every step
    else:
        model = build_model(cfg, device="cpu", dtype=torch.float32, seed=9)
        eng = TrainEngine(model, torch.optim.AdamW(model.parameters(), lr=3e-4), "cpu", max_grad_norm=0.5)
        curve = []
        for mb in batches:
            norm = float(sum(b.n_scored for b in mb))
            eng.global_scored_tokens = lambda batch, norm=norm: norm      # one normaliser for the whole step
            total = 0.0
            for i, b in enumerate(mb):
                o = eng.train_step(b, accumulate=i < len(mb) - 1)
                total += float(o.loss)
            curve.append([total, float(o.grad_norm)])
    if rank == 0:
        np.save(out_path, np.asarray(curve))


def test_pipeline_training_follows_the_single_process_curve(tmp_path):
    import numpy as np

    single, pp = str(tmp_path / "single.npy"), str(tmp_path / "pp.npy")
    _train_worker(0, 1, single)
    run_gloo_ranks(_train_worker, 2, args=(pp,), timeout=180.0)
    a, b = np.load(single), np.load(pp)
    assert np.max(np.abs(a[:, 0] - b[:, 0])) < 2e-3, (a, b)
    assert np.max(np.abs(a[:, 1] - b[:, 1]) / a[:, 1]) < 5e-3, (a, b)


def _save_worker(rank, world, directory):
    import dataclasses

    import torch.distributed as dist

    from halo_b200.checkpoint.load import from_pretrained, load_model_weights
    from halo_b200.checkpoint.save import save_pipeline_stages
    from halo_b200.models.config import PRESETS
    from halo_b200.models.qwen3 import build_model
    from halo_b200.parallel.pipeline import build_stage_model

    cfg = dataclasses.replace(PRESETS["tiny-moe"](), num_hidden_layers=4)
    stage_model = build_stage_model(cfg, rank, world, "cpu", dtype=torch.float32, seed=5, split=[2])
    save_pipeline_stages(stage_model, directory, rank, world, save_dtype=None, max_shard_bytes=2 << 20)
    dist.barrier()
    # the merged directory is an ordinary checkpoint: the whole model loads from it and equals the unsplit build ...
    whole = from_pretrained(directory, device="cpu", dtype=torch.float32)
    want = build_model(cfg, device="cpu", dtype=torch.float32, seed=5)
    for (n, a), (_, b) in zip(whole.named_parameters(), want.named_parameters()):
        assert torch.equal(a, b), n
    # ... and a stage reads only its own layers back
    again = build_stage_model(cfg, rank, world, "cpu", dtype=torch.float32, seed=99, split=[2])
    load_model_weights(again, directory)
    for (n, a), (_, b) in zip(again.named_parameters(), stage_model.named_parameters()):
        assert torch.equal(a, b), n


def test_stages_save_one_ordinary_checkpoint(tmp_path):
    import json
    import os

    d = str(tmp_path / "ckpt")
    run_gloo_ranks(_save_worker, 2, args=(d,), timeout=120.0)
    index = json.load(open(os.path.join(d, "model.safetensors.index.json")))
    files = set(index["weight_map"].values())
    assert any(f.startswith("model-stage000-") for f in files) and any(f.startswith("model-stage001-") for f in files)
    assert all(os.path.isfile(os.path.join(d, f)) for f in files) and os.path.isfile(os.path.join(d, "config.json"))


def test_pipeline_times_expert_parallel_through_the_entry_point(tmp_path):
    """``pipeline_parallel_size: 2`` with ``expert_parallel_size: 2`` on four CPU ranks through the launcher (the layout
    of the 8-GPU PP2 x EP4 runs, halved): stages load only their layers, the step runs the 1F1B schedule over the
    step's micro-batches, the two replicas of a stage shard the experts, and the loss goes down as in a single process."""
    import os
    import re
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def run(name, extra, n):
        cfg = tmp_path / f"{name}.yaml"
        cfg.write_text("model_preset: tiny-moe\ninit_from_scratch: true\ndataset_format: synthetic\npacked_row_length: 128\n"
                       "max_steps: 6\nlearning_rate: 3.0e-3\nlr_scheduler_type: constant\noptim: adamw_torch\nweight_decay: 0.0\n"
                       f"gradient_accumulation_steps: 2\noutput_dir: {tmp_path}/{name}\nlogging_steps: 1\n" + extra)
        r = subprocess.run([sys.executable, "-m", "halo_b200.cli", "launch", "sft", str(cfg), "-n", str(n), "--port", "29731"],
                           cwd=root, capture_output=True, text=True, timeout=600,
                           env=dict(os.environ, CUDA_VISIBLE_DEVICES="", NVLINK_DOMAIN_SIZE="2"))
        out = r.stdout + r.stderr
        assert r.returncode == 0, out[-4000:]
        return [float(x) for x in re.findall(r"step \d+ loss ([0-9.]+)", out)], out

    pp, out = run("pp2ep2", "pipeline_parallel_size: 2\nexpert_parallel_size: 2\nmax_grad_norm: 0.0\n", 4)
    assert len(pp) >= 6, out[-3000:]
    assert "pipeline stage 0 of 2" in out and "pipeline stage 1 of 2" in out
    flat, out2 = run("ep2", "expert_parallel_size: 2\nmax_grad_norm: 0.0\n", 2)
    # the same two data-parallel replicas, the same rows and the same initialisation with and without the pipeline:
    # the first step's loss is the same number, the curves stay together (the optimizer sees the same gradients up to
    # one common factor, which Adam divides out)
    assert abs(pp[0] - flat[0]) < 4e-4, (pp[:2], flat[:2])
    assert max(abs(a - b) / b for a, b in zip(pp[::2][:6], flat[::2][:6])) < 5e-3, (pp, flat)
    # the stages wrote one ordinary checkpoint: every tensor of the unsplit model, experts gathered
    import json

    idx = json.load(open(tmp_path / "pp2ep2" / "final" / "model.safetensors.index.json"))["weight_map"]
    ref = json.load(open(tmp_path / "ep2" / "final" / "model.safetensors.index.json"))["weight_map"] \
        if os.path.isfile(tmp_path / "ep2" / "final" / "model.safetensors.index.json") else None
    assert any(k.startswith("model.embed_tokens") for k in idx) and any(k.startswith("lm_head") or k.startswith("model.norm") for k in idx)
    if ref is not None:
        assert set(idx) == set(ref)
