"""Chunk planning / packing of the weight sync and the gloo broadcast path (CPU)."""

import torch

from halo_b200.weight_sync.chunking import manifest_of, pack_chunk, plan_chunks, unpack_chunk
from tests.common.gloo import run_gloo_ranks


def test_chunk_plan_round_trip():
    tensors = {"a": torch.randn(100, 7).bfloat16(), "b": torch.randn(33), "c": torch.arange(1000, dtype=torch.int32)}
    slots, sizes = plan_chunks(manifest_of(tensors.items()), chunk_bytes=2048)
    assert len(sizes) >= 2 and all(s.offset % 256 == 0 for s in slots)
    out = {k: torch.zeros_like(v) for k, v in tensors.items()}
    for c, size in enumerate(sizes):
        buf = torch.zeros(size, dtype=torch.uint8)
        pack_chunk(slots, c, tensors, buf)
        unpack_chunk(slots, c, buf, out)
    for k in tensors:
        assert torch.equal(out[k], tensors[k])


def _worker(rank, world):
    import torch.distributed as dist

    from halo_b200.weight_sync.group import BroadcastSync

    torch.manual_seed(0)
    src = {"w1": torch.randn(64, 64), "w2": torch.randn(1000)}
    sync = BroadcastSync(dist.group.WORLD, "cpu", manifest_of(src.items()), src_rank=0, chunk_bytes=4096)
    if rank == 0:
        sync.push(src)
    else:
        dst = {k: torch.zeros_like(v) for k, v in src.items()}
        sync.push(None, into=dst)
        for k in src:
            assert torch.equal(dst[k], src[k])


def test_broadcast_sync_over_gloo():
    run_gloo_ranks(_worker, 2)


def _split_worker(rank, world):
    """Two expert-parallel trainer ranks and one rollout rank: after a push the rollout rank's unsharded
    serving copy equals the trainers' gathered weights, tensor for tensor."""
    import torch.distributed as dist

    from halo_b200.models.config import PRESETS
    from halo_b200.models.qwen3 import build_model
    from halo_b200.parallel.expert_parallel import CollectiveTransport
    from halo_b200.weight_sync.group import build_manifest, full_manifest, full_named_tensors
    from halo_b200.weight_sync.roles import ModelWeightPusher, make_sync, rollout_loop, split_roles

    roles = split_roles(1)
    cfg = PRESETS["tiny-moe"]()
    if roles.is_trainer:
        torch.manual_seed(1)
        model = build_model(cfg, device="cpu", dtype=torch.float32, transport=CollectiveTransport(roles.trainer_group))
        with torch.no_grad():
            for p in model.parameters():
                p.add_(0.25)                      # the trainers moved away from the initial weights
        sync = make_sync(roles, "cpu", full_manifest(model), chunk_bytes=1 << 16)
        pusher = ModelWeightPusher(sync, roles, "cpu", roles.trainer_group)
        pusher.push(model)
        want = dict(full_named_tensors(model, roles.trainer_group))
        pusher.close()
        if rank == roles.src_rank:
            dist.send(torch.stack([t.double().sum() for t in want.values()]), dst=roles.rollout_ranks[0])
    else:
        torch.manual_seed(1)
        serving = build_model(cfg, device="cpu", dtype=torch.float32, transport=None)
        params = dict(serving.named_parameters())
        sync = make_sync(roles, "cpu", build_manifest(serving), chunk_bytes=1 << 16)
        assert rollout_loop(sync, roles, "cpu", params) == 1
        sums = torch.zeros(len(params), dtype=torch.float64)
        dist.recv(sums, src=roles.src_rank)
        got = torch.stack([p.detach().double().sum() for p in params.values()])
        assert torch.allclose(got, sums, rtol=0, atol=1e-9)


def test_split_roles_push_reaches_the_rollout_copy():
    run_gloo_ranks(_split_worker, 3)


def test_one_trainer_one_rollout_job_finishes(tmp_path):
    """A split job whose trainer side is a single rank: saves and barriers must involve the trainer alone (the
    rollout rank sits in its receive loop), and closing the pusher ends the rollout rank."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = tmp_path / "grpo.yaml"
    cfg.write_text("model_preset: tiny-moe\ninit_from_scratch: true\nmax_steps: 2\noptim: adamw_torch\n"
                   f"output_dir: {tmp_path}/run\nnum_generations: 4\ntoken_budget: 2048\nmax_completion_length: 64\n"
                   "rollout_gpus: 1\n")
    r = subprocess.run([sys.executable, "-m", "halo_b200.cli", "launch", "grpo", str(cfg), "-n", "2", "--port", "29683"],
                       cwd=root, capture_output=True, text=True, timeout=240, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert os.path.isfile(tmp_path / "run" / "final" / "config.json")


def test_push_parity_compares_fixed_row_scores():
    import numpy as np
    import pytest

    from halo_b200.models.config import tiny_moe_config
    from halo_b200.models.qwen3 import build_model
    from halo_b200.weight_sync import parity

    class Store(dict):
        def set(self, k, v):
            self[k] = v

        def check(self, keys):
            return all(k in self for k in keys)

        def get(self, k):
            return self[k]

    trainer = build_model(tiny_moe_config(), device="cpu", seed=0, gradient_checkpointing=False)
    copy = build_model(tiny_moe_config(), device="cpu", seed=0, gradient_checkpointing=False)
    store = Store()
    parity.publish(store, parity.score_fixed_row(copy, "cpu"))
    mine = parity.score_fixed_row(trainer, "cpu")
    assert mine.shape == (94,) and parity.compare(store, mine, 0.05, 1.0) < 1e-6
    with torch.no_grad():
        copy.layers[1].self_attn.o_proj.mul_(1.5)                 # a tensor that did not arrive intact
    parity.publish(store, parity.score_fixed_row(copy, "cpu"))
    with pytest.raises(RuntimeError, match="push parity failed"):
        parity.compare(store, mine, 0.05, 1.0)
    with pytest.raises(TimeoutError):
        parity.compare(Store(), mine, 0.05, 0.1)
