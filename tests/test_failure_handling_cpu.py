"""Failure handling, injected on the host only: a rank that fails while the others are healthy turns into the same
exception everywhere; an interrupted save is never resumed from; a non-finite gradient norm skips the update and a
streak of them stops the run; bounded waits give up with an error instead of hanging; environment knobs reject
malformed values."""

import os
import time

import pytest
import torch

from halo_b200 import env
from tests.common.gloo import run_gloo_ranks


# ---- raise-everywhere --------------------------------------------------------------------------------
def _one_rank_fails(rank, world):
    import torch.distributed as dist

    from halo_b200.runtime.consensus import DeferredRankFailure, RankFailure, rank_consensus, reject_across_ranks

    guard = DeferredRankFailure()
    with guard.catch():
        if rank == 1:
            raise OSError("No space left on device")          # a local failure inside a collective section
    t = torch.ones(1)
    dist.all_reduce(t)                                         # the failing rank still takes part
    assert int(t.item()) == world
    with pytest.raises(RankFailure, match="rank 1.*No space left"):
        guard.raise_if_any(None, "saving failed")
    with pytest.raises(RankFailure, match="rank 0"):
        reject_across_ranks("bad value" if rank == 0 else None, what="configuration")
    reject_across_ranks(None)                                  # nobody objects: no exception anywhere
    assert rank_consensus(rank == 0, "any") is True and rank_consensus(rank == 0, "all") is False


def test_one_failing_rank_raises_on_every_rank():
    run_gloo_ranks(_one_rank_fails, 2, timeout=60.0)


def _store_phase_times_out(rank, world):
    from datetime import timedelta

    from halo_b200.runtime.consensus import RankFailure, StorePhase, default_store

    ok = StorePhase(default_store(), "everyone-joins", world, rank, timeout=timedelta(seconds=20))
    ok.arrive()
    assert ok.wait_all() == ["ok"] * world
    failed = StorePhase(default_store(), "one-fails", world, rank, timeout=timedelta(seconds=20))
    if rank == 1:
        failed.fail("dataset download failed")
    else:
        failed.arrive()
    with pytest.raises(RankFailure, match="rank 1: dataset download failed"):
        failed.wait_all()                                      # one rank's failure is raised by every rank
    late = StorePhase(default_store(), "never-joined", world, rank, timeout=timedelta(seconds=1))
    if rank == 0:
        late.arrive()
        t0 = time.monotonic()
        with pytest.raises(RankFailure, match="rank 1 never reached"):
            late.wait_all()                                    # rank 1 never arrives: the wait is bounded
        assert time.monotonic() - t0 < 10.0


def test_store_join_is_bounded_when_a_rank_never_arrives():
    run_gloo_ranks(_store_phase_times_out, 2, timeout=60.0)


# ---- interrupted saves, non-finite steps --------------------------------------------------------------
def test_interrupted_save_is_skipped_on_resume(tmp_path):
    from halo_b200.trainers.base import newest_complete_checkpoint

    for step, complete in ((10, True), (20, False)):
        d = tmp_path / f"checkpoint-{step}"
        d.mkdir()
        (d / "model.safetensors").write_bytes(b"x")
        if complete:
            (d / "trainer_state.json").write_text("{}")
    assert newest_complete_checkpoint(str(tmp_path)).endswith("checkpoint-10")


def test_non_finite_gradients_skip_the_update_and_a_streak_stops_the_run(tmp_path):
    import dataclasses

    from halo_b200.configs.arguments import TrainingArguments
    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.config import PRESETS
    from halo_b200.models.qwen3 import build_model
    from halo_b200.trainers.base import NonFiniteRun, Trainer

    cfg = dataclasses.replace(PRESETS["tiny-moe"](), num_hidden_layers=1)
    model = build_model(cfg, device="cpu", dtype=torch.float32, seed=0)
    batches = [synthetic_packed_batch(64, cfg.vocab_size, seed=i, lo=8, hi=32) for i in range(8)]
    args = TrainingArguments(output_dir=str(tmp_path), max_steps=8, optim="adamw_torch", logging_steps=0,
                             max_consecutive_nonfinite_steps=2)

    class Poisoned(Trainer):
        def compute_loss(self, model, batch, normalizer):
            loss = super().compute_loss(model, batch, normalizer)
            return loss * float("nan") if self.global_step >= 1 else loss     # every step after the first is poisoned

    trainer = Poisoned(model, args, batches, device="cpu")
    before = None
    with pytest.raises(NonFiniteRun):
        trainer.train()
    # the healthy first step moved the weights; the poisoned ones did not, and no weight became non-finite
    assert all(torch.isfinite(p).all() for p in model.parameters())
    assert trainer.global_step <= 5 and before is None


# ---- bounded waits and environment knobs ----------------------------------------------------------------
def test_bounded_event_wait_gives_up():
    from halo_b200.runtime.bounded_waits import WaitExpired, bounded_event_wait

    class NeverDone:
        def query(self):
            return False

    t0 = time.monotonic()
    with pytest.raises(WaitExpired, match="weight push"):
        bounded_event_wait(NeverDone(), timeout_seconds=0.2, what="weight push")
    assert time.monotonic() - t0 < 5.0

    class Done:
        def query(self):
            return True

    bounded_event_wait(Done(), timeout_seconds=0.2)


def test_environment_knobs_catalogue(monkeypatch):
    for name in ("DIST_NCCL_TIMEOUT_MINUTES", "HALO_WEIGHT_SYNC_CHUNK_MB", "HALO_EP_CAPACITY_FACTOR"):
        monkeypatch.delenv(name, raising=False)
    assert env.nccl_timeout().total_seconds() == 30 * 60
    assert env.weight_sync_chunk_bytes() == 1024 << 20
    monkeypatch.setenv("DIST_NCCL_TIMEOUT_MINUTES", "5")
    monkeypatch.setenv("HALO_WEIGHT_SYNC_CHUNK_MB", "64")
    assert env.nccl_timeout().total_seconds() == 300 and env.weight_sync_chunk_bytes() == 64 << 20
    # a malformed value never changes behaviour silently: it is reported once and the default is used
    monkeypatch.setenv("HALO_TEST_FLAG", "maybe")
    assert env.env_flag("HALO_TEST_FLAG", default=False) is False
    monkeypatch.setenv("HALO_TEST_INT", "-3")
    assert env.env_positive_int("HALO_TEST_INT", 7) == 7
    monkeypatch.setenv("HALO_TEST_FLAG", "1")
    assert env.env_flag("HALO_TEST_FLAG") is True
    # every knob the package reads is spelled in one of the documented families
    import re

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    names = set()
    for dirpath, _, files in os.walk(os.path.join(root, "halo_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                names |= set(re.findall(r'"((?:HALO|DIST|NVLINK)_[A-Z0-9_]+)"', open(os.path.join(dirpath, f)).read()))
    assert names, "no environment knobs found"
    assert all(n.startswith(("HALO_", "DIST_", "NVLINK_")) for n in names)
