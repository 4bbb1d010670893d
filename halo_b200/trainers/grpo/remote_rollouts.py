"""Rollouts generated on the job's rollout ranks and handed to the trainers through the rendezvous store.

A rollout rank holds the serving copy of the policy. Before the first optimizer step and after every weight push
it samples the next round(s) for the trainer ranks it serves and publishes each as one pickled blob under
``halo/rollouts/<trainer rank>/<round>``; a trainer's :class:`StoreRolloutSource` waits for its key with a
deadline, reads it and deletes it. ``prefetch = 0`` is strictly on-policy (round ``k`` is sampled after update
``k``, the trainers wait while it is sampled); ``prefetch = 1`` samples round ``k + 1`` while the trainers work on
round ``k``, one update stale - the sampler's log-probabilities travel with the rollouts, so the objective's
importance weights account for it.

Control stays where it was: the trainers' push announcement drives the rollout ranks' loop, so no extra thread or
collective is needed. The role of the reference's asynchronous rollout workers
(halo/trainers/grpo/environmental/async_rollouts.py:88-695), without Ray: both sides are ranks of one launcher.
"""

from __future__ import annotations

import pickle
import time

import numpy as np

from halo_b200 import env
from halo_b200.trainers.grpo.trainer import Rollout

KEY = "halo/rollouts/{trainer}/{round}"
END = b"__end__"


def served_trainers(rollout_index: int, n_rollout: int, n_trainers: int) -> list[int]:
    """Trainer ranks whose rounds rollout rank ``rollout_index`` (0-based among the rollout ranks) samples."""
    return [t for t in range(n_trainers) if t % n_rollout == rollout_index]


class RolloutPublisher:
    """Rollout-rank side. ``make_source(trainer_rank)`` builds the on-policy source for one trainer rank."""

    def __init__(self, store, trainers: list[int], make_source, prefetch: int = 0):
        self.store, self.trainers, self.prefetch = store, trainers, max(0, prefetch)
        self.sources = {t: make_source(t) for t in trainers}
        self.next_round = 0
        self.exhausted = False

    def _publish_round(self, version: int) -> None:
        for t in self.trainers:
            rollouts = self.sources[t](self.next_round)
            key = KEY.format(trainer=t, round=self.next_round)
            if rollouts is None:
                self.store.set(key, END)
                self.exhausted = True
                continue
            blob = [(r.prompt_ids, r.completion_ids, r.sampler_logprobs, r.reward, r.completion_mask, r.routing, r.routing_layers)
                    for r in rollouts]
            self.store.set(key, pickle.dumps({"version": version, "rollouts": blob, "mean_reward": self.sources[t].mean_reward}))
        self.next_round += 1

    def start(self) -> None:
        """Rounds sampled with the initial weights: round 0, plus ``prefetch`` rounds ahead."""
        for _ in range(1 + self.prefetch):
            self._publish_round(0)

    def on_update(self, n_updates: int) -> None:
        """Called after the ``n_updates``-th weight push has landed in the serving copy."""
        if not self.exhausted:
            self._publish_round(n_updates)


class StoreRolloutSource:
    """Trainer-rank side: what :class:`halo_b200.trainers.grpo.trainer.GRPOTrainer` calls for each round."""

    def __init__(self, store, trainer_rank: int, timeout_seconds: float | None = None, poll_seconds: float = 0.02):
        self.store, self.rank, self.poll = store, trainer_rank, poll_seconds
        self.timeout = timeout_seconds if timeout_seconds is not None else float(env.env_positive_int("HALO_ROLLOUT_WAIT_SECONDS", 1800))
        self.last_version, self.mean_reward, self.waited_seconds = -1, float("nan"), 0.0

    def __call__(self, round_index: int):
        key = KEY.format(trainer=self.rank, round=round_index)
        t0 = time.monotonic()
        while True:
            try:
                if self.store.check([key]):
                    break
            except RuntimeError:
                pass
            if time.monotonic() - t0 > self.timeout:
                raise TimeoutError(f"round {round_index} for trainer rank {self.rank} did not arrive within {self.timeout:.0f} s: "
                                   f"the rollout rank serving it is gone or stuck")
            time.sleep(self.poll)
        self.waited_seconds += time.monotonic() - t0
        blob = self.store.get(key)
        try:
            self.store.delete_key(key)
        except (RuntimeError, NotImplementedError):
            pass
        if blob == END:
            return None
        msg = pickle.loads(blob)
        self.last_version, self.mean_reward = msg["version"], msg["mean_reward"]
        return [Rollout(np.asarray(p), np.asarray(c), None if lp is None else np.asarray(lp, dtype=np.float32), float(r), mask, routing, layers)
                for p, c, lp, r, mask, routing, layers in msg["rollouts"]]
