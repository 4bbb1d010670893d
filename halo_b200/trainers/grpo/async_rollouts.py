"""Rollouts produced ahead of the trainer by a background thread (halo/trainers/grpo/environmental/
async_rollouts.py:88-695): the producer calls ``generate(round_index, policy_version)``, the trainer takes rounds
in order; a round generated with weights older than ``max_staleness`` optimizer steps is discarded and produced
again, and the producer pauses while a weight push is in flight."""

from __future__ import annotations

import queue
import threading


class AsyncRolloutSource:
    def __init__(self, generate, prefetch: int = 1, max_staleness: int = 1):
        self.generate, self.max_staleness = generate, max_staleness
        self.q: queue.Queue = queue.Queue(maxsize=max(1, prefetch))
        self.version = 0                     # optimizer steps whose weights the rollout side has received
        self._next_round = 0
        self._pause = threading.Event()
        self._pause.set()
        self._stop = threading.Event()
        self._error: BaseException | None = None
        self.discarded = 0
        self._thread = threading.Thread(target=self._produce, daemon=True)
        self._thread.start()

    def _produce(self) -> None:
        try:
            while not self._stop.is_set():
                self._pause.wait()
                i, v = self._next_round, self.version
                rollouts = self.generate(i, v)
                if rollouts is None:
                    self.q.put((i, v, None))
                    return
                self._next_round += 1
                while not self._stop.is_set():
                    try:
                        self.q.put((i, v, rollouts), timeout=0.1)
                        break
                    except queue.Full:
                        continue
        except BaseException as exc:  # noqa: BLE001 - surfaced to the trainer thread
            self._error = exc
            self.q.put((-1, -1, None))

    def __call__(self, round_index: int):
        """What :class:`GRPOTrainer` calls for the next round; blocks until a fresh enough round is ready."""
        while True:
            i, v, rollouts = self.q.get()
            if self._error is not None:
                raise RuntimeError("the rollout producer failed") from self._error
            if rollouts is None:
                return None
            if self.version - v > self.max_staleness:
                self.discarded += 1           # generated with weights that are too old: produce it again
                self._next_round = min(self._next_round, i)
                continue
            return rollouts

    # ---- weight pushes -------------------------------------------------------------------------
    def pause(self) -> None:
        self._pause.clear()

    def resume(self, new_version: int) -> None:
        self.version = new_version
        self._pause.set()

    def close(self) -> None:
        self._stop.set()
        self._pause.set()
        self._thread.join(timeout=5.0)
