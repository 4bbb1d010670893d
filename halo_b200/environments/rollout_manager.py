"""Environment episodes against generation servers, played by a pool of worker processes.

``RolloutManager`` owns ``n_workers`` child processes. A worker builds environments from task rows, plays each episode
with an endpoint policy (an OpenAI-compatible chat route, tool calls passed through) and sends back the finished
``EpisodeRecord``. The manager fans a round's tasks over the workers and the server URLs (round-robin), keeps at most
``max_in_flight`` episodes running, gives every episode a deadline that does not count the time generation was paused for
a weight update, retries an episode whose worker died (a sandboxed tool can take its process down) on a fresh worker, and
returns the records in task order - a failed episode as a record with ``done_reason = "failed: ..."`` and score 0, so a
round never loses its shape.

The reference runs the same roles as Ray actors (halo/environments/rollouts/ray_actors.py:210-600: ``EnvironmentActor``,
``RolloutManager``); there is no Ray here, the pool is ``multiprocessing`` (spawn), which is what one box needs.
"""

from __future__ import annotations

import asyncio
import multiprocessing as mp
import queue
import time
import traceback
from dataclasses import dataclass

from .base import EpisodeRecord, Turn


@dataclass
class RolloutConfig:
    env_type: str
    env_options: dict | None = None
    model: str = ""
    max_tokens: int = 1024
    temperature: float = 1.0
    top_p: float = 1.0
    episode_timeout_s: float = 600.0
    turn_timeout_s: float = 300.0
    max_retries: int = 1
    api_key: str = ""


class EnginePauseClock:
    """Seconds generation was paused (weight updates); deadlines are extended by what elapsed while an episode ran."""

    def __init__(self):
        self.total = 0.0
        self._began = None

    def begin(self) -> None:
        self._began = time.monotonic()

    def end(self) -> None:
        if self._began is not None:
            self.total += time.monotonic() - self._began
            self._began = None

    def paused_seconds(self) -> float:
        return self.total + (time.monotonic() - self._began if self._began is not None else 0.0)


def endpoint_policy(url: str, cfg: RolloutConfig, transport=None):
    """``generate(messages, tools) -> Turn`` over ``POST {url}/chat/completions``. ``transport``: an async callable
    ``(url, payload, headers) -> dict`` (tests inject one)."""

    async def generate(messages, tools):
        payload = {"model": cfg.model, "messages": messages, "max_tokens": cfg.max_tokens, "temperature": cfg.temperature,
                   "top_p": cfg.top_p, "logprobs": True}
        if tools:
            payload["tools"] = tools
        headers = {"Authorization": f"Bearer {cfg.api_key}"} if cfg.api_key else {}
        if transport is not None:
            raw = await transport(url.rstrip("/") + "/chat/completions", payload, headers)
        else:
            import aiohttp

            async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=cfg.turn_timeout_s)) as session:
                async with session.post(url.rstrip("/") + "/chat/completions", json=payload, headers=headers) as resp:
                    if resp.status != 200:
                        raise RuntimeError(f"generation server error (status {resp.status}): {(await resp.text())[:300]}")
                    raw = await resp.json()
        msg = raw["choices"][0]["message"]
        lp = (raw["choices"][0].get("logprobs") or {}).get("content") or []
        return Turn("assistant", msg.get("content") or "", msg.get("tool_calls"),
                    [t.get("logprob") for t in lp] or None, None)

    return generate


def _worker_main(worker_id: int, cfg: RolloutConfig, tasks_q, results_q, policy_factory):
    """Child process: play episodes until the sentinel arrives."""
    from .episode_loop import play_episode
    from .registry import make_environment

    loop = asyncio.new_event_loop()
    asyncio.set_event_loop(loop)
    while True:
        item = tasks_q.get()
        if item is None:
            return
        ticket, task, url = item
        try:
            env = make_environment(cfg.env_type, task, **(cfg.env_options or {}))
            generate = policy_factory(url, cfg)
            record = loop.run_until_complete(play_episode(env, generate, None, cfg.turn_timeout_s))
            results_q.put((ticket, worker_id, record, None))
        except BaseException as exc:  # noqa: BLE001 - reported to the manager, the worker lives on
            results_q.put((ticket, worker_id, None, f"{type(exc).__name__}: {exc}\n{traceback.format_exc(limit=3)}"))


class RolloutManager:
    def __init__(self, cfg: RolloutConfig, urls: list[str], n_workers: int = 4, max_in_flight: int = 0, policy_factory=None):
        if not urls:
            raise ValueError("the rollout manager needs at least one generation server URL")
        self.cfg, self.urls = cfg, list(urls)
        self.n_workers = n_workers
        self.max_in_flight = max_in_flight or 4 * n_workers
        self.policy_factory = policy_factory or endpoint_policy
        self.clock = EnginePauseClock()
        self._ctx = mp.get_context("spawn")
        self._results = self._ctx.Queue()
        self._workers: dict[int, tuple] = {}
        self._next_worker_id = 0
        self._next_url = 0
        self.failures: list[str] = []
        for _ in range(n_workers):
            self._spawn()

    # ---- workers ---------------------------------------------------------------------------------------
    def _spawn(self) -> int:
        wid = self._next_worker_id
        self._next_worker_id += 1
        q = self._ctx.Queue()
        proc = self._ctx.Process(target=_worker_main, args=(wid, self.cfg, q, self._results, self.policy_factory), daemon=True)
        proc.start()
        self._workers[wid] = (proc, q)
        return wid

    def _least_loaded(self, load: dict) -> int:
        return min(self._workers, key=lambda w: load.get(w, 0))

    def begin_engine_pause(self) -> None:
        self.clock.begin()

    def end_engine_pause(self) -> None:
        self.clock.end()

    # ---- one round -------------------------------------------------------------------------------------
    def play(self, tasks: list[dict]) -> list[EpisodeRecord]:
        """Play one episode per task; records come back in task order."""
        records: list[EpisodeRecord | None] = [None] * len(tasks)
        attempts = [0] * len(tasks)
        pending = list(range(len(tasks)))
        running: dict[int, tuple] = {}            # ticket -> (task index, worker id, deadline base, paused at start)
        load: dict[int, int] = {}
        ticket = 0

        def fail(i: int, why: str) -> None:
            rec = EpisodeRecord()
            rec.done_reason, rec.score = f"failed: {why.splitlines()[0][:200]}", 0.0
            records[i] = rec
            self.failures.append(why)

        def submit(i: int) -> None:
            nonlocal ticket
            wid = self._least_loaded(load)
            url = self.urls[self._next_url % len(self.urls)]
            self._next_url += 1
            self._workers[wid][1].put((ticket, tasks[i], url))
            running[ticket] = (i, wid, time.monotonic(), self.clock.paused_seconds())
            load[wid] = load.get(wid, 0) + 1
            attempts[i] += 1
            ticket += 1

        while pending or running:
            while pending and len(running) < self.max_in_flight:
                submit(pending.pop(0))
            try:
                t, wid, record, error = self._results.get(timeout=0.2)
            except queue.Empty:
                t = None
            if t is not None and t in running:
                i, wid, _, _ = running.pop(t)
                load[wid] -= 1
                if error is None:
                    records[i] = record
                elif attempts[i] <= self.cfg.max_retries:
                    pending.append(i)
                else:
                    fail(i, error)
            # deadlines (generation pauses do not count) and dead workers
            now = time.monotonic()
            for t2, (i, wid, began, paused0) in list(running.items()):
                if t2 not in running:
                    continue                      # re-queued a moment ago with the rest of a replaced worker's episodes
                proc = self._workers[wid][0] if wid in self._workers else None
                dead = proc is None or not proc.is_alive()
                late = (now - began) - (self.clock.paused_seconds() - paused0) > self.cfg.episode_timeout_s
                if not dead and not late:
                    continue
                running.pop(t2)
                if wid in self._workers:
                    # a worker that died or sits on an overdue episode is replaced; its other episodes are re-queued
                    proc.kill()
                    proc.join(5)
                    del self._workers[wid]
                    load.pop(wid, None)
                    for t3, (j, w3, *_r) in list(running.items()):
                        if w3 == wid:
                            running.pop(t3)
                            pending.append(j)
                            attempts[j] -= 1
                    self._spawn()
                if dead and attempts[i] <= self.cfg.max_retries:
                    pending.append(i)
                else:
                    fail(i, "worker died" if dead else f"episode exceeded {self.cfg.episode_timeout_s:g} s")
        return records  # type: ignore[return-value]

    def close(self) -> None:
        for proc, q in self._workers.values():
            try:
                q.put(None)
            except Exception:  # noqa: BLE001
                pass
        for proc, _ in self._workers.values():
            proc.join(5)
            if proc.is_alive():
                proc.kill()
        self._workers.clear()
