"""Trainer side of a weight push into an external generation server, and rollouts sampled from that server.

``EngineWeightPusher`` has the interface the GRPO trainer expects from a weight pusher (``push(model)`` after an
optimizer step, ``close()`` at the end). Every trainer takes part in gathering the expert banks (a collective over the
expert-parallel group); the forwarding rank converts each tensor to its hub names as it arrives and streams it to the
server a few hundred megabytes at a time, so no rank ever holds a second full copy of the model.

``ServerRolloutSource`` asks the server's OpenAI-compatible completion route for ``num_generations`` samples per
prompt with the sampled tokens' log-probabilities, and hands the trainer ``Rollout`` records.

Counterpart of halo/trainers/grpo/rollout/weight_push.py and halo/weight_sync/update_stream.py:1-187.
"""

from __future__ import annotations

import concurrent.futures as cf

import numpy as np
import torch
import torch.distributed as dist

from halo_b200.checkpoint.hub_layout import runtime_to_hub
from halo_b200.weight_sync.group import full_named_tensors


class EngineWeightPusher:
    def __init__(self, client, device, ep_group=None, trainer_group=None, src_rank: int = 0, batch_bytes: int = 512 << 20):
        self.client, self.device = client, torch.device(device)
        self.ep_group, self.trainer_group, self.src_rank = ep_group, trainer_group, src_rank
        self.batch_bytes = batch_bytes
        self.pushes = 0
        initialized = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank(trainer_group) if initialized else 0
        self.parity_tolerance = 0.0
        self.parity_gap = None

    def _agree(self, ok: bool, what: str) -> None:
        """Every trainer learns whether the forwarding rank's step worked before any of them goes on."""
        if not (dist.is_available() and dist.is_initialized()):
            if not ok:
                raise RuntimeError(what)
            return
        flag = torch.tensor([0 if ok else 1], device=self.device if self.device.type == "cuda" else "cpu")
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.trainer_group)
        if int(flag.item()):
            raise RuntimeError(what)

    def push(self, model) -> None:
        sender = self.rank == self.src_rank
        error = None
        try:
            if sender:
                self.client.begin_update(self.device)
        except Exception as exc:  # noqa: BLE001 - reported on every rank below
            error = exc
        self._agree(error is None, f"the generation server did not open a weight update: {error}")
        pending, pending_bytes = {}, 0
        for name, t in full_named_tensors(model, self.ep_group):        # collective: every trainer walks the same list
            if not sender or error is not None:
                continue
            try:
                for hub_name, hub_t in runtime_to_hub(name, t, model.cfg).items():
                    pending[hub_name] = hub_t
                    pending_bytes += hub_t.numel() * hub_t.element_size()
                if pending_bytes >= self.batch_bytes:
                    self.client.send_tensors(pending)
                    pending, pending_bytes = {}, 0
            except Exception as exc:  # noqa: BLE001
                error = exc
        if sender and error is None:
            try:
                self.client.send_tensors(pending)
                self.client.end_update()
            except Exception as exc:  # noqa: BLE001
                error = exc
        self._agree(error is None, f"the weight push to the generation server failed: {error}")
        self.pushes += 1

    def close(self) -> None:
        if self.rank == self.src_rank:
            self.client.close()


class ServerRolloutSource:
    """``source(round_index) -> list[Rollout]`` sampled from a served copy of the policy."""

    def __init__(self, url: str, model_id: str, prompts, reward_fn, num_generations: int, max_new_tokens: int, temperature: float = 1.0,
                 top_p: float = 1.0, top_k: int = 0, prompts_per_round: int = 8, max_prompt_length: int = 0, concurrency: int = 16,
                 session=None, timeout_s: float = 1800.0):
        if not len(prompts):
            raise ValueError("server rollouts need at least one prompt")
        self.url, self.model_id = url.rstrip("/"), model_id
        self.prompts, self.reward_fn = prompts, reward_fn
        self.g, self.max_new, self.temperature, self.top_p, self.top_k = num_generations, max_new_tokens, temperature, top_p, top_k
        self.per_round, self.max_prompt, self.concurrency = prompts_per_round, max_prompt_length, concurrency
        self._session, self.timeout_s = session, timeout_s
        self.mean_reward = float("nan")

    def _http(self):
        if self._session is None:
            import requests

            self._session = requests.Session()
        return self._session

    def _prompt(self, i: int):
        item = self.prompts[i % len(self.prompts)]
        task = item if isinstance(item, dict) else None
        ids = np.asarray(item["prompt_ids"] if task is not None else item, dtype=np.int64)
        return (ids[-self.max_prompt:] if self.max_prompt else ids), task

    def _sample(self, ids: np.ndarray) -> list[tuple[np.ndarray, np.ndarray]]:
        payload = {"model": self.model_id, "prompt": [int(x) for x in ids], "n": self.g, "max_tokens": self.max_new,
                   "temperature": self.temperature, "top_p": self.top_p, "logprobs": 0, "return_tokens_as_token_ids": True}
        if self.top_k > 0:
            payload["top_k"] = self.top_k
        resp = self._http().request("POST", self.url + "/v1/completions", json=payload, timeout=self.timeout_s)
        if resp.status_code >= 400:
            raise RuntimeError(f"the generation server refused a completion request: HTTP {resp.status_code} {resp.text[:300]}")
        out = []
        for choice in resp.json()["choices"]:
            lp = choice.get("logprobs") or {}
            tokens = lp.get("tokens") or []
            if not tokens or not all(str(t).startswith("token_id:") for t in tokens):
                raise RuntimeError("the server did not return sampled token ids (start it with token ids in the log-probability "
                                   "output, e.g. return_tokens_as_token_ids): re-tokenising its text would not give the sampled tokens")
            toks = np.asarray([int(str(t).split(":", 1)[1]) for t in tokens], dtype=np.int64)
            out.append((toks, np.asarray(lp.get("token_logprobs") or [], dtype=np.float32)))
        return out

    def __call__(self, round_index: int):
        from halo_b200.trainers.grpo.trainer import Rollout

        picks = [self._prompt(round_index * self.per_round + j) for j in range(self.per_round)]
        with cf.ThreadPoolExecutor(max_workers=min(self.concurrency, len(picks))) as pool:
            sampled = list(pool.map(lambda p: self._sample(p[0]), picks))
        rollouts = []
        self.last_tasks = [task for (_, task), group in zip(picks, sampled) for _ in group]
        for (ids, task), group in zip(picks, sampled):
            for toks, logps in group:
                rollouts.append(Rollout(ids, toks, logps if len(logps) == len(toks) else None, self.reward_fn(ids, toks, task)))
        self.mean_reward = float(np.mean([r.reward for r in rollouts])) if rollouts else float("nan")
        return rollouts
