"""Rollouts from environment episodes played against the job's own sampler: every round takes a few tasks, plays
``num_generations`` episodes of each (multi-turn, with tools where the environment has them), scores them with the
environment and the reward terms, and returns one training row per episode whose mask marks the policy's tokens
(halo/trainers/grpo/environmental/step_batch.py, halo/environments/rollouts/ray_actors.py:210-398 - here without
Ray: the episodes of a round run as coroutines over one sampler)."""

from __future__ import annotations

import asyncio

import numpy as np

from halo_b200.environments.episode_loop import play_episode
from halo_b200.environments.local_policy import LocalPolicy
from halo_b200.environments.registry import make_environment
from halo_b200.inference.generate import Generator, SamplingParams
from halo_b200.trainers.grpo.trainer import Rollout


class EnvironmentRolloutSource:
    def __init__(self, model, tokenizer, tasks: list[dict], env_type: str, num_generations: int, sampling: SamplingParams,
                 tasks_per_round: int = 4, composer=None, env_options: dict | None = None, seed: int = 0, rounds: int = 0):
        self.generator = Generator(model, eos_token_id=getattr(tokenizer, "eos_token_id", None))
        self.tokenizer, self.tasks, self.env_type = tokenizer, tasks, env_type
        self.g, self.sampling, self.per_round = num_generations, sampling, tasks_per_round
        self.composer, self.env_options, self.seed, self.rounds = composer, env_options or {}, seed, rounds
        self.mean_reward = float("nan")
        self.last_records: list = []
        self.drifted = 0

    async def _play_round(self, picks, round_index):
        policy = LocalPolicy(self.generator, self.tokenizer,
                             SamplingParams(self.sampling.max_new_tokens, self.sampling.temperature, self.sampling.top_k,
                                            self.sampling.top_p, self.sampling.stop_token_ids, None))
        jobs = []
        for ti, task in enumerate(picks):
            for k in range(self.g):
                env = make_environment(self.env_type, task, **self.env_options)
                jobs.append((ti * self.g + k, play_episode(env, policy.for_episode(ti * self.g + k), self.composer)))
        # the sampler is one device queue: the episodes take turns on it in a fixed order, so a round is reproducible
        records = []
        for key, coro in jobs:
            records.append((key, await coro))
        return policy, records

    def __call__(self, round_index: int):
        if self.rounds and round_index >= self.rounds:
            return None
        picks = [self.tasks[(round_index * self.per_round + j) % len(self.tasks)] for j in range(self.per_round)]
        was_training = self.generator.model.training
        import torch

        torch.manual_seed(self.seed * 1000003 + round_index)          # unseeded sampling draws from the global generator
        policy, records = asyncio.run(self._play_round(picks, round_index))
        self.generator.model.train(was_training)
        rollouts = []
        for key, rec in records:
            toks = policy.episodes[key]
            self.drifted += int(toks.drifted)
            reward = float(rec.info.get("reward", rec.score))
            mask = np.asarray(toks.policy_mask, dtype=np.int64)
            rollouts.append(Rollout(np.asarray(toks.prompt_ids, dtype=np.int64), np.asarray(toks.later_ids, dtype=np.int64),
                                    np.asarray(toks.logprobs, dtype=np.float32), reward, mask))
        self.last_records = [r for _, r in records]
        self.mean_reward = float(np.mean([r.reward for r in rollouts]))
        return rollouts
