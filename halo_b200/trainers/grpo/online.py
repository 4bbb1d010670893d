"""On-policy rollouts from the trainer's own weights: every round samples ``num_generations`` completions for
each of a few prompts with :class:`halo_b200.inference.generate.Generator`, scores them and hands the trainer
``Rollout`` records with the sampler's log-probabilities. Because the sampler is the policy itself, a round is
exactly on-policy at its first optimizer step.

Rewards come from a callable ``reward_fn(prompt_ids, completion_ids, task) -> float``; :func:`text_reward` adapts a
tokenizer plus a :class:`halo_b200.rewards.terms.RewardComposer` to it, :func:`token_match_reward` is a tokenizer-free
verifiable reward for smoke runs. The role of the reference's online GRPO trainer with its generation server
(halo/trainers/grpo/online.py, halo/trainers/grpo/on_policy.py).
"""

from __future__ import annotations

from typing import Callable, Sequence

import numpy as np

from halo_b200.inference.generate import Generator, SamplingParams
from halo_b200.trainers.grpo.trainer import Rollout


def token_match_reward(target_token: int) -> Callable:
    """Fraction of completion tokens equal to ``target_token``."""

    def reward(prompt_ids, completion_ids, task=None) -> float:
        return float(np.mean(np.asarray(completion_ids) == target_token)) if len(completion_ids) else 0.0

    return reward


def token_below_reward(threshold: int) -> Callable:
    """Fraction of completion tokens whose id is below ``threshold`` (a dense signal on any vocabulary)."""

    def reward(prompt_ids, completion_ids, task=None) -> float:
        return float(np.mean(np.asarray(completion_ids) < threshold)) if len(completion_ids) else 0.0

    return reward


def text_reward(tokenizer, composer) -> Callable:
    """Decode and score with a reward composer; a failing scorer counts as that term's failure value there."""

    def reward(prompt_ids, completion_ids, task=None) -> float:
        episode = dict(task or {})
        episode.setdefault("prompt", tokenizer.decode(list(map(int, prompt_ids))))
        episode["completion"] = tokenizer.decode(list(map(int, completion_ids)), skip_special_tokens=True)
        return float(composer.score(episode)[0])

    return reward


class OnPolicyRolloutSource:
    def __init__(self, model, prompts: Sequence, reward_fn: Callable, num_generations: int, sampling: SamplingParams,
                 prompts_per_round: int = 8, eos_token_id: int | None = None, seed: int = 0, max_prompt_length: int = 0,
                 rounds: int = 0, record_routing: bool = False):
        if not len(prompts):
            raise ValueError("on-policy rollouts need at least one prompt")
        self.generator = Generator(model, eos_token_id=eos_token_id)
        self.prompts, self.reward_fn = prompts, reward_fn
        self.g, self.sampling, self.per_round = num_generations, sampling, prompts_per_round
        self.seed, self.max_prompt, self.rounds = seed, max_prompt_length, rounds
        self.mean_reward = float("nan")
        self.record_routing = record_routing and model.cfg.is_moe

    def _prompt(self, i: int):
        item = self.prompts[i % len(self.prompts)]
        task = item if isinstance(item, dict) else None
        ids = np.asarray(item["prompt_ids"] if task is not None else item, dtype=np.int64)
        return (ids[-self.max_prompt:] if self.max_prompt else ids), task

    def __call__(self, round_index: int):
        if self.rounds and round_index >= self.rounds:
            return None
        picks = [self._prompt(round_index * self.per_round + j) for j in range(self.per_round)]
        batch = [ids for ids, _ in picks for _ in range(self.g)]
        params = SamplingParams(self.sampling.max_new_tokens, self.sampling.temperature, self.sampling.top_k, self.sampling.top_p,
                                self.sampling.stop_token_ids, self.seed * 1000003 + round_index)
        was_training = self.generator.model.training
        outs = self.generator.generate(batch, params, record_routing=self.record_routing)
        self.generator.model.train(was_training)
        rollouts = []
        self.last_tasks = [picks[n // self.g][1] for n in range(len(outs))]      # the task row of every rollout, in order
        for n, out in enumerate(outs):
            ids, task = picks[n // self.g]
            rollouts.append(Rollout(ids, out.token_ids, out.logprobs, self.reward_fn(ids, out.token_ids, task),
                                    routing=out.extra.get("routing"), routing_layers=out.extra.get("routing_layers")))
        self.mean_reward = float(np.mean([r.reward for r in rollouts]))
        return rollouts
