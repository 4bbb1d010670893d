"""The policy side of an episode served by the job's own sampler instead of an HTTP endpoint: ``LocalPolicy`` is the
``generate(messages, tools) -> Turn`` callable of :func:`halo_b200.environments.episode_loop.play_episode`, and
:class:`EpisodeTokens` turns a finished multi-turn episode into ONE training row - the first prompt, then every later
token in order, with a mask that is 1 on the tokens the policy sampled and 0 on what the environment put between them
(tool results, user turns, template tokens).

A later prompt must extend what the policy has already seen: the chat template is re-rendered every turn and its
token ids must start with ``previous prompt + sampled tokens``. Where re-tokenisation breaks that (a template that
rewrites history), the row is cut at the last consistent turn and the episode is flagged.
(halo/environments/rollouts/episode_loop.py:117, halo/trainers/grpo/environmental/trajectory_tokenize.py)
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .base import Turn


@dataclass
class EpisodeTokens:
    prompt_ids: list[int] = field(default_factory=list)      # the first prompt
    later_ids: list[int] = field(default_factory=list)       # everything after it, in order
    policy_mask: list[int] = field(default_factory=list)     # 1 where the policy sampled the token
    logprobs: list[float] = field(default_factory=list)      # sampler log-probs (0 on environment tokens)
    drifted: bool = False

    def seen(self) -> list[int]:
        return self.prompt_ids + self.later_ids


class LocalPolicy:
    def __init__(self, generator, tokenizer, sampling, max_context: int = 0):
        self.generator, self.tokenizer, self.sampling, self.max_context = generator, tokenizer, sampling, max_context
        self.episodes: dict[int, EpisodeTokens] = {}

    def track(self, key: int) -> EpisodeTokens:
        self.episodes[key] = EpisodeTokens()
        return self.episodes[key]

    def _render(self, messages, tools) -> list[int]:
        from halo_b200.data.chat_render import template_ids

        return template_ids(self.tokenizer, messages, True, tools)

    def for_episode(self, key: int):
        """The ``generate`` callable bound to one episode's token record."""
        rec = self.track(key)

        async def generate(messages, tools):
            ids = self._render(messages, tools)
            if not rec.prompt_ids:
                rec.prompt_ids = ids
            else:
                seen = rec.seen()
                if ids[:len(seen)] != seen:
                    rec.drifted = True                   # history was re-tokenised differently: stop extending the row
                else:
                    extra = ids[len(seen):]
                    rec.later_ids += extra
                    rec.policy_mask += [0] * len(extra)
                    rec.logprobs += [0.0] * len(extra)
            if self.max_context and len(ids) >= self.max_context:
                return Turn("assistant", "", token_ids=[], logprobs=[])
            out = self.generator.generate([np.asarray(ids)], self.sampling)[0]
            toks, lps = out.token_ids.tolist(), out.logprobs.tolist()
            if not rec.drifted:
                rec.later_ids += toks
                rec.policy_mask += [1] * len(toks)
                rec.logprobs += lps
            return Turn("assistant", self.tokenizer.decode(toks, skip_special_tokens=True), token_ids=toks, logprobs=lps)

        return generate
