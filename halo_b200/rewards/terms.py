"""Typed reward terms and their composition (halo/rewards/terms.py:151-507, halo/rewards/composer.py:47-141).

reward = sum over terms of ``weight * score ** exponent``. A term's score comes from the environment's own
verdict, a verifiable grader, a judge model or a reward model; external scorers (judge, reward model) are
asynchronous callables settled together by the composer. Terms are parsed and validated at configuration
time, so a typo fails before the first rollout."""

from __future__ import annotations

import asyncio
from dataclasses import dataclass, field
from typing import Awaitable, Callable

from . import graders


@dataclass(frozen=True)
class RewardTerm:
    name: str
    weight: float = 1.0
    exponent: float = 1.0

    def __post_init__(self):
        if self.exponent <= 0:
            raise ValueError(f"term {self.name!r}: exponent must be positive")

    def shaped(self, score: float) -> float:
        s = min(max(float(score), 0.0), 1.0) if self.exponent != 1.0 else float(score)
        return self.weight * s ** self.exponent


@dataclass(frozen=True)
class EnvironmentTerm(RewardTerm):
    """The environment's own verdict (tests passed, task solved ...), read from the episode record."""
    key: str = "score"


@dataclass(frozen=True)
class GraderTerm(RewardTerm):
    grader: str = "boxed_accuracy"

    def __post_init__(self):
        super().__post_init__()
        if self.grader not in graders.GRADERS and self.grader not in ("think_answer_format",):
            raise ValueError(f"term {self.name!r}: unknown grader {self.grader!r}")


@dataclass(frozen=True)
class FormatTerm(RewardTerm):
    pattern: str = r".*"


@dataclass(frozen=True)
class JudgeTerm(RewardTerm):
    """An LLM judge returns a JSON verdict with a ``score`` in [0, 1]."""
    rubric: str = ""
    model: str = ""


@dataclass(frozen=True)
class RewardModelTerm(RewardTerm):
    endpoint: str = ""


@dataclass(frozen=True)
class PolicyCheckTerm(RewardTerm):
    """The White Circle API's policy check of the completion in its conversation against the policies of
    ``environment_id``. With nothing listed the score is 1 unless the completion was flagged, else 0; with ``policies``
    (policy ids) it is the fraction of them the completion did not violate; a ``checklist`` (the policy ids of its
    items) is one judgment: its confidence is the fraction of items hit, its score 1 minus that. A term lists
    ``policies`` or a ``checklist``, not both. ``view``: "full" reads every assistant turn of the completion, "final"
    the last one. ``max_retries`` bounds the retries of a rate-limited or failed request, ``retry_wait`` is the first
    backoff in seconds."""
    environment_id: str = ""
    policies: tuple = ()
    checklist: tuple = ()
    region: str = "us"
    view: str = "full"
    max_retries: int = 4
    retry_wait: float = 1.0
    request_timeout: float = 30.0
    max_concurrency: int = 8

    def __post_init__(self):
        super().__post_init__()
        if not str(self.environment_id).strip():
            raise ValueError(f"term {self.name!r}: environment_id is required")
        for f in ("policies", "checklist"):
            ids = getattr(self, f)
            if isinstance(ids, str) or not hasattr(ids, "__iter__"):
                raise ValueError(f"term {self.name!r}: {f} must be a list of policy ids, got {ids!r}")
            object.__setattr__(self, f, tuple(ids))
        if self.policies and self.checklist:
            raise ValueError(f"term {self.name!r}: list policies or a checklist, not both")
        if self.view not in ("full", "final"):
            raise ValueError(f"term {self.name!r}: view must be 'full' or 'final'")
        if self.max_retries < 0 or self.retry_wait < 0 or self.request_timeout <= 0 or self.max_concurrency < 1:
            raise ValueError(f"term {self.name!r}: max_retries / retry_wait must not be negative, request_timeout and "
                             "max_concurrency must be positive")


TERM_TYPES = {"environment": EnvironmentTerm, "grader": GraderTerm, "format": FormatTerm, "judge": JudgeTerm,
              "reward_model": RewardModelTerm, "whitecircle": PolicyCheckTerm}


def parse_terms(spec: list[dict]) -> list[RewardTerm]:
    out, seen = [], set()
    for i, item in enumerate(spec):
        item = dict(item)
        kind = item.pop("type", None)
        if kind not in TERM_TYPES:
            raise ValueError(f"reward term {i}: unknown type {kind!r}; choose from {sorted(TERM_TYPES)}")
        item.setdefault("name", f"{kind}_{i}")
        try:
            term = TERM_TYPES[kind](**item)
        except TypeError as exc:
            raise ValueError(f"reward term {i} ({kind}): {exc}") from None
        if term.name in seen:
            raise ValueError(f"two reward terms are named {term.name!r}")
        seen.add(term.name)
        out.append(term)
    if not out:
        raise ValueError("a reward needs at least one term")
    return out


@dataclass
class RewardComposer:
    terms: list[RewardTerm]
    judge: Callable[[JudgeTerm, dict], Awaitable[float]] | None = None
    reward_model: Callable[[RewardModelTerm, dict], Awaitable[float]] | None = None
    policy_check: Callable[[PolicyCheckTerm, dict], Awaitable[float]] | None = None
    timeout_s: float = 120.0
    failures: int = field(default=0, init=False)

    def _local(self, term: RewardTerm, episode: dict) -> float | None:
        if isinstance(term, EnvironmentTerm):
            return float(episode.get(term.key, 0.0))
        if isinstance(term, GraderTerm):
            if term.grader == "think_answer_format":
                return graders.think_answer_format(episode["completion"])
            return graders.GRADERS[term.grader](episode["completion"], episode.get("target", ""))
        if isinstance(term, FormatTerm):
            return graders.regex_format(episode["completion"], term.pattern)
        return None

    async def score_async(self, episode: dict) -> tuple[float, dict]:
        parts, pending = {}, {}
        for t in self.terms:
            s = self._local(t, episode)
            if s is not None:
                parts[t.name] = s
            elif isinstance(t, JudgeTerm):
                if self.judge is None:
                    raise RuntimeError(f"term {t.name!r} needs a judge scorer")
                pending[t.name] = asyncio.ensure_future(self.judge(t, episode))
            elif isinstance(t, RewardModelTerm):
                if self.reward_model is None:
                    raise RuntimeError(f"term {t.name!r} needs a reward-model scorer")
                pending[t.name] = asyncio.ensure_future(self.reward_model(t, episode))
            elif isinstance(t, PolicyCheckTerm):
                if self.policy_check is None:
                    raise RuntimeError(f"term {t.name!r} needs a policy-check scorer")
                pending[t.name] = asyncio.ensure_future(self.policy_check(t, episode))
        if pending:
            done, late = await asyncio.wait(pending.values(), timeout=self.timeout_s)
            for name, fut in pending.items():
                if fut in done and fut.exception() is None:
                    parts[name] = float(fut.result())
                else:                      # a scorer that failed or timed out scores zero and is counted
                    fut.cancel()
                    parts[name] = 0.0
                    self.failures += 1
        total = sum(t.shaped(parts[t.name]) for t in self.terms)
        return total, parts

    def score(self, episode: dict) -> tuple[float, dict]:
        return asyncio.run(self.score_async(episode))
