"""Environment lifecycle (halo/environments/environment_base.py:41-347).

An environment owns a task instance for one episode: ``reset`` returns the opening messages, ``step`` takes
the policy's reply and returns the next observation (tool result, user turn) or ends the episode, ``score``
returns the verdict the reward terms read. Tool calls are counted against a budget; a malformed turn is
answered with a corrective observation a bounded number of times before the episode is cut."""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class Turn:
    role: str
    content: str
    tool_calls: list | None = None
    logprobs: list | None = None
    token_ids: list | None = None


@dataclass
class EpisodeRecord:
    messages: list[dict] = field(default_factory=list)
    turns: list[Turn] = field(default_factory=list)
    score: float = 0.0
    done_reason: str = ""
    tool_calls_used: int = 0
    info: dict = field(default_factory=dict)

    @property
    def completion(self) -> str:
        return "\n".join(t.content for t in self.turns if t.role == "assistant")


class Environment:
    env_type = "base"
    max_turns = 8
    max_tool_calls = 16
    max_recoveries = 2

    def __init__(self, task: dict, **options):
        self.task, self.options = task, options
        self.record = EpisodeRecord()
        self._recoveries = 0

    # ---- to implement ------------------------------------------------------------------------
    def reset(self) -> list[dict]:
        """Opening messages of the episode."""
        raise NotImplementedError

    def step(self, reply: Turn) -> tuple[list[dict], bool]:
        """Observation messages for the next turn and whether the episode is over."""
        raise NotImplementedError

    def score(self) -> float:
        raise NotImplementedError

    # ---- shared behaviour ----------------------------------------------------------------------
    def tools(self) -> list[dict]:
        return []

    def charge_tool_calls(self, n: int) -> bool:
        self.record.tool_calls_used += n
        return self.record.tool_calls_used <= self.max_tool_calls

    def recover(self, why: str) -> tuple[list[dict], bool]:
        """A turn the environment could not parse: say why and let the policy retry, a bounded number of times."""
        self._recoveries += 1
        if self._recoveries > self.max_recoveries:
            self.record.done_reason = "malformed_turns"
            return [], True
        return [{"role": "user", "content": f"Your last message could not be used: {why}. Try again."}], False

    def close(self) -> None:
        """Release sandboxes and other resources."""
