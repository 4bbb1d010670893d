"""Built-in tasks: single-turn question answering with a verifiable answer, and code problems graded on hidden
tests in a sandbox (halo/environments/tasks/qa.py, halo/environments/tasks/coding/*.py)."""

from __future__ import annotations

import re

from halo_b200.rewards import graders

from .base import Environment, Turn
from .registry import register_environment
from .sandbox import make_sandbox

_CODE_BLOCK = re.compile(r"```(?:python)?\n(.*?)```", re.DOTALL)


@register_environment("qa")
class QAEnvironment(Environment):
    env_type = "qa"
    max_turns = 1

    def reset(self):
        sys_prompt = self.options.get("system_prompt", "Answer the question. Put the final answer in \\boxed{}.")
        self.record.messages = [{"role": "system", "content": sys_prompt}, {"role": "user", "content": self.task["question"]}]
        return list(self.record.messages)

    def step(self, reply: Turn):
        self.record.turns.append(reply)
        self.record.done_reason = "answered"
        return [], True

    def score(self) -> float:
        self.record.score = graders.boxed_accuracy(self.record.completion, self.task["answer"],
                                                   strict=self.options.get("strict", True))
        return self.record.score


def verdict(expected: str, got: str, comparator: str = "tokens") -> bool:
    """Output comparators of programming judges: exact, whitespace-insensitive tokens, or floats within 1e-6."""
    if comparator == "exact":
        return expected == got
    a, b = expected.split(), got.split()
    if comparator == "float":
        if len(a) != len(b):
            return False
        try:
            return all(abs(float(x) - float(y)) <= 1e-6 * max(1.0, abs(float(x))) for x, y in zip(a, b))
        except ValueError:
            return False
    return a == b


@register_environment("code")
class CodeEnvironment(Environment):
    """The policy writes a program; feedback on the public tests is given for up to ``max_turns`` attempts; the score
    is the fraction of hidden tests passed (or 0/1 with ``all_or_nothing``)."""

    env_type = "code"
    max_turns = 3

    def __init__(self, task, **options):
        super().__init__(task, **options)
        self.sandbox = make_sandbox(options.get("sandbox", "subprocess"))
        self.last_program = ""

    def reset(self):
        prompt = (self.task["statement"] + "\n\nWrite a Python program that reads stdin and writes stdout. "
                  "Reply with one ```python code block.")
        self.record.messages = [{"role": "user", "content": prompt}]
        return list(self.record.messages)

    def _run_tests(self, tests) -> list[bool]:
        out = []
        for t in tests:
            r = self.sandbox.run(self.last_program, t["input"], timeout_s=self.options.get("time_limit_s", 5.0))
            out.append(r.exit_code == 0 and not r.timed_out
                       and verdict(t["output"], r.stdout, self.task.get("comparator", "tokens")))
        return out

    def step(self, reply: Turn):
        self.record.turns.append(reply)
        m = _CODE_BLOCK.findall(reply.content)
        if not m:
            return self.recover("it holds no ```python code block")
        self.last_program = m[-1]
        public = self._run_tests(self.task.get("public_tests", []))
        if all(public) or len(self.record.turns) >= self.max_turns:
            self.record.done_reason = "submitted"
            return [], True
        failed = public.index(False)
        return [{"role": "user", "content": f"Public test {failed + 1} failed. Fix the program and send it again."}], False

    def score(self) -> float:
        hidden = self._run_tests(self.task.get("hidden_tests", []))
        frac = sum(hidden) / max(1, len(hidden))
        self.record.score = float(frac == 1.0) if self.options.get("all_or_nothing", False) else frac
        self.record.info["hidden_passed"] = sum(hidden)
        return self.record.score

    def close(self):
        self.sandbox.close()


@register_environment("tool_qa")
class ToolQAEnvironment(Environment):
    """A question answered over several turns with tools (calculator, optionally a sandboxed ``python``), under the
    native tool-call protocol or ReAct (``protocol`` option). The score is the graded final answer."""

    env_type = "tool_qa"
    max_turns = 6

    def __init__(self, task, **options):
        super().__init__(task, **options)
        from .protocols import PROTOCOLS, default_tools

        self.protocol = options.get("protocol", "native")
        self.parse, self.render = PROTOCOLS[self.protocol]
        self.sandbox = make_sandbox(options["sandbox"]) if options.get("sandbox") else None
        self.registry = options.get("tools") or default_tools(self.sandbox)
        self.answer = None

    def tools(self):
        return self.registry.definitions() if self.protocol == "native" else []

    def reset(self):
        from .protocols import REACT_INSTRUCTIONS

        system = self.options.get("system_prompt", "Solve the problem; use the tools when they help.")
        if self.protocol == "react":
            system += "\n" + REACT_INSTRUCTIONS.format(names=", ".join(self.registry.names()))
        self.record.messages = [{"role": "system", "content": system}, {"role": "user", "content": self.task["question"]}]
        return list(self.record.messages)

    def step(self, reply: Turn):
        from .protocols import MalformedTurn

        self.record.turns.append(reply)
        try:
            parsed = self.parse(reply)
        except MalformedTurn as exc:
            return self.recover(str(exc))
        if parsed.final_answer is not None:
            self.answer, self.record.done_reason = parsed.final_answer, "answered"
            return [], True
        if not self.charge_tool_calls(len(parsed.calls)):
            self.record.done_reason = "tool_budget"
            return [], True
        return [self.render(c, self.registry.call(c)) for c in parsed.calls], False

    def score(self) -> float:
        text = self.answer or ""
        if "\\boxed" in text:
            self.record.score = graders.boxed_accuracy(text, self.task["answer"], strict=False)
        else:
            self.record.score = float(graders.normalize_answer(text) == graders.normalize_answer(str(self.task["answer"])))
        return self.record.score

    def close(self):
        if self.sandbox is not None:
            self.sandbox.close()
