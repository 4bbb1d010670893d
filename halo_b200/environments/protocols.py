"""How a policy's text becomes tool calls and how results go back (halo/environments/protocols/{native_tool_use,react}.py).

* native tool use - the reply carries calls either as structured ``tool_calls`` (an endpoint parsed them) or as
  ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` tags in the text (what Qwen / Hermes chat templates
  emit); results return as ``{"role": "tool", ...}`` messages;
* ReAct - plain text: ``Thought: ...`` / ``Action: <tool>`` / ``Action Input: <json or text>``, ended by
  ``Final Answer: ...``; results return as ``Observation: ...`` user messages.

Both parse into :class:`ToolCall` lists plus an optional final answer, and both refuse malformed turns with a reason
the environment can hand back to the policy. :class:`ToolRegistry` holds OpenAI-format definitions and dispatches
calls with arguments checked against the declared parameters.
"""

from __future__ import annotations

import json
import re
from dataclasses import dataclass, field


class MalformedTurn(ValueError):
    """The reply does not follow the protocol; ``str(exc)`` is the reason given back to the policy."""


@dataclass
class ToolCall:
    name: str
    arguments: dict
    call_id: str = ""


@dataclass
class ParsedTurn:
    calls: list[ToolCall] = field(default_factory=list)
    final_answer: str | None = None
    thought: str = ""


_TAG = re.compile(r"<tool_call>\s*(.*?)\s*</tool_call>", re.DOTALL)


def parse_native(reply) -> ParsedTurn:
    """``reply``: a :class:`halo_b200.environments.base.Turn`. A turn without calls is a final answer."""
    calls = []
    if reply.tool_calls:
        for i, c in enumerate(reply.tool_calls):
            fn = c.get("function", c)
            args = fn.get("arguments", {})
            if isinstance(args, str):
                try:
                    args = json.loads(args or "{}")
                except json.JSONDecodeError as exc:
                    raise MalformedTurn(f"the arguments of call {i + 1} are not JSON ({exc.msg})") from None
            calls.append(ToolCall(fn["name"], args, c.get("id", f"call_{i}")))
        return ParsedTurn(calls, None)
    for i, body in enumerate(_TAG.findall(reply.content)):
        try:
            obj = json.loads(body)
        except json.JSONDecodeError as exc:
            raise MalformedTurn(f"tool call {i + 1} is not JSON ({exc.msg})") from None
        if not isinstance(obj, dict) or "name" not in obj:
            raise MalformedTurn(f"tool call {i + 1} has no \"name\"")
        args = obj.get("arguments", {})
        if not isinstance(args, dict):
            raise MalformedTurn(f"the arguments of tool call {i + 1} are not an object")
        calls.append(ToolCall(obj["name"], args, f"call_{i}"))
    if "<tool_call>" in reply.content and not calls:
        raise MalformedTurn("a <tool_call> tag is not closed")
    if calls:
        return ParsedTurn(calls, None)
    return ParsedTurn([], _TAG.sub("", reply.content).strip())


def render_native_result(call: ToolCall, result: str) -> dict:
    return {"role": "tool", "tool_call_id": call.call_id, "name": call.name, "content": result}


_REACT_ACTION = re.compile(r"Action:\s*(.+?)\s*\n\s*Action Input:\s*(.*?)(?=\n\s*(?:Thought:|Action:|Observation:|Final Answer:)|\Z)",
                           re.DOTALL)
_REACT_FINAL = re.compile(r"Final Answer:\s*(.*)", re.DOTALL)
_REACT_THOUGHT = re.compile(r"Thought:\s*(.*?)(?=\n\s*(?:Action:|Final Answer:)|\Z)", re.DOTALL)


def parse_react(reply) -> ParsedTurn:
    text = reply.content
    thought = (_REACT_THOUGHT.search(text) or [None, ""])[1].strip() if _REACT_THOUGHT.search(text) else ""
    final = _REACT_FINAL.search(text)
    action = _REACT_ACTION.search(text)
    if action and (not final or action.start() < final.start()):
        # text after the first action is the policy imagining the observation: only the first action counts
        raw = action.group(2).strip()
        try:
            args = json.loads(raw) if raw.startswith("{") else {"input": raw}
        except json.JSONDecodeError as exc:
            raise MalformedTurn(f"the Action Input is not JSON ({exc.msg})") from None
        return ParsedTurn([ToolCall(action.group(1).strip(), args, "react_0")], None, thought)
    if final:
        return ParsedTurn([], final.group(1).strip(), thought)
    raise MalformedTurn("it has neither an \"Action:\" with an \"Action Input:\" nor a \"Final Answer:\"")


def render_react_result(call: ToolCall, result: str) -> dict:
    return {"role": "user", "content": f"Observation: {result}"}


REACT_INSTRUCTIONS = ("Use this format.\nThought: what you need next\nAction: one of [{names}]\nAction Input: a JSON object with the "
                      "tool's arguments\nAfter the observation continue, and finish with\nFinal Answer: the answer")

PROTOCOLS = {"native": (parse_native, render_native_result), "react": (parse_react, render_react_result)}


class ToolRegistry:
    def __init__(self):
        self._tools: dict[str, tuple[dict, object]] = {}

    def register(self, name: str, description: str, parameters: dict, fn) -> None:
        """``parameters``: JSON-schema ``properties`` (name -> {"type": ..., "description": ...}); all are required
        unless a property carries ``"optional": true``."""
        required = [k for k, v in parameters.items() if not v.get("optional")]
        props = {k: {kk: vv for kk, vv in v.items() if kk != "optional"} for k, v in parameters.items()}
        definition = {"type": "function", "function": {"name": name, "description": description,
                                                       "parameters": {"type": "object", "properties": props, "required": required}}}
        self._tools[name] = (definition, fn)

    def definitions(self) -> list[dict]:
        return [d for d, _ in self._tools.values()]

    def names(self) -> list[str]:
        return sorted(self._tools)

    def call(self, call: ToolCall) -> str:
        if call.name not in self._tools:
            return f"error: no tool named {call.name!r}; available: {', '.join(self.names())}"
        definition, fn = self._tools[call.name]
        schema = definition["function"]["parameters"]
        missing = [k for k in schema["required"] if k not in call.arguments]
        extra = [k for k in call.arguments if k not in schema["properties"]]
        if missing or extra:
            return f"error: {call.name} takes {sorted(schema['properties'])}" + (f", missing {missing}" if missing else "") + \
                (f", unknown {extra}" if extra else "")
        try:
            return str(fn(**call.arguments))
        except Exception as exc:  # noqa: BLE001 - a tool's failure is an observation, not a crash of the episode
            return f"error: {type(exc).__name__}: {exc}"


def calculator(expression: str) -> str:
    """Arithmetic on numbers only (no names, no calls): the AST is walked, never evaluated as code."""
    import ast
    import operator as op

    ops = {ast.Add: op.add, ast.Sub: op.sub, ast.Mult: op.mul, ast.Div: op.truediv, ast.Pow: op.pow, ast.Mod: op.mod,
           ast.FloorDiv: op.floordiv, ast.USub: op.neg, ast.UAdd: op.pos}

    def ev(node):
        if isinstance(node, ast.Constant) and isinstance(node.value, (int, float)):
            return node.value
        if isinstance(node, ast.BinOp) and type(node.op) in ops:
            left, right = ev(node.left), ev(node.right)
            if isinstance(node.op, ast.Pow) and abs(right) > 64:
                raise ValueError("exponent too large")
            return ops[type(node.op)](left, right)
        if isinstance(node, ast.UnaryOp) and type(node.op) in ops:
            return ops[type(node.op)](ev(node.operand))
        raise ValueError("only numbers and + - * / // % ** are allowed")

    return repr(ev(ast.parse(expression, mode="eval").body))


def default_tools(sandbox=None) -> ToolRegistry:
    reg = ToolRegistry()
    reg.register("calculator", "Evaluate an arithmetic expression.", {"expression": {"type": "string", "description": "e.g. (3 + 4) * 2"}},
                 calculator)
    if sandbox is not None:
        def run_python(code: str, stdin: str = "") -> str:
            r = sandbox.run(code, stdin, timeout_s=5.0)
            return (r.stdout if r.exit_code == 0 and not r.timed_out else f"exit {r.exit_code}{' (timed out)' if r.timed_out else ''}\n"
                    f"{r.stdout}{r.stderr}")[:4000]

        reg.register("python", "Run a Python program and return what it prints.",
                     {"code": {"type": "string", "description": "the program"},
                      "stdin": {"type": "string", "description": "its standard input", "optional": True}}, run_python)
    return reg
