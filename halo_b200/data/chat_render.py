"""Conversations -> token ids with the spans a loss may count (halo/data/{chat_render,completion_spans,turn_markers}.py).

The tokenizer's own chat template is the source of truth. The tokens an assistant turn owns are found by rendering
prefixes: ``render(messages[:i], add_generation_prompt=True)`` is what the model has seen when it starts turn ``i``,
``render(messages[:i + 1])`` what exists after it, and the difference is the turn (its end-of-turn marker included,
so the model learns to stop). A template whose longer rendering does not extend the shorter one (it rewrites
history, e.g. by dropping earlier reasoning) is detected and the affected turn is left unscored rather than scored
on the wrong tokens. Without a chat template the ChatML fallback is used.
"""

from __future__ import annotations

import numpy as np

CHATML_ROLES = ("system", "user", "assistant", "tool")


def load_chat_template(name: str = "chatml") -> str:
    """A bundled training-time chat template (``halo_b200/data/templates/<name>.jinja``: ``chatml`` with tool calls,
    ``llama3``, ``gemma``, ``mistral``, ``harmony`` for gpt-oss), for tokenizers that ship none or ship one without
    generation markers: ``tokenizer.chat_template = load_chat_template()``. (The reference bundles training-time
    templates per family under ``jinja-templates/``.)"""
    import os

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "templates", f"{name}.jinja")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no bundled chat template named {name!r}")
    return open(path).read()


def chatml(messages: list[dict], add_generation_prompt: bool = False) -> str:
    text = "".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in messages)
    return text + ("<|im_start|>assistant\n" if add_generation_prompt else "")


def template_ids(tokenizer, messages, add_generation_prompt: bool, tools=None) -> list[int]:
    """Token ids of the tokenizer's own chat template (whatever container its version returns them in)."""
    kw = {"tools": tools} if tools else {}
    out = tokenizer.apply_chat_template(messages, add_generation_prompt=add_generation_prompt, tokenize=True, **kw)
    if hasattr(out, "keys"):
        out = out["input_ids"]
    return [int(t) for t in out]


def _render_ids(tokenizer, messages, add_generation_prompt: bool, tools=None) -> list[int]:
    if getattr(tokenizer, "chat_template", None) or not hasattr(tokenizer, "__call__"):
        return template_ids(tokenizer, messages, add_generation_prompt, tools)
    return list(tokenizer(chatml(messages, add_generation_prompt), add_special_tokens=False)["input_ids"])


def render_conversation(tokenizer, messages: list[dict], tools=None, train_on: str = "assistant", last_turn_only: bool = False):
    """Returns ``(ids [n], loss_mask [n] bool, report)``. ``train_on``: ``"assistant"`` (assistant turns) or ``"all"``.
    ``last_turn_only``: only the final assistant turn counts (preference / distillation rows). ``report["rewritten"]``
    counts turns whose prefix rendering was not a prefix of the full one."""
    full = _render_ids(tokenizer, messages, False, tools)
    mask = np.zeros(len(full), dtype=bool)
    if train_on == "all":
        mask[:] = True
        return np.asarray(full, dtype=np.int64), mask, {"rewritten": 0, "turns": 0}
    rewritten = turns = 0
    assistant = [i for i, m in enumerate(messages) if m["role"] == "assistant"]
    if last_turn_only:
        assistant = assistant[-1:]
    for i in assistant:
        before = _render_ids(tokenizer, messages[:i], True, tools)
        after = _render_ids(tokenizer, messages[:i + 1], False, tools)
        turns += 1
        if full[:len(after)] != after or after[:len(before)] != before:
            rewritten += 1
            continue
        mask[len(before):len(after)] = True
    return np.asarray(full, dtype=np.int64), mask, {"rewritten": rewritten, "turns": turns}


def completion_spans(mask: np.ndarray) -> list[tuple[int, int]]:
    """``[start, stop)`` runs of a loss mask."""
    edges = np.flatnonzero(np.diff(np.concatenate([[0], mask.astype(np.int8), [0]])))
    return list(zip(edges[0::2].tolist(), edges[1::2].tolist()))
