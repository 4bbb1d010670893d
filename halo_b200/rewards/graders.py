"""Verifiable graders: answer normalisation, strict ``\\boxed{}`` accuracy, regex format checks
(halo/rewards/graders/matching.py, halo/rewards/graders/verifiable.py)."""

from __future__ import annotations

import re
import unicodedata

_BOXED = re.compile(r"\\boxed\s*\{")


def normalize_answer(text: str) -> str:
    t = unicodedata.normalize("NFKC", str(text)).strip().lower()
    t = re.sub(r"\\(?:text|mathrm|mathbf)\s*\{([^{}]*)\}", r"\1", t)
    t = t.replace("\\!", "").replace("\\,", "").replace("\\ ", "").replace("$", "")
    t = re.sub(r"\s+", " ", t).strip(" .")
    t = re.sub(r"(?<=\d),(?=\d{3}\b)", "", t)               # 1,000 -> 1000
    if re.fullmatch(r"-?\d+\.\d*0+", t):
        t = t.rstrip("0").rstrip(".")
    return t


def last_boxed(text: str) -> str | None:
    """Content of the last ``\\boxed{...}`` with balanced braces, else None."""
    last = None
    for m in _BOXED.finditer(text):
        depth, i = 1, m.end()
        while i < len(text) and depth:
            depth += {"{": 1, "}": -1}.get(text[i], 0)
            i += 1
        if depth == 0:
            last = text[m.end():i - 1]
    return last


def boxed_accuracy(completion: str, target: str, strict: bool = True) -> float:
    got = last_boxed(completion)
    if got is None:
        if strict:
            return 0.0
        got = completion.strip().splitlines()[-1] if completion.strip() else ""
    a, b = normalize_answer(got), normalize_answer(target)
    if a == b:
        return 1.0
    try:
        return float(abs(float(a) - float(b)) <= 1e-9 * max(1.0, abs(float(b))))
    except ValueError:
        return 0.0


def exact_match(completion: str, target: str) -> float:
    return float(normalize_answer(completion) == normalize_answer(target))


def regex_format(completion: str, pattern: str, full: bool = True) -> float:
    rx = re.compile(pattern, re.DOTALL)
    return float(bool(rx.fullmatch(completion) if full else rx.search(completion)))


def think_answer_format(completion: str) -> float:
    return regex_format(completion.strip(), r"<think>.*?</think>\s*\S.*")


GRADERS = {"boxed_accuracy": boxed_accuracy, "exact_match": exact_match}
