"""Freeze parameters by name pattern before the optimizer is built (halo/model_loading/parallel/freeze_patterns.py):
``freeze: ["embed_tokens", "layers\\.(0|1)\\."]`` turns ``requires_grad`` off for every parameter whose name matches
any pattern; ``train_only`` does the reverse. A pattern that matches nothing is an error (a typo must not silently
train everything)."""

from __future__ import annotations

import re


def apply_freeze_patterns(model, freeze: list[str] | None = None, train_only: list[str] | None = None) -> dict:
    if freeze and train_only:
        raise ValueError("give either freeze patterns or train_only patterns, not both")
    names = [n for n, _ in model.named_parameters()]
    patterns = freeze or train_only or []
    compiled = [(p, re.compile(p)) for p in patterns]
    for p, rx in compiled:
        if not any(rx.search(n) for n in names):
            raise ValueError(f"pattern {p!r} matches no parameter of the model")
    frozen = trained = 0
    for name, param in model.named_parameters():
        hit = any(rx.search(name) for _, rx in compiled)
        grad = (not hit) if freeze else hit if train_only else True
        param.requires_grad_(grad)
        if grad:
            trained += param.numel()
        else:
            frozen += param.numel()
    if trained == 0:
        raise ValueError("the patterns freeze every parameter: nothing is left to train")
    return {"trainable": trained, "frozen": frozen}
