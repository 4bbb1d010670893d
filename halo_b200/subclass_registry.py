"""Registries read off a base class's subclass tree: a family registers by subclassing and naming
what it claims (the role of halo/subclass_registry.py). Used by the MoE family specs, the trainers
and the checkpoint savers."""

from __future__ import annotations

from typing import Callable, Iterable, TypeVar

import torch.nn as nn

T = TypeVar("T")


def all_subclasses(base: type) -> list[type]:
    out, stack = [], list(base.__subclasses__())
    while stack:
        c = stack.pop()
        if c not in out:
            out.append(c)
            stack.extend(c.__subclasses__())
    return out


def build_class_claim_map(base: type, claim_attr: str) -> dict:
    """{claimed key: subclass} over every subclass that sets ``claim_attr`` (a key or an iterable of
    keys). Two subclasses claiming one key is a programming error."""
    out: dict = {}
    for cls in all_subclasses(base):
        claim = cls.__dict__.get(claim_attr)
        if claim is None:
            continue
        keys = claim if isinstance(claim, (tuple, list, set, frozenset)) else (claim,)
        for k in keys:
            if k in out and out[k] is not cls:
                raise TypeError(f"{k!r} is claimed by both {out[k].__name__} and {cls.__name__}")
            out[k] = cls
    return out


def swap_registered_modules(model: nn.Module, claim_map: dict[type, Callable[[nn.Module], nn.Module]]) -> int:
    """Replace every sub-module whose class is a key of ``claim_map`` by ``claim_map[cls](module)``."""
    n = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            make = claim_map.get(type(child))
            if make is not None:
                setattr(parent, name, make(child))
                n += 1
    return n


def registered_names(base: type, claim_attr: str) -> Iterable[str]:
    return sorted(map(str, build_class_claim_map(base, claim_attr)))
