"""Small guards shared by every config dataclass: bounds, choices, "differs from default" and
refusal of arguments a code path cannot honour (the role of halo/config_validation.py)."""

from __future__ import annotations

import dataclasses
from typing import Any, Iterable


class ConfigError(ValueError):
    """A configuration the framework refuses, with the remedy in the message."""


def require_positive(name: str, value) -> None:
    if not isinstance(value, (int, float)) or isinstance(value, bool) or value <= 0:
        raise ConfigError(f"{name} must be a positive number, got {value!r}")


def require_positive_int(name: str, value) -> None:
    if not isinstance(value, int) or isinstance(value, bool) or value < 1:
        raise ConfigError(f"{name} must be an integer >= 1, got {value!r}")


def require_non_negative(name: str, value) -> None:
    if not isinstance(value, (int, float)) or isinstance(value, bool) or value < 0:
        raise ConfigError(f"{name} must be >= 0, got {value!r}")


def require_in_range(name: str, value, lo, hi) -> None:
    if not (lo <= value <= hi):
        raise ConfigError(f"{name} must lie in [{lo}, {hi}], got {value!r}")


def require_choice(name: str, value, choices: Iterable) -> None:
    choices = tuple(choices)
    if value not in choices:
        raise ConfigError(f"{name} must be one of {', '.join(map(repr, choices))}; got {value!r}")


def require_divides(name_a: str, a: int, name_b: str, b: int) -> None:
    if a == 0 or b % a:
        raise ConfigError(f"{name_a} ({a}) must divide {name_b} ({b})")


def differs_from_default(obj, field_name: str) -> bool:
    for f in dataclasses.fields(obj):
        if f.name == field_name:
            if f.default is not dataclasses.MISSING:
                default = f.default
            elif f.default_factory is not dataclasses.MISSING:  # type: ignore[misc]
                default = f.default_factory()  # type: ignore[misc]
            else:
                return True
            return getattr(obj, field_name) != default
    raise AttributeError(field_name)


def reject_non_default_args(obj, names: Iterable[str], reason: str) -> None:
    """Raise when any of ``names`` was moved off its default although ``reason`` makes it inert."""
    moved = [n for n in names if differs_from_default(obj, n)]
    if moved:
        raise ConfigError(f"{', '.join(moved)} cannot be set here: {reason}")


class ValidatedConfig:
    """Mixin: ``__post_init__`` runs ``validate()``; ``replace`` re-validates."""

    def __post_init__(self) -> None:
        self.validate()

    def validate(self) -> None:  # pragma: no cover - overridden
        pass

    def replace(self, **changes: Any):
        return dataclasses.replace(self, **changes)
