"""``env_type`` -> factory (halo/environments/registry.py:28-96). Built-ins register at import."""

from __future__ import annotations

_FACTORIES: dict = {}


def register_environment(env_type: str, factory=None):
    def deco(f):
        if env_type in _FACTORIES:
            raise ValueError(f"environment type {env_type!r} is already registered")
        _FACTORIES[env_type] = f
        return f

    return deco(factory) if factory is not None else deco


def make_environment(env_type: str, task: dict, **options):
    _load_builtins()
    try:
        factory = _FACTORIES[env_type]
    except KeyError:
        raise KeyError(f"unknown environment type {env_type!r}; registered: {sorted(_FACTORIES)}") from None
    return factory(task, **options)


def environment_types() -> list[str]:
    _load_builtins()
    return sorted(_FACTORIES)


def _load_builtins() -> None:
    from . import tasks  # noqa: F401  (registers qa, code, tool_qa)
    from . import mcp  # noqa: F401  (registers mcp)
