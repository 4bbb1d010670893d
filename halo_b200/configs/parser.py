"""YAML + ``--key=value`` -> dataclasses (the role of halo/configs/parser.py).

Rules kept from the reference: toolkit defaults only fill fields the user left unset
(halo/configs/parser.py:17-35); an unknown key raises with the closest known names; a retired key
raises with its remedy (halo/configs/parser.py:38-45); container-typed fields may only be given
in the YAML file; a field annotated ``Literal[...]`` only accepts its choices; ``%Y%m%d``-style
patterns in ``output_dir`` are expanded once (on rank 0, then shared).
"""

from __future__ import annotations

import dataclasses
import difflib
import sys
import time
import types
import typing
from typing import Any, Sequence

import yaml

from halo_b200.config_validation import ConfigError

TOOLKIT_DEFAULTS = {"bf16": True, "use_fused_kernels": True, "logging_nan_inf_filter": False,
                    "gradient_checkpointing": True, "packing": True}

RETIRED_KEYS = {
    "use_liger_kernel": "the fused RMSNorm / RoPE / SwiGLU / linear-cross-entropy kernels are always on; drop the key",
    "attn_implementation": "attention is the built-in sm_100a flash kernel; drop the key",
    "fsdp": "data parallelism is configured through the parallelism fields; drop the key",
    "deepspeed": "DeepSpeed is not used; configure parallelism through the parallelism fields",
    "ep_num_sms": "the expert transport sizes its own grids; drop the key",
}


def _is_container(tp) -> bool:
    origin = typing.get_origin(tp)
    if origin in (list, dict, tuple, set):
        return True
    if origin in (typing.Union, types.UnionType):
        return any(_is_container(a) for a in typing.get_args(tp))
    return tp in (list, dict, tuple, set)


def _coerce(name: str, tp, raw: Any, from_cli: bool):
    origin = typing.get_origin(tp)
    if origin in (typing.Union, types.UnionType):
        args = [a for a in typing.get_args(tp) if a is not type(None)]
        if raw is None or (isinstance(raw, str) and raw.lower() in ("none", "null")):
            return None
        last = None
        for a in args:
            try:
                return _coerce(name, a, raw, from_cli)
            except (ConfigError, ValueError, TypeError) as exc:
                last = exc
        raise ConfigError(f"{name}: cannot read {raw!r} as {tp}: {last}")
    if origin is typing.Literal:
        choices = typing.get_args(tp)
        for c in choices:
            if raw == c or (isinstance(raw, str) and str(c) == raw):
                return c
        raise ConfigError(f"{name} must be one of {', '.join(map(repr, choices))}; got {raw!r}")
    if _is_container(tp):
        if from_cli:
            raise ConfigError(f"{name} holds a container and can only be set in the YAML file")
        return raw
    if tp is bool:
        if isinstance(raw, bool):
            return raw
        if isinstance(raw, str) and raw.lower() in ("1", "true", "yes", "on"):
            return True
        if isinstance(raw, str) and raw.lower() in ("0", "false", "no", "off"):
            return False
        raise ConfigError(f"{name} must be a boolean, got {raw!r}")
    if tp is int:
        if isinstance(raw, bool):
            raise ConfigError(f"{name} must be an integer, got {raw!r}")
        if isinstance(raw, float) and raw != int(raw):
            raise ConfigError(f"{name} must be an integer, got {raw!r}")
        return int(raw)
    if tp is float:
        return float(raw)
    if tp is str:
        return str(raw)
    return raw


class ArgumentParser:
    """``ArgumentParser(SFTConfig, ModelArguments, ParallelismArguments).parse(argv)`` returns one
    instance per dataclass; every key must belong to exactly one of them."""

    def __init__(self, *dataclass_types):
        self.types = dataclass_types
        self.owner: dict[str, Any] = {}
        for t in dataclass_types:
            for f in dataclasses.fields(t):
                if f.name in self.owner:
                    raise TypeError(f"field {f.name!r} is declared by both {self.owner[f.name].__name__} and {t.__name__}")
                self.owner[f.name] = t

    def load_values(self, argv: Sequence[str] | None = None) -> tuple[dict, set[str]]:
        """(values, names given on the command line). The first non-option argument is the YAML file."""
        argv = list(sys.argv[1:] if argv is None else argv)
        values: dict[str, Any] = {}
        cli: set[str] = set()
        for arg in argv:
            if arg.startswith("--"):
                if "=" not in arg:
                    key, raw = arg[2:], "true"
                else:
                    key, raw = arg[2:].split("=", 1)
                key = key.replace("-", "_")
                values[key] = raw
                cli.add(key)
            else:
                with open(arg) as f:
                    loaded = yaml.safe_load(f) or {}
                if not isinstance(loaded, dict):
                    raise ConfigError(f"{arg} must hold a mapping at its top level")
                for k, v in loaded.items():
                    values.setdefault(k, v) if k in cli else values.__setitem__(k, v)
        return values, cli

    def parse_dict(self, values: dict, cli: set[str] | frozenset = frozenset()):
        for key in values:
            if key in RETIRED_KEYS:
                raise ConfigError(f"{key} is retired: {RETIRED_KEYS[key]}")
            if key not in self.owner:
                near = difflib.get_close_matches(key, self.owner, n=3)
                hint = f" Did you mean {', '.join(near)}?" if near else ""
                raise ConfigError(f"unknown configuration key {key!r}.{hint}")
        merged = dict(values)
        for k, v in TOOLKIT_DEFAULTS.items():
            if k in self.owner and k not in merged:
                merged[k] = v
        out = []
        for t in self.types:
            hints = typing.get_type_hints(t)
            kwargs = {}
            for f in dataclasses.fields(t):
                if f.name in merged and f.init:
                    kwargs[f.name] = _coerce(f.name, hints[f.name], merged[f.name], f.name in cli)
            try:
                out.append(t(**kwargs))
            except TypeError as exc:
                raise ConfigError(f"{t.__name__}: {exc}") from exc
        return tuple(out)

    def parse(self, argv: Sequence[str] | None = None):
        values, cli = self.load_values(argv)
        return self.parse_dict(values, cli)


def expand_output_dir(path: str, now: float | None = None) -> str:
    """``runs/%Y%m%d-%H%M`` -> ``runs/20250101-1200`` (call on rank 0 and broadcast the result)."""
    if "%" not in path:
        return path
    return time.strftime(path, time.localtime(now))
