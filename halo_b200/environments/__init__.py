"""Environments for RL rollouts: lifecycle base class, registry, episode loop, sandboxes, tasks."""
from .base import Environment, EpisodeRecord, Turn  # noqa: F401
from .registry import make_environment, register_environment  # noqa: F401
