"""Logging set-up: one root handler, quiet third parties, warn-once, rank-tagged run-log names
(the role of halo/log.py)."""

from __future__ import annotations

import logging
import os
import sys

_FORMAT = "%(asctime)s %(levelname).1s %(name)s: %(message)s"
_QUIET = ("urllib3", "filelock", "fsspec", "datasets", "httpx", "matplotlib", "asyncio")
_seen: set[str] = set()
_configured = False


def configure_logging(level: str | int | None = None, stream=None) -> None:
    global _configured
    level = level or os.environ.get("HALO_LOG_LEVEL", "INFO")
    root = logging.getLogger()
    if not _configured:
        handler = logging.StreamHandler(stream or sys.stderr)
        handler.setFormatter(logging.Formatter(_FORMAT, "%H:%M:%S"))
        root.addHandler(handler)
        _configured = True
    root.setLevel(level)
    for name in _QUIET:
        logging.getLogger(name).setLevel(logging.WARNING)


def warn_once(logger: logging.Logger, message: str) -> None:
    if message not in _seen:
        _seen.add(message)
        logger.warning(message)


def rank_tag() -> str:
    rank = os.environ.get("RANK")
    return f"rank{rank}" if rank is not None else "rank0"


def run_log_name(prefix: str = "run") -> str:
    return f"{prefix}.{rank_tag()}.log" if int(os.environ.get("WORLD_SIZE", "1")) > 1 else f"{prefix}.log"


def is_main_process() -> bool:
    return int(os.environ.get("RANK", "0")) == 0


def info_rank0(logger: logging.Logger, message: str) -> None:
    if is_main_process():
        logger.info(message)


class TeeStream:
    """Duplicates a text stream into a file (the ``run.log`` tee of a training script)."""

    def __init__(self, stream, path: str):
        self.stream = stream
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self.file = open(path, "a", buffering=1)

    def write(self, data):
        self.stream.write(data)
        self.file.write(data)
        return len(data)

    def flush(self):
        self.stream.flush()
        self.file.flush()

    def isatty(self):
        return False
