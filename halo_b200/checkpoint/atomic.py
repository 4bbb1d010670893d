"""Atomic file publication: write to a staged name, fsync, rename, fsync the directory. A reader
never sees a half-written file and a crash leaves either the old file or the new one (the role of
halo/checkpoint/atomic.py)."""

from __future__ import annotations

import json
import os
import tempfile
from contextlib import contextmanager


def fsync_dir(directory: str) -> None:
    try:
        fd = os.open(directory, os.O_RDONLY)
    except OSError:
        return
    try:
        os.fsync(fd)
    except OSError:
        pass
    finally:
        os.close(fd)


@contextmanager
def staged_path(final_path: str):
    """Yields a temporary path in the same directory; on success it is renamed over ``final_path``."""
    directory = os.path.dirname(os.path.abspath(final_path)) or "."
    os.makedirs(directory, exist_ok=True)
    fd, tmp = tempfile.mkstemp(prefix=".staged-", suffix="-" + os.path.basename(final_path), dir=directory)
    os.close(fd)
    try:
        yield tmp
        with open(tmp, "rb") as f:
            os.fsync(f.fileno())
        os.replace(tmp, final_path)
        fsync_dir(directory)
    except BaseException:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise


def atomic_write_bytes(path: str, data: bytes) -> None:
    with staged_path(path) as tmp:
        with open(tmp, "wb") as f:
            f.write(data)
            f.flush()
            os.fsync(f.fileno())


def atomic_write_json(path: str, obj, indent: int = 2) -> None:
    atomic_write_bytes(path, json.dumps(obj, indent=indent, sort_keys=True).encode())


def atomic_torch_save(obj, path: str) -> None:
    import torch

    with staged_path(path) as tmp:
        torch.save(obj, tmp)


def remove_stale_staged(directory: str) -> int:
    """Delete leftovers of an interrupted save."""
    n = 0
    if os.path.isdir(directory):
        for name in os.listdir(directory):
            if name.startswith(".staged-"):
                try:
                    os.remove(os.path.join(directory, name))
                    n += 1
                except OSError:
                    pass
    return n
