"""Is a path on storage every node sees, or per node? Which rank writes? (the role of
halo/runtime/filesystem.py). ``DIST_INPUT_SHARED_FILESYSTEM`` / ``DIST_OUTPUT_SHARED_FILESYSTEM``
declare it; a sentinel-file probe checks the declaration on multi-node jobs."""

from __future__ import annotations

import os
import time
import uuid
from contextlib import contextmanager

from halo_b200 import env
from halo_b200.runtime import ranks
from halo_b200.runtime.collectives import all_gather_object, broadcast_object
from halo_b200.runtime.consensus import RankFailure


def input_is_shared() -> bool:
    return env.env_flag("DIST_INPUT_SHARED_FILESYSTEM", default=ranks.get_num_nodes() == 1)


def output_is_shared() -> bool:
    return env.env_flag("DIST_OUTPUT_SHARED_FILESYSTEM", default=ranks.get_num_nodes() == 1)


def is_writer_rank(shared: bool | None = None) -> bool:
    """Global rank 0 on shared storage, local rank 0 of every node otherwise."""
    shared = output_is_shared() if shared is None else shared
    return ranks.is_global_main_process() if shared else ranks.is_local_main_process()


def probe_shared_directory(directory: str, group=None) -> bool:
    """COLLECTIVE. Rank 0 drops a sentinel; True iff every rank sees it before the probe times out."""
    os.makedirs(directory, exist_ok=True)
    name = broadcast_object(f".halo_probe_{uuid.uuid4().hex}" if ranks.is_global_main_process() else None, 0, group)
    path = os.path.join(directory, name)
    if ranks.is_global_main_process():
        with open(path, "w") as f:
            f.write("probe")
            f.flush()
            os.fsync(f.fileno())
    deadline = time.monotonic() + env.fs_probe_timeout().total_seconds()
    seen = os.path.exists(path)
    while not seen and time.monotonic() < deadline and ranks.get_num_nodes() > 1:
        time.sleep(0.2)
        seen = os.path.exists(path)
    verdicts = all_gather_object(seen, group)
    if ranks.is_global_main_process():
        try:
            os.remove(path)
        except OSError:
            pass
    return all(verdicts)


def verify_filesystem_sharing(directory: str, declared_shared: bool, what: str, group=None) -> None:
    """COLLECTIVE. Refuse a declaration the probe contradicts (silent per-node divergence otherwise)."""
    if ranks.get_num_nodes() <= 1:
        return
    actual = probe_shared_directory(directory, group)
    if declared_shared and not actual:
        raise RankFailure(f"{what} directory {directory!r} was declared shared but some node cannot see rank 0's file")


@contextmanager
def main_first(shared: bool | None = None, group=None):
    """The writer rank(s) run the block first, the others after (e.g. building a cache)."""
    import torch.distributed as dist

    live = dist.is_available() and dist.is_initialized()
    first = is_writer_rank(shared)
    if live and not first:
        dist.barrier(group)
    try:
        yield first
    finally:
        if live and first:
            dist.barrier(group)
