"""At most N ranks of a node read weights from disk at once (host RAM and page cache are per node).
Default: half the node, capped at 4; 0 means no limit (the role of halo/runtime/load_coordination.py)."""

from __future__ import annotations

from contextlib import contextmanager

import torch.distributed as dist

from halo_b200.runtime import ranks


def default_concurrency(local_world: int) -> int:
    return max(1, min(4, local_world // 2))


def loading_waves(local_world: int, max_concurrent: int | None) -> list[list[int]]:
    """Local ranks grouped into the waves in which they load."""
    n = default_concurrency(local_world) if max_concurrent is None else (max_concurrent or local_world)
    n = max(1, min(n, local_world))
    return [list(range(s, min(local_world, s + n))) for s in range(0, local_world, n)]


@contextmanager
def throttled_load_within_node(max_concurrent: int | None = None, group=None):
    """COLLECTIVE over the default group: enter the block wave by wave."""
    local_world = ranks.get_local_world_size()
    waves = loading_waves(local_world, max_concurrent)
    live = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    my_wave = next(i for i, w in enumerate(waves) if ranks.get_local_rank() % local_world in w)
    if not live:
        yield
        return
    for i in range(len(waves)):
        if i == my_wave:
            yield
        dist.barrier(group)
