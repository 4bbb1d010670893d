"""Is a path on storage every node sees, or per node? Which rank writes, which rank fills a cache, and who waits for
whom? (the role of halo/runtime/filesystem.py).

``DIST_SHARED_FILESYSTEM`` declares both sides at once, ``DIST_INPUT_SHARED_FILESYSTEM`` (downloads, dataset caches)
and ``DIST_OUTPUT_SHARED_FILESYSTEM`` (checkpoints, logs) each side; a single-node job defaults to shared. The three
flags choose the scope of every main-first wait, so ranks must agree on them: :func:`resolve_consensus` makes rank 0's
values the job's. A sentinel-file probe checks the declaration against what the mounts do on multi-node jobs, in both
directions (declared shared but not visible everywhere; declared per node but visible everywhere)."""

from __future__ import annotations

import logging
import os
import time
import uuid
from contextlib import contextmanager
from datetime import timedelta

from halo_b200 import env
from halo_b200.runtime import ranks
from halo_b200.runtime.collectives import all_gather_object, broadcast_object
from halo_b200.runtime.consensus import RankFailure, StorePhase, barrier_on_exit, default_store

log = logging.getLogger(__name__)

_UMBRELLA, _INPUT, _OUTPUT = "DIST_SHARED_FILESYSTEM", "DIST_INPUT_SHARED_FILESYSTEM", "DIST_OUTPUT_SHARED_FILESYSTEM"
_agreed: dict[str, bool] | None = None       # the job-wide values once resolve_consensus has run


def _local_flags() -> dict[str, bool]:
    umbrella = env.env_flag(_UMBRELLA, default=ranks.get_num_nodes() == 1)
    return {_UMBRELLA: umbrella, _INPUT: env.env_flag(_INPUT, default=umbrella), _OUTPUT: env.env_flag(_OUTPUT, default=umbrella)}


def _flag(name: str) -> bool:
    return (_agreed if _agreed is not None else _local_flags())[name]


def input_is_shared() -> bool:
    return _flag(_INPUT)


def output_is_shared() -> bool:
    return _flag(_OUTPUT)


def resolve_consensus(group=None) -> dict[str, bool]:
    """COLLECTIVE. Agree on the three flags: rank 0's values win, and a rank whose own environment says otherwise warns
    (a per-node override is the usual cause). Ranks that disagreed would wait for each other in different scopes."""
    global _agreed
    local = _local_flags()
    agreed = broadcast_object(local, 0, group)
    differing = sorted(k for k in agreed if agreed[k] != local[k])
    if differing:
        log.warning("shared-filesystem flags differ from rank 0's on this rank (%s): rank 0's values are used; fix the launch "
                    "environment", ", ".join(f"{k}: here {local[k]}, rank 0 {agreed[k]}" for k in differing))
    _agreed = dict(agreed)
    if ranks.is_global_main_process():
        log.info("filesystem scope: %s", {k: ("shared" if v else "per-node") for k, v in agreed.items()})
    return _agreed


def forget_consensus() -> None:
    """Back to this process's own environment (tests; a job that re-initialises its process group)."""
    global _agreed
    _agreed = None


def is_writer_rank(shared: bool | None = None) -> bool:
    """Global rank 0 on shared storage, local rank 0 of every node otherwise."""
    shared = output_is_shared() if shared is None else shared
    return ranks.is_global_main_process() if shared else ranks.is_local_main_process()


def is_load_rank() -> bool:
    """The rank that does shared read-side work (downloads, cache fills) for its scope."""
    return ranks.is_global_main_process() if input_is_shared() else ranks.is_local_main_process()


def makedirs_on_writer(path: str, group=None, writer: bool | None = None) -> None:
    """COLLECTIVE. The writer rank(s) create ``path``; every rank leaves together, and a failure to create it raises
    on every rank rather than on the writer alone."""
    with barrier_on_exit(group):
        if is_writer_rank() if writer is None else writer:
            os.makedirs(path, exist_ok=True)


@contextmanager
def main_first_by_store(tag: str, store=None, timeout: timedelta | None = None):
    """The load rank of each scope (global rank 0 on shared input storage, local rank 0 of each node otherwise) runs the
    body first; the others wait on a store key and run it afterwards (finding the cache filled). The wait is a store
    wait, not a collective, so it may outlast the collective watchdog (a download, a dataset pack); in exchange the body
    must issue no collective. ``tag`` names the call site; each tag is used once per job. A body that raises on the
    first rank releases the waiters with its error."""
    store = store if store is not None else default_store()
    if store is None:
        yield True
        return
    if input_is_shared():
        scope, me, first = "shared", ranks.get_global_rank(), ranks.is_global_main_process()
    else:
        scope, me, first = f"node{ranks.get_node_rank()}", ranks.get_local_rank(), ranks.is_local_main_process()
    phase = StorePhase(store, f"main_first/{tag}/{scope}", 1, 0, timeout)
    if first:
        try:
            yield True
        except BaseException as e:
            phase.fail(f"{type(e).__name__}: {e}")
            raise
        phase.arrive()
    else:
        phase.wait_all()
        yield False


def contradiction(side: str, directory: str, declared_shared: bool, seen: list[bool]) -> str | None:
    """Why the declared sharing of ``side`` ("input" / "output") contradicts ``seen`` (per rank: did it see rank 0's
    sentinel in ``directory``), or None when the declaration holds."""
    if not seen:
        return None
    flag = _INPUT if side == "input" else _OUTPUT
    if not seen[0]:
        return (f"{side} filesystem probe: rank 0 could not read back the file it just wrote in {directory!r}; check the "
                "mount, its permissions and its free space")
    observed = all(seen)
    if observed == declared_shared:
        return None
    if declared_shared:
        blind = [r for r, ok in enumerate(seen) if not ok]
        return (f"{side} filesystem is declared shared, but {len(blind)} of {len(seen)} ranks (first: rank {blind[0]}) "
                f"cannot see a file rank 0 wrote in {directory!r}. If the mount's attribute cache outlasts the probe, raise "
                f"DIST_FS_PROBE_TIMEOUT_SECONDS; otherwise set {flag}=0 so that every node keeps its own copy")
    return (f"{side} filesystem is declared per-node, but all {len(seen)} ranks see a file rank 0 wrote in {directory!r}: "
            f"the nodes would write the same files at the same time. Set {flag}=1")


def sentinel_visibility(directory: str, group=None) -> list[bool]:
    """COLLECTIVE. Rank 0 drops a sentinel in ``directory``; per rank, whether it saw the file before the probe timed
    out (ranks of rank 0's node see it at once; the others poll)."""
    if ranks.is_global_main_process():
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
    return list(verdicts)


def probe_shared_directory(directory: str, group=None) -> bool:
    """COLLECTIVE. True iff every rank sees a file rank 0 writes in ``directory``."""
    return all(sentinel_visibility(directory, group))


def verify_filesystem_sharing(directory: str, declared_shared: bool, what: str, group=None) -> None:
    """COLLECTIVE. Refuse a declaration the probe contradicts, in either direction (declared shared on per-node disks:
    silent divergence; declared per-node on a shared mount: every node writes the same files). Single-node jobs skip it."""
    if ranks.get_num_nodes() <= 1:
        return
    why = contradiction(what, directory, declared_shared, sentinel_visibility(directory, group))
    if why:
        raise RankFailure(why)


def verify_job_directories(output_dir: str | None, input_caches: dict[str, str] | None = None, group=None) -> None:
    """COLLECTIVE. The start-up check of a multi-node job: the output directory against the output declaration, every
    named input cache against the input declaration."""
    if output_dir:
        verify_filesystem_sharing(output_dir, output_is_shared(), "output", group)
    for _, path in sorted((input_caches or {}).items()):
        verify_filesystem_sharing(path, input_is_shared(), "input", group)


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
