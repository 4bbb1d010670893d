"""Every "raise on all ranks or on none" seam (the role of halo/runtime/consensus.py:126-440).

A failure that only one rank sees (a full disk, a bad local file, an out-of-memory in a gather)
must not leave the others waiting in the next collective until the watchdog fires. These helpers
turn a one-rank verdict into the same exception everywhere, and provide store-based joins for
waits that legitimately outlast the collective watchdog.
"""

from __future__ import annotations

import time
from contextlib import contextmanager
from datetime import timedelta

import torch.distributed as dist

from halo_b200 import env
from halo_b200.runtime.collectives import _live, all_gather_object


class RankFailure(RuntimeError):
    """Raised on every rank when at least one rank reported a failure."""


def gather_reasons(reason: str | None, group=None) -> list[tuple[int, str]]:
    reasons = all_gather_object(reason, group)
    return [(i, r) for i, r in enumerate(reasons) if r]


def reject_across_ranks(reason: str | None, group=None, what: str = "configuration") -> None:
    """COLLECTIVE. ``reason`` is this rank's complaint or None; raises the union everywhere."""
    bad = gather_reasons(reason, group)
    if bad:
        lines = "; ".join(f"rank {i}: {r}" for i, r in bad[:8])
        more = f" (+{len(bad) - 8} more)" if len(bad) > 8 else ""
        raise RankFailure(f"{what} rejected on {len(bad)} rank(s): {lines}{more}")


def rank_consensus(flag: bool, mode: str = "all", group=None) -> bool:
    """COLLECTIVE. ``all``: True iff every rank says True; ``any``: True iff some rank does."""
    flags = all_gather_object(bool(flag), group)
    return all(flags) if mode == "all" else any(flags)


def rank0_verdict(value, group=None):
    """Rank 0's value on every rank."""
    from halo_b200.runtime.collectives import broadcast_object

    return broadcast_object(value, 0, group)


def assert_rank_uniform(value, what: str, group=None) -> None:
    vals = all_gather_object(value, group)
    if any(v != vals[0] for v in vals):
        shown = ", ".join(f"rank {i}: {v!r}" for i, v in enumerate(vals[:8]))
        raise RankFailure(f"{what} differs across ranks: {shown}")


def reject_divergent_settings(settings: dict, group=None) -> None:
    vals = all_gather_object(settings, group)
    for key in settings:
        seen = {repr(v.get(key)) for v in vals}
        if len(seen) > 1:
            raise RankFailure(f"setting {key!r} differs across ranks: {sorted(seen)}")


def reject_divergent_environment(group=None) -> None:
    """COLLECTIVE. The start-up check over the environment catalogue: a knob that picks a kernel form, a timeout or a
    coordination scope must read the same on every rank (a per-node override would make ranks take different code
    paths into the same collective). Names every differing knob with the ranks' values."""
    from halo_b200 import env

    mine = env.rank_uniform_snapshot()
    every = all_gather_object(mine, group)
    bad = []
    for name in mine:
        seen = [v.get(name) for v in every]
        if len({repr(x) for x in seen}) > 1:
            by_value: dict[str, list[int]] = {}
            for r, x in enumerate(seen):
                by_value.setdefault("unset" if x is None else repr(x), []).append(r)
            bad.append(f"{name}: " + ", ".join(f"{v} on ranks {rs}" for v, rs in sorted(by_value.items())))
    if bad:
        raise RankFailure("environment knobs differ across ranks: " + "; ".join(bad))


class DeferredRankFailure:
    """Collect a local exception inside a block that contains collectives, keep participating, and
    raise everywhere at the end::

        guard = DeferredRankFailure()
        with guard.catch():
            write_my_file()          # may raise on one rank only
        guard.raise_if_any(group)     # COLLECTIVE
    """

    def __init__(self):
        self.error: BaseException | None = None

    @contextmanager
    def catch(self):
        try:
            yield
        except Exception as exc:  # noqa: BLE001 - the point is to defer any failure
            if self.error is None:
                self.error = exc

    def raise_if_any(self, group=None, what: str = "a rank failed") -> None:
        reason = f"{type(self.error).__name__}: {self.error}" if self.error else None
        bad = gather_reasons(reason, group)
        if bad:
            lines = "; ".join(f"rank {i}: {r}" for i, r in bad[:8])
            raise RankFailure(f"{what}: {lines}") from self.error


@contextmanager
def barrier_on_exit(group=None):
    """Leave the block together; a rank that raised still lets its peers out before re-raising."""
    guard = DeferredRankFailure()
    with guard.catch():
        yield
    guard.raise_if_any(group)


class StorePhase:
    """Join through the c10d store for waits longer than the collective watchdog (a rank downloading
    or packing a dataset). ``arrive()`` then ``wait_all()``; each phase name is used once."""

    def __init__(self, store, name: str, world_size: int, rank: int, timeout: timedelta | None = None,
                 poll_seconds: float = 0.05):
        self.store, self.name, self.world, self.rank = store, name, world_size, rank
        self.timeout = timeout or env.store_timeout()
        self.poll = poll_seconds

    def _key(self, rank: int) -> str:
        return f"halo/phase/{self.name}/{rank}"

    def arrive(self, payload: str = "ok") -> None:
        self.store.set(self._key(self.rank), payload)

    def wait_all(self) -> list[str]:
        deadline = time.monotonic() + self.timeout.total_seconds()
        out = []
        for r in range(self.world):
            key = self._key(r)
            while True:
                try:
                    if self.store.check([key]):
                        out.append(self.store.get(key).decode())
                        break
                except RuntimeError:
                    pass
                if time.monotonic() > deadline:
                    raise RankFailure(f"rank {r} never reached phase {self.name!r} within {self.timeout}")
                time.sleep(self.poll)
        failed = [(r, p) for r, p in enumerate(out) if p.startswith("error:")]
        if failed:
            raise RankFailure("; ".join(f"rank {r}: {p[6:]}" for r, p in failed))
        return out

    def fail(self, reason: str) -> None:
        self.arrive("error:" + reason)


def default_store():
    if _live():
        return dist.distributed_c10d._get_default_store()
    return None
