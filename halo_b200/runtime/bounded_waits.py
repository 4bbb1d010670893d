"""Host waits on device work with a deadline (the role of
halo/weight_sync/transport/bounded_waits.py:25-51): poll a CUDA event instead of blocking in a
synchronise that a wedged peer would turn into a hang, and raise when the deadline passes so the
caller can abort its communicator and surface the failure on every rank."""

from __future__ import annotations

import time

from halo_b200 import env


class WaitExpired(TimeoutError):
    pass


def bounded_event_wait(event, timeout_seconds: float | None = None, poll_seconds: float = 0.001, what: str = "device work"):
    """``event``: anything with ``query() -> bool`` (a ``torch.cuda.Event``)."""
    if timeout_seconds is None:
        timeout_seconds = float(env.env_positive_int("HALO_BOUNDED_WAIT_SECONDS", 600))
    deadline = time.monotonic() + timeout_seconds
    while not event.query():
        if time.monotonic() > deadline:
            raise WaitExpired(f"{what} did not finish within {timeout_seconds:.0f} s")
        time.sleep(poll_seconds)


def bounded_stream_sync(stream, timeout_seconds: float | None = None, what: str = "stream"):
    import torch

    ev = torch.cuda.Event()
    ev.record(stream)
    bounded_event_wait(ev, timeout_seconds, what=what)
