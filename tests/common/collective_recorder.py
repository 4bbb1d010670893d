"""Record the collectives a rank enters, in order: every ``torch.distributed`` entry point used by the framework is
wrapped so that a call appends ``(name, ranks in the group, elements)`` to a trace before running for real. Traces of
different ranks (and of successive steps) can then be compared: a rank-uniform program enters the same collectives in
the same order everywhere."""

from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist

NAMES = ("all_reduce", "all_gather_into_tensor", "all_gather", "all_gather_object", "reduce_scatter_tensor", "all_to_all_single",
         "all_to_all", "broadcast", "broadcast_object_list", "barrier", "send", "recv", "isend", "irecv", "reduce", "gather")


def _numel(args):
    for a in args:
        if isinstance(a, torch.Tensor):
            return int(a.numel())
        if isinstance(a, (list, tuple)) and a and isinstance(a[0], torch.Tensor):
            return int(sum(t.numel() for t in a))
    return 0


@contextlib.contextmanager
def recording():
    trace: list[tuple] = []
    originals = {}

    def wrap(name, fn):
        def recorded(*args, **kwargs):
            group = kwargs.get("group")
            trace.append((name, dist.get_world_size(group), _numel(args)))
            return fn(*args, **kwargs)

        return recorded

    for name in NAMES:
        if hasattr(dist, name):
            originals[name] = getattr(dist, name)
            setattr(dist, name, wrap(name, originals[name]))
    try:
        yield trace
    finally:
        for name, fn in originals.items():
            setattr(dist, name, fn)
