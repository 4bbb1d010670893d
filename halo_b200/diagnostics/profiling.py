"""torch.profiler schedule helper (wait 5, warm-up 1, active 3, rank 0 by default), CUDA memory
history snapshots and all-thread stack dumps (halo/callbacks/torch_profiler.py:26-134,
halo/diagnostics/py_spy.py)."""

from __future__ import annotations

import faulthandler
import os
import sys

import torch

from halo_b200 import env


def parse_ranks(spec: str, world: int) -> set[int]:
    if spec == "all":
        return set(range(world))
    return {int(x) for x in str(spec).split(",") if x.strip() != ""}


def make_profiler(rank: int, ranks: str = "0", world: int = 1, with_cpu: bool = False, out_dir: str | None = None):
    if rank not in parse_ranks(ranks, world):
        return None
    out_dir = out_dir or env.torch_trace_dir()
    os.makedirs(out_dir, exist_ok=True)
    acts = [torch.profiler.ProfilerActivity.CUDA] if torch.cuda.is_available() else []
    if with_cpu or not acts:
        acts.append(torch.profiler.ProfilerActivity.CPU)
    return torch.profiler.profile(
        activities=acts, schedule=torch.profiler.schedule(wait=5, warmup=1, active=3, repeat=1),
        on_trace_ready=torch.profiler.tensorboard_trace_handler(out_dir, worker_name=f"rank{rank}"))


def start_memory_history(max_entries: int = 100000) -> None:
    if torch.cuda.is_available():
        torch.cuda.memory._record_memory_history(max_entries=max_entries)


def dump_memory_snapshot(path: str) -> None:
    if torch.cuda.is_available():
        torch.cuda.memory._dump_snapshot(path)


def dump_stacks(file=None) -> None:
    """All Python threads' stacks of this process (what a py-spy dump would show)."""
    faulthandler.dump_traceback(file=file or sys.stderr, all_threads=True)


def install_hang_dump(seconds: float) -> None:
    """Dump every thread's stack if the process is still alive after ``seconds`` (repeats)."""
    faulthandler.dump_traceback_later(seconds, repeat=True)
