"""Group construction and the object / tensor collectives the control plane uses (the role of
halo/runtime/collectives.py:41-230). Every function degrades to the single-process answer when
no process group exists, so the same code runs in unit tests."""

from __future__ import annotations

import pickle
from contextlib import contextmanager
from typing import Any, Sequence

import torch
import torch.distributed as dist

from halo_b200 import env

GATHER_WINDOW_BYTES = 64 * 1024 * 1024


def _live(group=None) -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1


def build_groups(rank_lists: Sequence[Sequence[int]], backend: str | None = None):
    """Create every (disjoint) group of one kind; all ranks call this with the same lists in the same
    order. Returns the group this rank belongs to (or None)."""
    mine = None
    me = dist.get_rank()
    for ranks in rank_lists:
        g = dist.new_group(list(ranks), timeout=env.nccl_timeout(), backend=backend)
        if me in ranks:
            mine = g
    return mine


def _device_for(group=None) -> torch.device:
    backend = dist.get_backend(group)
    return torch.device("cuda", torch.cuda.current_device()) if "nccl" in str(backend) else torch.device("cpu")


def all_gather_object(obj: Any, group=None) -> list:
    if not _live(group):
        return [obj]
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, obj, group=group)
    return out


def broadcast_object(obj: Any, src: int = 0, group=None) -> Any:
    if not _live(group):
        return obj
    box = [obj]
    dist.broadcast_object_list(box, src=src, group=group)
    return box[0]


def share_from_leader(produce, group=None) -> Any:
    """COLLECTIVE over ``group``. The group's first rank calls ``produce()``; every rank returns its result (None is a
    result like any other). For ranks that must process identical inputs - the slices of one tensor-parallel replica -
    when each would otherwise draw its own (sampled rollouts, a shuffled batch)."""
    if not _live(group) or dist.get_world_size(group) == 1:
        return produce()
    leader = dist.get_rank(group) == 0
    src = dist.get_global_rank(group, 0) if group is not None else 0
    box = [produce() if leader else None]
    dist.broadcast_object_list(box, src=src, group=group)
    return box[0]


def gather_on_rank0(obj: Any, group=None) -> list | None:
    """Every rank's object on group rank 0 (None elsewhere). Large pickles move in 64 MiB windows as
    a SUM-reduce of byte buffers, which needs no per-peer point-to-point buffers."""
    if not _live(group):
        return [obj]
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    dev = _device_for(group)
    blob = pickle.dumps(obj)
    sizes = torch.zeros(world, dtype=torch.int64, device=dev)
    sizes[rank] = len(blob)
    dist.all_reduce(sizes, group=group)
    sizes = sizes.tolist()
    offsets = [0]
    for s in sizes:
        offsets.append(offsets[-1] + s)
    total = offsets[-1]
    mine = torch.frombuffer(bytearray(blob), dtype=torch.uint8)
    result = bytearray(total) if rank == 0 else None
    root = dist.get_global_rank(group, 0) if group is not None else 0
    for start in range(0, total, GATHER_WINDOW_BYTES):
        end = min(total, start + GATHER_WINDOW_BYTES)
        win = torch.zeros(end - start, dtype=torch.uint8, device=dev)
        lo, hi = max(start, offsets[rank]), min(end, offsets[rank + 1])
        if lo < hi:
            win[lo - start:hi - start] = mine[lo - offsets[rank]:hi - offsets[rank]].to(dev)
        dist.reduce(win, dst=root, group=group)
        if rank == 0:
            result[start:end] = win.cpu().numpy().tobytes()
    if rank != 0:
        return None
    return [pickle.loads(bytes(result[offsets[i]:offsets[i + 1]])) for i in range(world)]


def combine_across_ranks(value: float, op: str = "sum", group=None) -> float:
    if not _live(group):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=_device_for(group))
    dist.all_reduce(t, op={"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[op], group=group)
    return float(t.item())


def all_gather_cat(t: torch.Tensor, group=None, dim: int = 0) -> torch.Tensor:
    """Concatenate equally-shaped tensors of every rank along ``dim``."""
    if not _live(group):
        return t
    world = dist.get_world_size(group)
    t = t.contiguous()
    out = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, t, group=group)
    parts = list(out.unbind(0))
    return torch.cat(parts, dim=dim)


def all_gather_varlen(t: torch.Tensor, group=None) -> list[torch.Tensor]:
    """Rows of every rank when the row counts differ (pads to the longest)."""
    if not _live(group):
        return [t]
    world = dist.get_world_size(group)
    n = torch.tensor([t.shape[0]], dtype=torch.int64, device=t.device)
    counts = torch.empty(world, dtype=torch.int64, device=t.device)
    dist.all_gather_into_tensor(counts, n, group=group)
    counts = counts.tolist()
    longest = max(counts)
    pad = torch.zeros((longest,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    pad[: t.shape[0]] = t
    out = torch.empty((world,) + tuple(pad.shape), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, pad, group=group)
    return [out[i, :c] for i, c in enumerate(counts)]


def gather_cat_to_rank(t: torch.Tensor, dst: int = 0, group=None, dim: int = 0) -> torch.Tensor | None:
    """Like :func:`all_gather_cat` but only group rank ``dst`` keeps the result."""
    if not _live(group):
        return t
    full = all_gather_cat(t, group, dim)
    return full if dist.get_rank(group) == dst else None


def safe_broadcast(t: torch.Tensor, src: int, group=None) -> torch.Tensor:
    """Broadcast any dtype by moving bytes (some backends lack int16 / bool kernels)."""
    if not _live(group):
        return t
    view = t.contiguous().view(torch.uint8)
    dist.broadcast(view, src=src, group=group)
    return view.view(t.dtype).reshape(t.shape)


@contextmanager
def collective_side_stream(device=None):
    """Run collectives on a side stream that is ordered after the current one; the caller joins with
    ``torch.cuda.current_stream().wait_stream(side)``."""
    if not torch.cuda.is_available():
        yield None
        return
    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        yield side
