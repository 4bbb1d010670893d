"""The weight-sync group of one box: trainer ranks push a full bf16 copy of the model into buffers
held by the rollout ranks.

``ResidentCopySync`` is the single-node form used when trainer and rollout GPUs share an NVSwitch
domain: the rollout ranks expose one symmetric-memory arena, the forwarding trainer rank packs
chunks and stores each chunk into every rollout GPU's arena with one kernel (one read of the local
weights, one NVLink store per destination) - no collective library call carries the payload.
Expert banks are gathered to the forwarding rank one layer ahead of the send.
``BroadcastSync`` is the portable fallback over a process-group broadcast (what the reference does
with packed NCCL broadcasts, halo/weight_sync/transport/pynccl.py:68-146).
Both bound their waits and report a failed peer as an exception rather than a hang.
"""

from __future__ import annotations

import time

import torch
import torch.distributed as dist

from halo_b200 import env
from halo_b200.ops import _lib
from halo_b200.runtime.bounded_waits import bounded_event_wait

from .chunking import manifest_of, pack_chunk, plan_chunks, unpack_chunk


def full_named_tensors(model, ep_group=None):
    """Yield (hub-independent runtime name, full tensor) with expert banks gathered over the EP group."""
    tr = getattr(model, "transport", None)
    n_ep = getattr(tr, "n_ranks", 1) if tr is not None else 1
    for name, p in model.named_parameters():
        t = p.detach()
        if getattr(p, "is_expert", False) and n_ep > 1:
            out = torch.empty((n_ep * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
            dist.all_gather_into_tensor(out, t.contiguous(), group=ep_group)
            t = out
        yield name, t


class ResidentCopySync:
    """All ranks of ``group`` call the constructor; ``rollout_ranks`` receive, ``src_rank`` sends."""

    def __init__(self, group, device, manifest, src_rank: int, rollout_ranks: list[int], chunk_bytes: int | None = None):
        import torch.distributed._symmetric_memory as symm

        self.group, self.device = group, torch.device(device)
        self.rank = dist.get_rank(group)
        self.src_rank, self.rollout_ranks = src_rank, list(rollout_ranks)
        self.slots, self.sizes = plan_chunks(manifest, chunk_bytes or env.weight_sync_chunk_bytes())
        self.chunk_base = [0]
        for s in self.sizes:
            self.chunk_base.append(self.chunk_base[-1] + s)
        self.arena = symm.empty((max(self.chunk_base[-1], 256),), dtype=torch.uint8, device=self.device)
        self.handle = symm.rendezvous(self.arena, group)
        ptrs = list(self.handle.buffer_ptrs)
        self._dst = (_lib.c_void_p * len(self.rollout_ranks))(*[ptrs[r] for r in self.rollout_ranks])
        # NVLS: when the arena is bound to an NVLink multicast object, one multimem.st per 16 bytes reaches every rank of
        # the group (the rollout copies and, harmlessly, the other trainers' arenas), so the sender's links carry the
        # weights once however many rollout GPUs listen
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self._mc = mc if (mc and env.weight_sync_nvls() and len(self.rollout_ranks) > 1) else 0
        self.staging = (torch.empty(max(self.sizes or [256]), dtype=torch.uint8, device=self.device)
                        if self.rank == src_rank else None)
        self.last_seconds = 0.0
        self.bytes_per_push = self.chunk_base[-1]

    def push(self, tensors: dict | None) -> None:
        """COLLECTIVE over the group. The sender passes {name: full tensor}; the others pass None."""
        self.handle.barrier(channel=1)          # receivers are not reading the arena any more
        t0 = time.perf_counter()
        if self.rank == self.src_rank:
            L = _lib.lib()
            for c, size in enumerate(self.sizes):
                pack_chunk(self.slots, c, tensors, self.staging)
                if self._mc:
                    rc = L.halo_broadcast_bytes_mc(_lib.ptr(self.staging), _lib.c_void_p(self._mc), _lib.c_ll(self.chunk_base[c]),
                                                   _lib.c_ll((size + 15) // 16 * 16), _lib.stream_ptr(self.device))
                    _lib.check(rc, "halo_broadcast_bytes_mc")
                    continue
                rc = L.halo_broadcast_bytes(_lib.ptr(self.staging), self._dst, _lib.c_int(len(self.rollout_ranks)),
                                            _lib.c_ll(self.chunk_base[c]), _lib.c_ll((size + 15) // 16 * 16),
                                            _lib.stream_ptr(self.device))
                _lib.check(rc, "halo_broadcast_bytes")
            ev = torch.cuda.Event()
            ev.record()
            bounded_event_wait(ev, what="weight push")
        self.handle.barrier(channel=1)          # every store has landed
        self.last_seconds = time.perf_counter() - t0

    def receive_into(self, named_params: dict) -> None:
        """On a rollout rank: copy the arena's tensors into the serving copy."""
        for c in range(len(self.sizes)):
            view = self.arena[self.chunk_base[c]:self.chunk_base[c] + self.sizes[c]]
            unpack_chunk(self.slots, c, view, named_params)


class ShardedCopySync:
    """Every trainer pushes the weights it holds, nobody gathers. The rollout ranks' arena is laid out for the FULL
    tensors (expert banks with all experts); trainer t stores its expert slice at the slice's offset inside the bank and
    its share of the replicated tensors (dealt round-robin over the trainers) whole, each with one kernel that reads the
    parameter memory once and stores to every rollout GPU over NVLink. With T trainers and R rollout GPUs every trainer
    sends 1/T of the model R times and every rollout GPU receives the model once, so all links are busy for
    (model bytes) / (link bandwidth): the floor of a full copy per rollout GPU.

    All ranks of ``group`` call the constructor with the same ``full_manifest`` ((name, full shape, dtype) in one
    order). Counterpart of the reference's sharded weight-update streams (halo/weight_sync/update_stream.py,
    halo/trainers/grpo/rollout/weight_push.py), without their gather to one sender."""

    def __init__(self, group, device, full_manifest, trainer_ranks: list[int], rollout_ranks: list[int]):
        import torch.distributed._symmetric_memory as symm

        self.group, self.device = group, torch.device(device)
        self.rank = dist.get_rank(group)
        self.trainer_ranks, self.rollout_ranks = list(trainer_ranks), list(rollout_ranks)
        self.slots, sizes = plan_chunks(full_manifest, 1 << 62)           # one chunk: offsets inside one arena
        self.offset = {s.name: s.offset for s in self.slots}
        self.nbytes = {s.name: s.nbytes for s in self.slots}
        self.total = sizes[0] if sizes else 256
        self.arena = symm.empty((max(self.total, 256),), dtype=torch.uint8, device=self.device)
        self.handle = symm.rendezvous(self.arena, group)
        ptrs = list(self.handle.buffer_ptrs)
        self._dst = (_lib.c_void_p * len(self.rollout_ranks))(*[ptrs[r] for r in self.rollout_ranks])
        self.last_seconds = 0.0
        self.bytes_sent = 0

    def owner_of_replicated(self, index: int) -> int:
        """Trainer (position in ``trainer_ranks``) that sends the ``index``-th replicated tensor."""
        return index % len(self.trainer_ranks)

    def push(self, pieces) -> None:
        """COLLECTIVE over the group. A trainer passes ``[(name, tensor, first_row)]``: ``tensor`` holds rows
        ``[first_row, first_row + tensor.shape[0])`` of the full tensor ``name`` (``first_row = 0`` and the whole tensor
        for a replicated one); the rollout ranks pass an empty list."""
        self.handle.barrier(channel=1)          # receivers are not reading the arena any more
        L = _lib.lib()
        self.bytes_sent = 0
        for name, t, first_row in pieces:
            t = t.detach()
            if not t.is_contiguous():
                t = t.contiguous()
            row_bytes = t[0].numel() * t.element_size() if t.dim() > 0 and t.shape[0] > 0 else t.element_size()
            n = t.numel() * t.element_size()
            off = self.offset[name] + first_row * row_bytes
            if off % 16 or n % 16:
                raise ValueError(f"{name}: a piece of {n} bytes at offset {off} is not 16-byte aligned")
            if off + n > self.offset[name] + (self.nbytes[name] + 255) // 256 * 256:
                raise ValueError(f"{name}: the piece runs past its tensor in the arena")
            rc = L.halo_broadcast_bytes(_lib.ptr(t), self._dst, _lib.c_int(len(self.rollout_ranks)), _lib.c_ll(off), _lib.c_ll(n),
                                        _lib.stream_ptr(self.device))
            _lib.check(rc, "halo_broadcast_bytes")
            self.bytes_sent += n
        if pieces:
            ev = torch.cuda.Event()
            ev.record()
            bounded_event_wait(ev, what="weight push")
        self.handle.barrier(channel=1)          # every store has landed

    def view(self, name: str, shape, dtype) -> torch.Tensor:
        """On a rollout rank: the full tensor ``name`` inside the arena (no copy)."""
        n = self.nbytes[name]
        return self.arena[self.offset[name]:self.offset[name] + n].view(dtype).view(shape)


class BroadcastSync:
    """Portable path: packed chunks broadcast from ``src_rank`` over a process group."""

    def __init__(self, group, device, manifest, src_rank: int, chunk_bytes: int | None = None):
        self.group, self.device, self.src_rank = group, torch.device(device), src_rank
        self.rank = dist.get_rank(group)
        self.slots, self.sizes = plan_chunks(manifest, chunk_bytes or env.weight_sync_chunk_bytes())
        self.staging = torch.empty(max(self.sizes or [256]), dtype=torch.uint8, device=self.device)

    def push(self, tensors: dict | None, into: dict | None = None) -> None:
        src = dist.get_global_rank(self.group, self.src_rank) if self.group is not None else self.src_rank
        for c, size in enumerate(self.sizes):
            buf = self.staging[:size]
            if self.rank == self.src_rank:
                pack_chunk(self.slots, c, tensors, buf)
            dist.broadcast(buf, src=src, group=self.group)
            if self.rank != self.src_rank and into is not None:
                unpack_chunk(self.slots, c, buf, into)


def build_manifest(model) -> list:
    return manifest_of((n, p) for n, p in model.named_parameters())


def full_manifest(model, n_ep: int | None = None) -> list:
    """Manifest of the gathered (unsharded) tensors of an expert-parallel model, without gathering them."""
    tr = getattr(model, "transport", None)
    n_ep = n_ep if n_ep is not None else (getattr(tr, "n_ranks", 1) if tr is not None else 1)

    class _Shape:
        def __init__(self, shape, dtype):
            self.shape, self.dtype = torch.Size(shape), dtype

        def numel(self):
            return self.shape.numel()

        def element_size(self):
            return torch.empty((), dtype=self.dtype).element_size()

    out = []
    for n, p in model.named_parameters():
        shape = tuple(p.shape)
        if getattr(p, "is_expert", False) and n_ep > 1:
            shape = (n_ep * shape[0],) + shape[1:]
        out.append((n, _Shape(shape, p.dtype)))
    return manifest_of(out)
