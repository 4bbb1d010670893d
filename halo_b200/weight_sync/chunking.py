"""Pack named tensors into fixed-size byte chunks (default 1 GiB, ``HALO_WEIGHT_SYNC_CHUNK_MB``) so a
sync is a handful of large transfers rather than one per tensor (halo/weight_sync/update_stream.py,
halo/weight_sync/transport/packed_broadcast.py:12-74). The layout is deterministic: sender and
receiver derive the same offsets from the same (name, shape, dtype) manifest."""

from __future__ import annotations

from dataclasses import dataclass

import torch

ALIGN = 256


@dataclass(frozen=True)
class Slot:
    name: str
    shape: tuple
    dtype: torch.dtype
    chunk: int
    offset: int      # bytes inside the chunk
    nbytes: int


def manifest_of(named_tensors) -> list[tuple[str, tuple, torch.dtype]]:
    return [(n, tuple(t.shape), t.dtype) for n, t in named_tensors]


def plan_chunks(manifest, chunk_bytes: int) -> tuple[list[Slot], list[int]]:
    """Greedy fill in manifest order; a tensor larger than a chunk gets a chunk of its own size.
    Returns (slots, size of every chunk in bytes)."""
    slots, sizes, cur, used = [], [], 0, 0
    for name, shape, dtype in manifest:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        padded = (nbytes + ALIGN - 1) // ALIGN * ALIGN
        if used and used + padded > chunk_bytes:
            sizes.append(used)
            cur, used = cur + 1, 0
        slots.append(Slot(name, shape, dtype, cur, used, nbytes))
        used += padded
    if used:
        sizes.append(used)
    return slots, sizes


def pack_chunk(slots: list[Slot], chunk: int, tensors: dict, out: torch.Tensor) -> None:
    """Copy the tensors of ``chunk`` into the uint8 staging buffer ``out``."""
    for s in slots:
        if s.chunk == chunk:
            out[s.offset:s.offset + s.nbytes].copy_(tensors[s.name].detach().contiguous().view(-1).view(torch.uint8))


def unpack_chunk(slots: list[Slot], chunk: int, buf: torch.Tensor, into: dict) -> None:
    for s in slots:
        if s.chunk == chunk:
            into[s.name].view(-1).view(torch.uint8).copy_(buf[s.offset:s.offset + s.nbytes])
