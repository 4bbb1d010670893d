"""Checks that run before a save starts (halo/checkpoint/parallel/disk_budget.py): is there room for the
checkpoint, and for the temporary second copy an atomic publish needs, on the filesystem of the output directory."""

from __future__ import annotations

import os
import shutil


def checkpoint_bytes(model, save_dtype_bytes: int | None = None, with_optimizer: bool = True, ep_world: int = 1) -> int:
    """Bytes one checkpoint writes: every parameter once (expert banks counted for all ranks), plus two moments per
    parameter when the optimizer state is saved."""
    total = 0
    for p in model.parameters():
        n = p.numel() * (ep_world if getattr(p, "is_expert", False) else 1)
        size = save_dtype_bytes or p.element_size()
        total += n * size
        if with_optimizer and p.requires_grad:
            total += 2 * n * p.element_size()
    return total


def require_free_space(directory: str, need_bytes: int, safety: float = 1.1) -> int:
    """Raises ``OSError`` with the numbers when the filesystem holding ``directory`` has less than
    ``safety * need_bytes`` free. Returns the free bytes."""
    probe = directory
    while not os.path.isdir(probe):
        parent = os.path.dirname(probe.rstrip("/")) or "."
        if parent == probe:
            break
        probe = parent
    free = shutil.disk_usage(probe).free
    if free < safety * need_bytes:
        raise OSError(f"saving to {directory!r} needs about {need_bytes / 2**30:.1f} GiB (x{safety} safety) but only "
                      f"{free / 2**30:.1f} GiB are free")
    return free
