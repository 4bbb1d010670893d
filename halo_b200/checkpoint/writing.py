"""Streaming SafeTensors shard writer: tensors arrive one by one (already on the host), shards are
cut at a size limit, every file is published atomically and the merged ``model.safetensors.index.json``
is written last (the role of halo/checkpoint/writing.py and halo/checkpoint/parallel/writing.py)."""

from __future__ import annotations

import os

import torch
from safetensors.torch import save_file

from .atomic import atomic_write_json, staged_path

INDEX_NAME = "model.safetensors.index.json"
SINGLE_NAME = "model.safetensors"


class StreamingShardWriter:
    def __init__(self, directory: str, max_shard_bytes: int = 5 * 1024**3, save_dtype: torch.dtype | None = None,
                 prefix: str = "model"):
        """``prefix``: stem of the shard files. Writers that share a directory (pipeline stages) use distinct stems
        and leave the merged index to their leader (``finish(write_index=False)``)."""
        self.directory = directory
        self.prefix = prefix
        self.weight_map: dict[str, str] = {}
        self.max_shard_bytes = max_shard_bytes
        self.save_dtype = save_dtype
        self.pending: dict[str, torch.Tensor] = {}
        self.pending_bytes = 0
        self.shards: list[tuple[str, list[str]]] = []
        self.total_bytes = 0
        os.makedirs(directory, exist_ok=True)

    def add(self, name: str, tensor: torch.Tensor) -> None:
        t = tensor.detach()
        if self.save_dtype is not None and t.is_floating_point():
            t = t.to(self.save_dtype)
        t = t.to("cpu").contiguous().clone()
        nbytes = t.numel() * t.element_size()
        if self.pending and self.pending_bytes + nbytes > self.max_shard_bytes:
            self._flush()
        if name in self.pending or any(name in names for _, names in self.shards):
            raise KeyError(f"tensor {name!r} written twice")
        self.pending[name] = t
        self.pending_bytes += nbytes
        self.total_bytes += nbytes

    def _flush(self) -> None:
        if not self.pending:
            return
        tmp_name = f"{self.prefix}-part-{len(self.shards) + 1:05d}.safetensors"
        with staged_path(os.path.join(self.directory, tmp_name)) as tmp:
            save_file(self.pending, tmp, metadata={"format": "pt"})
        self.shards.append((tmp_name, list(self.pending)))
        self.pending, self.pending_bytes = {}, 0

    def finish(self, write_index: bool = True) -> list[str]:
        """Cut the last shard, give the files their final names and write the index (``self.weight_map`` holds it
        either way). Returns file names."""
        self._flush()
        n = len(self.shards)
        names = []
        if n == 1 and write_index and self.prefix == "model":
            self.weight_map = {t: SINGLE_NAME for t in self.shards[0][1]}
            os.replace(os.path.join(self.directory, self.shards[0][0]), os.path.join(self.directory, SINGLE_NAME))
            names.append(SINGLE_NAME)
            stale = os.path.join(self.directory, INDEX_NAME)
            if os.path.exists(stale):
                os.remove(stale)
            return names
        weight_map = {}
        for i, (tmp_name, tensors) in enumerate(self.shards):
            final = f"{self.prefix}-{i + 1:05d}-of-{n:05d}.safetensors"
            os.replace(os.path.join(self.directory, tmp_name), os.path.join(self.directory, final))
            names.append(final)
            for t in tensors:
                weight_map[t] = final
        self.weight_map = weight_map
        if write_index:
            atomic_write_json(os.path.join(self.directory, INDEX_NAME),
                              {"metadata": {"total_size": self.total_bytes}, "weight_map": weight_map})
        return names
