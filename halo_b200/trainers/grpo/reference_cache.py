"""Memory-mapped ragged cache of reference-policy log-probs for offline GRPO: the frozen reference scores every
completion once at run start, the training loop then reads rows by index without keeping the reference model
resident (halo/trainers/grpo/offline/reference.py, reference_cache.py)."""

from __future__ import annotations

import json
import os

import numpy as np

from halo_b200.checkpoint.atomic import atomic_write_json


class ReferenceCache:
    def __init__(self, directory: str):
        self.directory = directory
        meta = json.load(open(os.path.join(directory, "reference_cache.json")))
        if meta.get("version") != 1:
            raise ValueError(f"reference cache {directory!r} has an unknown format")
        self.key = meta["key"]
        self.offsets = np.load(os.path.join(directory, "offsets.npy"))
        self.values = np.memmap(os.path.join(directory, "logps.f32"), dtype=np.float32, mode="r", shape=(int(self.offsets[-1]),))

    def __len__(self) -> int:
        return len(self.offsets) - 1

    def __getitem__(self, i: int) -> np.ndarray:
        return np.asarray(self.values[self.offsets[i]:self.offsets[i + 1]])

    @staticmethod
    def exists(directory: str, key: str) -> bool:
        p = os.path.join(directory, "reference_cache.json")
        return os.path.isfile(p) and json.load(open(p)).get("key") == key

    @staticmethod
    def build(directory: str, key: str, rows) -> "ReferenceCache":
        """``rows``: iterable of 1-D float arrays (one per completion, in dataset order). The metadata is written
        last, so a cache whose build was interrupted is rebuilt."""
        os.makedirs(directory, exist_ok=True)
        offsets = [0]
        with open(os.path.join(directory, "logps.f32"), "wb") as f:
            for r in rows:
                a = np.asarray(r, dtype=np.float32).reshape(-1)
                a.tofile(f)
                offsets.append(offsets[-1] + a.size)
        np.save(os.path.join(directory, "offsets.npy"), np.asarray(offsets, dtype=np.int64))
        atomic_write_json(os.path.join(directory, "reference_cache.json"), {"version": 1, "key": key, "rows": len(offsets) - 1})
        return ReferenceCache(directory)
