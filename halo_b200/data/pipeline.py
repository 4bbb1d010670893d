"""Rank-coordinated ``map`` / ``filter`` / ``pack`` over a dataset, with deterministic cache keys.

A pipeline is a source (files of records) and an ordered list of stages. Every stage has a fingerprint - its name, its
parameters and the source text of its function - and the key of a stage's output is the hash of the source's
fingerprint and of every stage fingerprint up to it. So the same files, tokenizer and stages give the same key in every
run and on every rank, a changed stage invalidates exactly what comes after it, and a second run finds its artifacts.

One rank per filesystem scope does the work: global rank 0 when inputs are on storage every node sees, each node's local
rank 0 otherwise (:func:`halo_b200.runtime.filesystem.main_first_by_store`). The others wait on a store key, which may
outlast the collective watchdog, and then read the artifact. A failure of the working rank reaches the waiters by name.
Without a process group the caller is the working rank.

Artifacts are ragged arrays: one ``values`` vector per column and one shared ``offsets`` vector (``.npy`` files, read
memory-mapped), plus a ``.complete`` marker written last.

(The role of halo/data/pipeline/*.py: the coordinated map / filter / pack and its cache keys.)"""

from __future__ import annotations

import hashlib
import inspect
import json
import os
from dataclasses import dataclass, field
from typing import Callable

import numpy as np

from .datasets import list_files, pack_rows, read_records
from .packing import PackedBatch


def _digest(*parts) -> str:
    h = hashlib.sha256()
    for p in parts:
        h.update(json.dumps(p, sort_keys=True, default=str).encode())
        h.update(b"\0")
    return h.hexdigest()[:24]


def source_fingerprint(path: str) -> str:
    """The files of a dataset by name, size and modification time (content hashing a multi-terabyte corpus at every
    start would cost more than the cache saves). Object-store paths fingerprint by their URL."""
    if "://" in path:
        return _digest("url", path)
    files = list_files(path)
    return _digest("files", [(os.path.relpath(f, path) if os.path.isdir(path) else os.path.basename(f), os.path.getsize(f),
                              int(os.path.getmtime(f))) for f in files])


def function_fingerprint(fn: Callable) -> str:
    """A function by its source text (a changed tokenisation rule must not hit the old cache); callables without
    retrievable source fall back to their qualified name."""
    try:
        return _digest(inspect.getsource(fn))
    except (OSError, TypeError):
        return _digest(getattr(fn, "__module__", ""), getattr(fn, "__qualname__", repr(fn)))


@dataclass
class Stage:
    kind: str                     # "map" | "filter" | "pack"
    name: str
    fn: Callable | None = None
    params: dict = field(default_factory=dict)

    def fingerprint(self) -> str:
        return _digest(self.kind, self.name, self.params, function_fingerprint(self.fn) if self.fn else "")


class Ragged:
    """Documents as (tokens, label mask) pairs stored as two value vectors over shared offsets."""

    @staticmethod
    def write(directory: str, docs: list[tuple[np.ndarray, np.ndarray]]) -> None:
        os.makedirs(directory, exist_ok=True)
        lengths = np.fromiter((len(t) for t, _ in docs), dtype=np.int64, count=len(docs))
        offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int64)
        tokens = np.concatenate([np.asarray(t, dtype=np.int32) for t, _ in docs]) if docs else np.zeros(0, np.int32)
        masks = np.concatenate([np.asarray(m, dtype=np.uint8) for _, m in docs]) if docs else np.zeros(0, np.uint8)
        np.save(os.path.join(directory, "offsets.npy"), offsets)
        np.save(os.path.join(directory, "tokens.npy"), tokens)
        np.save(os.path.join(directory, "masks.npy"), masks)

    @staticmethod
    def read(directory: str) -> list[tuple[np.ndarray, np.ndarray]]:
        offsets = np.load(os.path.join(directory, "offsets.npy"))
        tokens = np.load(os.path.join(directory, "tokens.npy"), mmap_mode="r")
        masks = np.load(os.path.join(directory, "masks.npy"), mmap_mode="r")
        # the types the tokenising functions return, so that cached and freshly computed documents pack identically
        return [(np.asarray(tokens[a:b], dtype=np.int64), np.asarray(masks[a:b]).astype(bool)) for a, b in zip(offsets[:-1], offsets[1:])]


class Pipeline:
    """``Pipeline(path, cache_dir).map(tokenize, "tokenize", tokenizer="name").filter(...).pack(8192).rows()``."""

    def __init__(self, dataset_path: str, cache_dir: str, store=None, timeout=None):
        self.path, self.cache_dir, self.store, self.timeout = dataset_path, cache_dir, store, timeout
        self.stages: list[Stage] = []
        self.built: list[str] = []          # stage names this process computed (the rest came from the cache)

    # ---- building ------------------------------------------------------------------------------
    def map(self, fn: Callable, name: str, **params) -> "Pipeline":
        """``fn(record) -> (tokens, label_mask)`` for the first map (records in), ``fn(tokens, mask) -> (tokens, mask)``
        for later ones."""
        self.stages.append(Stage("map", name, fn, params))
        return self

    def filter(self, fn: Callable, name: str, **params) -> "Pipeline":
        """``fn(tokens, mask) -> bool``; documents answering False are dropped (and counted in the stage's report)."""
        self.stages.append(Stage("filter", name, fn, params))
        return self

    def pack(self, row_len: int, strategy: str = "sequential", completion_only: bool = False, shuffle_seed: int | None = 0) -> "Pipeline":
        self.stages.append(Stage("pack", "pack", None, {"row_len": row_len, "strategy": strategy, "completion_only": completion_only,
                                                        "shuffle_seed": shuffle_seed}))
        return self

    # ---- keys ----------------------------------------------------------------------------------
    def keys(self) -> list[str]:
        """The cache key after each stage, in order."""
        out, running = [], source_fingerprint(self.path)
        for s in self.stages:
            running = _digest(running, s.fingerprint())
            out.append(running)
        return out

    def _dir(self, key: str) -> str:
        return os.path.join(self.cache_dir, key)

    def _complete(self, key: str) -> bool:
        return os.path.isfile(os.path.join(self._dir(key), ".complete"))

    # ---- running -------------------------------------------------------------------------------
    def _compute(self) -> None:
        """Runs on the working rank only: the stages after the last complete artifact, each written and marked."""
        keys = self.keys()
        start = max((i + 1 for i, k in enumerate(keys) if self._complete(k)), default=0)
        docs = Ragged.read(self._dir(keys[start - 1])) if start and self.stages[start - 1].kind != "pack" else None
        first_map_done = any(s.kind == "map" for s in self.stages[:start])
        for i in range(start, len(self.stages)):
            s, directory = self.stages[i], self._dir(keys[i])
            report = {"stage": s.name, "kind": s.kind}
            if s.kind == "map":
                if not first_map_done:
                    docs = [s.fn(rec) for rec in read_records(self.path)]
                    first_map_done = True
                else:
                    docs = [s.fn(t, m) for t, m in docs]
                docs = [(np.asarray(t, dtype=np.int64), np.asarray(m, dtype=bool)) for t, m in docs]
                Ragged.write(directory, docs)
            elif s.kind == "filter":
                if docs is None:
                    raise ValueError(f"filter {s.name!r} needs a map before it (records have no tokens yet)")
                kept = [(t, m) for t, m in docs if s.fn(t, m)]
                report["dropped"] = len(docs) - len(kept)
                docs = kept
                Ragged.write(directory, docs)
            else:
                if docs is None:
                    raise ValueError("pack needs a map before it")
                p = s.params
                if p["shuffle_seed"] is not None:
                    order = np.random.default_rng(p["shuffle_seed"]).permutation(len(docs))
                    docs = [docs[j] for j in order]
                rows = pack_rows(docs, p["row_len"], p["completion_only"], p["strategy"])
                from .preprocessed import write_shards

                write_shards(rows, directory, source_key=keys[i])
                report["rows"] = len(rows)
            report["documents"] = len(docs)
            with open(os.path.join(directory, "stage.json"), "w") as f:
                json.dump(report, f)
            with open(os.path.join(directory, ".complete"), "w") as f:
                f.write(keys[i])
            self.built.append(s.name)

    def run(self) -> str:
        """The directory of the last stage's artifact, computed by the scope's working rank if it is not cached yet."""
        if not self.stages:
            raise ValueError("a pipeline needs at least one stage")
        from halo_b200.runtime import filesystem

        last = self.keys()[-1]
        with filesystem.main_first_by_store(f"pipeline/{last}", self.store, self.timeout) as working:
            if working and not self._complete(last):
                os.makedirs(self.cache_dir, exist_ok=True)
                self._compute()
        if not self._complete(last):
            raise FileNotFoundError(f"the pipeline artifact {last} is not visible from this rank: the working rank wrote to "
                                    f"{self.cache_dir!r}; is the cache directory on the storage the sharing flags declare?")
        return self._dir(last)

    def rows(self, dp_rank: int = 0, dp_world: int = 1) -> list[PackedBatch]:
        """The packed rows ``dp_rank, dp_rank + dp_world, ...`` (the last stage must be ``pack``)."""
        if not self.stages or self.stages[-1].kind != "pack":
            raise ValueError("rows() reads packed rows: end the pipeline with pack()")
        from .preprocessed import load_rows

        return load_rows(self.run(), dp_rank, dp_world)

    def documents(self) -> list[tuple[np.ndarray, np.ndarray]]:
        if self.stages and self.stages[-1].kind == "pack":
            raise ValueError("documents() reads a map / filter artifact; this pipeline ends with pack()")
        return Ragged.read(self.run())
