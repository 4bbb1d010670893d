"""Where training rows come from (halo/data/sources/{corpus,sharded_dataset,replica_identity}.py).

* :class:`CorpusMix` - several corpora drawn in fixed ratios: the sequence of corpus picks is a deterministic
  low-discrepancy schedule (each corpus is picked when it is furthest behind its share), so any prefix of the
  stream holds the requested proportions, every rank can compute the same schedule, and a resumed run continues it.
  A corpus that runs out starts its next epoch with a new shuffle.
* :func:`shard_for_rank` - per-rank shards: whole files are dealt round-robin when there are enough of them, else
  records are strided, so no rank reads what it will not use.
* :func:`assert_replicas_identical` - ranks that must see the same rows (the ranks of one tensor- or
  context-parallel group) compare a digest of their data; a difference is refused on every rank before the first
  step, because it would silently train on mismatched halves of a batch.
* :func:`best_fit_rows` - packing by best-fit-decreasing within a look-ahead window: fuller rows than sequential
  greedy packing at the same document order statistics.
"""

from __future__ import annotations

import hashlib

import numpy as np


class CorpusMix:
    def __init__(self, corpora: list, ratios: list[float], seed: int = 0):
        """``corpora``: sequences (lists of documents); ``ratios``: positive weights, normalised here."""
        if len(corpora) != len(ratios) or not corpora:
            raise ValueError("give one ratio per corpus")
        if any(r <= 0 for r in ratios) or any(len(c) == 0 for c in corpora):
            raise ValueError("ratios must be positive and corpora non-empty")
        self.corpora, self.seed = corpora, seed
        total = float(sum(ratios))
        self.share = [r / total for r in ratios]
        self.reset()

    def reset(self) -> None:
        self.drawn = [0] * len(self.corpora)
        self.epoch = [0] * len(self.corpora)
        self.order = [self._shuffle(i, 0) for i in range(len(self.corpora))]
        self.n = 0

    def _shuffle(self, i: int, epoch: int):
        return np.random.default_rng((self.seed, i, epoch)).permutation(len(self.corpora[i]))

    def next_corpus(self) -> int:
        """The corpus furthest behind its share after ``n`` draws (ties: the lower index)."""
        deficit = [self.share[i] * (self.n + 1) - self.drawn[i] for i in range(len(self.corpora))]
        return int(np.argmax(deficit))

    def __iter__(self):
        return self

    def __next__(self):
        i = self.next_corpus()
        k = self.drawn[i] - self.epoch[i] * len(self.corpora[i])
        if k >= len(self.corpora[i]):
            self.epoch[i] += 1
            self.order[i] = self._shuffle(i, self.epoch[i])
            k = 0
        doc = self.corpora[i][int(self.order[i][k])]
        self.drawn[i] += 1
        self.n += 1
        return i, doc

    def state_dict(self) -> dict:
        return {"drawn": list(self.drawn), "epoch": list(self.epoch), "n": self.n}

    def load_state_dict(self, state: dict) -> None:
        self.drawn, self.epoch, self.n = list(state["drawn"]), list(state["epoch"]), int(state["n"])
        self.order = [self._shuffle(i, e) for i, e in enumerate(self.epoch)]


def shard_for_rank(files: list[str], rank: int, world: int) -> tuple[list[str], tuple[int, int]]:
    """``(files this rank opens, (record offset, record stride) inside them)``."""
    files = sorted(files)
    if len(files) >= world:
        return files[rank::world], (0, 1)
    return files, (rank, world)


def data_digest(rows) -> str:
    """Digest of a rank's rows (token ids and document boundaries)."""
    h = hashlib.blake2b(digest_size=16)
    for r in rows:
        h.update(np.ascontiguousarray(np.asarray(r.input_ids)).tobytes())
        h.update(np.ascontiguousarray(np.asarray(r.cu_seqlens)).tobytes())
    return h.hexdigest()


def assert_replicas_identical(rows, group=None, what: str = "tensor-parallel group") -> None:
    """COLLECTIVE over ``group``."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return
    mine = data_digest(rows)
    seen = [None] * dist.get_world_size(group)
    dist.all_gather_object(seen, mine, group=group)
    if len(set(seen)) != 1:
        raise RuntimeError(f"the ranks of one {what} hold different data ({len(set(seen))} distinct digests): they must read "
                           f"the same rows - check the data-parallel rank each of them was given")


def best_fit_rows(lengths: list[int], row_len: int, window: int = 512) -> list[list[int]]:
    """Document indices per row. Documents are taken ``window`` at a time (so the stream stays roughly in order), each
    window is packed by best-fit-decreasing; a document longer than a row gets a row of its own (and is cut by the
    caller)."""
    rows: list[list[int]] = []
    for lo in range(0, len(lengths), window):
        idx = sorted(range(lo, min(lo + window, len(lengths))), key=lambda i: -lengths[i])
        open_rows: list[tuple[int, list[int]]] = []          # (free space, members)
        for i in idx:
            n = min(lengths[i], row_len)
            best = None
            for j, (free, _) in enumerate(open_rows):
                if free >= n and (best is None or free < open_rows[best][0]):
                    best = j
            if best is None:
                open_rows.append((row_len - n, [i]))
            else:
                free, members = open_rows[best]
                open_rows[best] = (free - n, members + [i])
        rows.extend(sorted(members) for _, members in open_rows)
    return rows
