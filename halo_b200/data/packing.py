"""Packed rows: several documents laid end to end in one token stream with per-document position
ids, ``cu_seqlens`` for the attention kernels and next-token labels that never cross a document
boundary.

A batch for this framework is one flat stream per rank - the layout the reference's packing
collator flattens to ``[1, total]`` (halo/data/collators/packing.py:75) with position ids reset per
document and a pad tail whose positions keep ramping (halo/data/collators/packing.py:36-41).
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

IGNORE_INDEX = -100


@dataclass
class PackedBatch:
    input_ids: torch.Tensor      # int64 [T]
    position_ids: torch.Tensor   # int32 [T]
    labels: torch.Tensor         # int64 [T], already shifted: labels[t] scores the prediction at t
    cu_seqlens: np.ndarray       # int64 [n_docs + 1] on the host
    n_scored: int                # number of labels != IGNORE_INDEX

    @property
    def n_tokens(self) -> int:
        return int(self.input_ids.numel())

    def pin(self) -> "PackedBatch":
        if torch.cuda.is_available():
            self.input_ids = self.input_ids.pin_memory()
            self.position_ids = self.position_ids.pin_memory()
            self.labels = self.labels.pin_memory()
        return self

    def to(self, device, non_blocking: bool = True) -> "PackedBatch":
        return PackedBatch(
            self.input_ids.to(device, non_blocking=non_blocking),
            self.position_ids.to(device, non_blocking=non_blocking),
            self.labels.to(device, non_blocking=non_blocking),
            self.cu_seqlens, self.n_scored,
        )

    def h2d_bytes(self) -> int:
        return int(self.input_ids.numel() * 8 + self.position_ids.numel() * 4 + self.labels.numel() * 8)


def pack_documents(docs, row_len: int | None = None, pad_token_id: int = 0, label_masks=None) -> PackedBatch:
    """Lay ``docs`` (lists / arrays of token ids) end to end.

    ``row_len``: pad the stream to this length with a tail "document" of pad tokens that is never
    scored (its positions ramp from 0 like any document). ``label_masks``: optional per-document
    boolean arrays, True where the token may be a training target (completion-only losses).
    """
    ids, pos, labels, cu = [], [], [], [0]
    for di, d in enumerate(docs):
        d = np.asarray(d, dtype=np.int64)
        n = len(d)
        if n == 0:
            continue
        ids.append(d)
        pos.append(np.arange(n, dtype=np.int32))
        lab = np.full(n, IGNORE_INDEX, dtype=np.int64)
        lab[:-1] = d[1:]
        if label_masks is not None:
            mask = np.asarray(label_masks[di], dtype=bool)
            tgt_ok = np.zeros(n, dtype=bool)
            tgt_ok[:-1] = mask[1:]
            lab[~tgt_ok] = IGNORE_INDEX
        labels.append(lab)
        cu.append(cu[-1] + n)
    total = cu[-1]
    if row_len is not None:
        if total > row_len:
            raise ValueError(f"documents hold {total} tokens, more than the row length {row_len}")
        pad = row_len - total
        if pad:
            ids.append(np.full(pad, pad_token_id, dtype=np.int64))
            pos.append(np.arange(pad, dtype=np.int32))
            labels.append(np.full(pad, IGNORE_INDEX, dtype=np.int64))
            cu.append(cu[-1] + pad)
    ids = np.concatenate(ids) if ids else np.zeros(0, dtype=np.int64)
    pos = np.concatenate(pos) if pos else np.zeros(0, dtype=np.int32)
    labels = np.concatenate(labels) if labels else np.zeros(0, dtype=np.int64)
    return PackedBatch(torch.from_numpy(ids), torch.from_numpy(pos), torch.from_numpy(labels),
                       np.asarray(cu, dtype=np.int64), int((labels != IGNORE_INDEX).sum()))


def sample_doc_lengths(total: int, rng: np.random.Generator, dist: str = "loguniform", lo: int = 256,
                       hi: int = 16384) -> list[int]:
    """Document lengths that fill exactly ``total`` tokens (the last one is truncated to fit)."""
    out, left = [], total
    while left > 0:
        if dist == "loguniform":
            n = int(np.exp(rng.uniform(np.log(lo), np.log(hi))))
        elif dist == "uniform":
            n = int(rng.integers(lo, hi + 1))
        elif dist == "single":
            n = total
        elif dist == "chat":
            # the shape of chat-template SFT rows the reference benchmarks on: about 55 whole documents
            # per 64k-token row, none longer than 4,579 tokens
            # (agent-docs/optimization/throughput-benchmarks.md:85-87)
            n = int(np.clip(rng.lognormal(6.90, 0.6), 64, 4579))
        else:
            raise ValueError(f"unknown length distribution {dist!r}")
        n = max(1, min(n, left))
        out.append(n)
        left -= n
    return out


def synthetic_packed_batch(seq_len: int, vocab_size: int, seed: int, dist: str = "loguniform", lo: int = 256,
                           hi: int = 16384) -> PackedBatch:
    """Uniform-random token ids in packed documents (all tokens scored)."""
    rng = np.random.default_rng(seed)
    lens = sample_doc_lengths(seq_len, rng, dist, lo, hi)
    docs = [rng.integers(0, vocab_size, size=n, dtype=np.int64) for n in lens]
    return pack_documents(docs)
