"""Collators beside the packing one (halo/data/collators/*.py).

``padding_free``: documents laid end to end WITHOUT padding to a fixed row (the stream is as long as the documents).
``fixed_shape``: every row padded to exactly ``row_len`` - what pipeline stages need, whose messages have one shape.
``padded``: classic ``[batch, max_len]`` right-padded tensors with an attention mask, for sequence-level heads fed
by other tooling."""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from halo_b200.data.packing import IGNORE_INDEX, PackedBatch, pack_documents


def padding_free(docs, label_masks=None) -> PackedBatch:
    return pack_documents(docs, row_len=None, label_masks=label_masks)


def fixed_shape(docs, row_len: int, pad_token_id: int = 0, label_masks=None) -> PackedBatch:
    total = sum(len(d) for d in docs)
    if total > row_len:
        raise ValueError(f"{total} tokens do not fit a fixed row of {row_len}")
    return pack_documents(docs, row_len=row_len, pad_token_id=pad_token_id, label_masks=label_masks)


def padded(docs, pad_token_id: int = 0, max_len: int | None = None, pad_to_multiple_of: int = 1) -> dict:
    n = max(len(d) for d in docs)
    n = min(n, max_len) if max_len else n
    n = (n + pad_to_multiple_of - 1) // pad_to_multiple_of * pad_to_multiple_of
    ids = np.full((len(docs), n), pad_token_id, dtype=np.int64)
    mask = np.zeros((len(docs), n), dtype=np.int64)
    labels = np.full((len(docs), n), IGNORE_INDEX, dtype=np.int64)
    for i, d in enumerate(docs):
        d = np.asarray(d, dtype=np.int64)[:n]
        ids[i, :len(d)] = d
        mask[i, :len(d)] = 1
        labels[i, :len(d) - 1] = d[1:]
    return {"input_ids": torch.from_numpy(ids), "attention_mask": torch.from_numpy(mask), "labels": torch.from_numpy(labels)}


@dataclass
class ClassificationBatch(PackedBatch):
    """A packed row whose every document carries one class label."""

    doc_labels: torch.Tensor = None      # [n_docs] int64

    def to(self, device, non_blocking: bool = True):
        b = PackedBatch.to(self, device, non_blocking)
        return ClassificationBatch(b.input_ids, b.position_ids, b.labels, b.cu_seqlens, b.n_scored,
                                   self.doc_labels.to(device, non_blocking=non_blocking))
