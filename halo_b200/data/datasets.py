"""Dataset sources and the packing pipeline (the part of halo/data/** the trainers need).

Sources: ``.jsonl`` / ``.json`` files or directories of them (text, chat ``messages``,
prompt/completion, preference pairs, pre-tokenised ``input_ids``), and the synthetic generator.
Tokenisation uses a Hugging Face tokenizer when one is available next to the checkpoint; rows are
sharded over data-parallel ranks Megatron-style (rank r takes rows r, r + dp, ...), packed into
fixed-length rows in a deterministic order, and cached under a key derived from the inputs so a
second run (or the other ranks) reads the cache instead of recomputing
(halo/data/pipeline/coordinated_map.py, halo/data/sources/sharded_dataset.py)."""

from __future__ import annotations

import glob
import hashlib
import json
import os
from typing import Iterator

import numpy as np

from halo_b200.data.packing import PackedBatch, pack_documents, synthetic_packed_batch


def list_files(path: str) -> list[str]:
    if os.path.isdir(path):
        return sorted(glob.glob(os.path.join(path, "**", "*.json*"), recursive=True))
    return [path]


def read_records(path: str) -> Iterator[dict]:
    if path.startswith("s3://"):
        # mirrored into the node's cache by the node's first rank; the other ranks wait for its completion marker
        from halo_b200.data.s3 import resolve_dataset_path

        path = resolve_dataset_path(path, is_downloader=int(os.environ.get("LOCAL_RANK", "0")) == 0)
    for f in list_files(path):
        with open(f) as fh:
            if f.endswith(".jsonl"):
                for line in fh:
                    if line.strip():
                        yield json.loads(line)
            else:
                data = json.load(fh)
                yield from (data if isinstance(data, list) else [data])


def cache_key(*parts) -> str:
    h = hashlib.blake2b(digest_size=12)
    for p in parts:
        h.update(json.dumps(p, sort_keys=True, default=str).encode())
    return h.hexdigest()


def render_messages(messages: list[dict]) -> tuple[str, list[tuple[int, int]]]:
    """Minimal ChatML rendering; returns the text and the character spans of assistant turns."""
    text, spans = "", []
    for m in messages:
        head = f"<|im_start|>{m['role']}\n"
        body = f"{m['content']}<|im_end|>\n"
        if m["role"] == "assistant":
            spans.append((len(text) + len(head), len(text) + len(head) + len(body)))
        text += head + body
    return text, spans


def tokenize_record(rec: dict, tokenizer, fmt: str = "auto") -> tuple[np.ndarray, np.ndarray]:
    """(token ids, bool mask of tokens that may be targets)."""
    if "input_ids" in rec:
        ids = np.asarray(rec["input_ids"], dtype=np.int64)
        mask = np.asarray(rec.get("loss_mask", np.ones(len(ids), bool)), dtype=bool)
        return ids, mask
    if tokenizer is None:
        raise ValueError("a tokenizer is needed for text records (or provide pre-tokenised 'input_ids')")
    if "messages" in rec and getattr(tokenizer, "chat_template", None):
        from .chat_render import render_conversation

        ids, mask, _ = render_conversation(tokenizer, rec["messages"], rec.get("tools"))
        return ids, mask
    if "messages" in rec:
        text, spans = render_messages(rec["messages"])
        enc = tokenizer(text, return_offsets_mapping=True, add_special_tokens=False)
        ids = np.asarray(enc["input_ids"], dtype=np.int64)
        mask = np.zeros(len(ids), bool)
        for i, (a, b) in enumerate(enc["offset_mapping"]):
            mask[i] = any(a >= s and b <= e for s, e in spans)
        return ids, mask
    if "prompt" in rec and "completion" in rec:
        p = tokenizer(rec["prompt"], add_special_tokens=False)["input_ids"]
        c = tokenizer(rec["completion"], add_special_tokens=False)["input_ids"]
        return np.asarray(p + c, dtype=np.int64), np.asarray([False] * len(p) + [True] * len(c))
    ids = np.asarray(tokenizer(rec.get("text", ""), add_special_tokens=False)["input_ids"], dtype=np.int64)
    return ids, np.ones(len(ids), bool)


def pack_rows(docs: list[tuple[np.ndarray, np.ndarray]], row_len: int, completion_only: bool, strategy: str = "sequential") -> list[PackedBatch]:
    """Packing into rows of ``row_len`` tokens; a document longer than a row is cut. ``sequential``: greedy in order;
    ``best_fit``: best-fit-decreasing inside a look-ahead window (fuller rows)."""
    if strategy == "best_fit":
        from .sources import best_fit_rows

        out = []
        for members in best_fit_rows([len(ids) for ids, _ in docs], row_len):
            out.append(pack_documents([docs[i][0][:row_len] for i in members], row_len=row_len,
                                      label_masks=[docs[i][1][:row_len] for i in members] if completion_only else None))
        return out
    rows, cur, cur_masks, used = [], [], [], 0
    for ids, mask in docs:
        ids, mask = ids[:row_len], mask[:row_len]
        if used + len(ids) > row_len and cur:
            rows.append(pack_documents(cur, row_len=row_len, label_masks=cur_masks if completion_only else None))
            cur, cur_masks, used = [], [], 0
        cur.append(ids)
        cur_masks.append(mask)
        used += len(ids)
    if cur:
        rows.append(pack_documents(cur, row_len=row_len, label_masks=cur_masks if completion_only else None))
    return rows


def build_sft_batches(data_args, tokenizer, dp_rank: int = 0, dp_world: int = 1, vocab_size: int = 0) -> list[PackedBatch]:
    if data_args.dataset_format == "synthetic" or not data_args.dataset_path:
        n = 64
        return [synthetic_packed_batch(data_args.packed_row_length, data_args.synthetic_vocab or vocab_size,
                                       seed=data_args.shuffle_seed * 100003 + i * dp_world + dp_rank,
                                       lo=data_args.doc_length_min, hi=data_args.doc_length_max) for i in range(n)]
    if getattr(data_args, "cache_dir", ""):
        # tokenise and pack once per filesystem scope, under a key of the files, the tokenizer and the packing settings;
        # the other ranks wait for the artifact and read their rows from it
        from .pipeline import Pipeline

        fmt = data_args.dataset_format
        pipe = Pipeline(data_args.dataset_path, data_args.cache_dir)
        pipe.map(lambda rec: tokenize_record(rec, tokenizer, fmt), "tokenize", format=fmt,
                 tokenizer=getattr(tokenizer, "name_or_path", type(tokenizer).__name__),
                 vocab=getattr(tokenizer, "vocab_size", 0))
        pipe.pack(data_args.packed_row_length, getattr(data_args, "packing_strategy", "sequential"),
                  data_args.completion_only_loss, data_args.shuffle_seed)
        return pipe.rows(dp_rank, dp_world)
    docs = [tokenize_record(r, tokenizer, data_args.dataset_format) for r in read_records(data_args.dataset_path)]
    order = np.random.default_rng(data_args.shuffle_seed).permutation(len(docs))
    docs = [docs[i] for i in order]
    rows = pack_rows(docs, data_args.packed_row_length, data_args.completion_only_loss,
                     getattr(data_args, "packing_strategy", "sequential"))
    return rows[dp_rank::dp_world]


def build_preference_batches(data_args, tokenizer, dp_rank: int = 0, dp_world: int = 1, vocab_size: int = 0,
                             kto: bool = False):
    """Rows of (chosen, rejected) document pairs laid out chosen-first: document 2i is chosen, 2i+1 rejected
    (the preference row processor of halo/data/pipeline/preferences.py). Prompt tokens are never scored."""
    import torch

    from halo_b200.trainers.preference import PreferenceBatch

    row_len = data_args.packed_row_length
    pairs = []
    if data_args.dataset_format == "synthetic" or not data_args.dataset_path:
        rng = np.random.default_rng(data_args.shuffle_seed + 7919 * dp_rank)
        v = data_args.synthetic_vocab or vocab_size
        for _ in range(256):
            p = rng.integers(0, v, size=int(rng.integers(8, 64)))
            c = rng.integers(0, v, size=int(rng.integers(8, 128)))
            r = rng.integers(0, v, size=int(rng.integers(8, 128)))
            pairs.append((p, c, r))
    else:
        for rec in read_records(data_args.dataset_path):
            tok = lambda s: np.asarray(tokenizer(s, add_special_tokens=False)["input_ids"], dtype=np.int64)  # noqa: E731
            pairs.append((tok(rec["prompt"]), tok(rec["chosen"]), tok(rec["rejected"])))
        pairs = pairs[dp_rank::dp_world]
    rows, docs, masks, used = [], [], [], 0

    def flush():
        nonlocal docs, masks, used
        if docs:
            b = pack_documents(docs, row_len=row_len, label_masks=masks)
            n_docs = len(b.cu_seqlens) - 1
            desirable = torch.tensor([(i % 2 == 0) for i in range(n_docs)]) if kto else None
            rows.append(PreferenceBatch(b.input_ids, b.position_ids, b.labels, b.cu_seqlens, b.n_scored, None, desirable))
        docs, masks, used = [], [], 0

    for p, c, r in pairs:
        need = 2 * len(p) + len(c) + len(r)
        if need > row_len:
            continue
        if used + need > row_len:
            flush()
        for tail in (c, r):
            docs.append(np.concatenate([p, tail]))
            masks.append(np.concatenate([np.zeros(len(p), bool), np.ones(len(tail), bool)]))
        used += need
    flush()
    return rows


def build_classification_batches(data_args, tokenizer, num_labels: int, dp_rank: int = 0, dp_world: int = 1, vocab_size: int = 0):
    """Packed rows of whole documents with one label each (``{"text" | "input_ids", "label"}`` records). Without a
    dataset: synthetic documents whose label is a function of their first token (learnable)."""
    import torch

    from halo_b200.data.collators import ClassificationBatch

    row_len = data_args.packed_row_length
    docs = []
    if data_args.dataset_format == "synthetic" or not data_args.dataset_path:
        rng = np.random.default_rng(data_args.shuffle_seed + 7919 * dp_rank)
        v = data_args.synthetic_vocab or vocab_size
        for _ in range(512):
            ids = rng.integers(0, v, size=int(rng.integers(8, 96)))
            docs.append((ids, int(ids[0] % num_labels)))
    else:
        for rec in read_records(data_args.dataset_path):
            ids, _ = tokenize_record(rec, tokenizer, data_args.dataset_format)
            label = int(rec["label"])
            if not 0 <= label < num_labels:
                raise ValueError(f"label {label} outside 0..{num_labels - 1}")
            docs.append((ids[:row_len], label))
        docs = docs[dp_rank::dp_world]
    rows, cur, labels, used = [], [], [], 0

    def flush():
        nonlocal cur, labels, used
        if cur:
            b = pack_documents(cur)              # no padding "document": every document of the row carries a label
            rows.append(ClassificationBatch(b.input_ids, b.position_ids, b.labels, b.cu_seqlens, b.n_scored, torch.tensor(labels)))
        cur, labels, used = [], [], 0

    for ids, label in docs:
        if used + len(ids) > row_len:
            flush()
        cur.append(ids)
        labels.append(label)
        used += len(ids)
    flush()
    return rows


def build_embedding_batches(data_args, tokenizer, dp_rank: int = 0, dp_world: int = 1, vocab_size: int = 0, pairs_per_row: int = 16):
    """Packed rows in which documents alternate query, positive (``{"query", "positive"}`` records); the other pairs of
    a row are the in-batch negatives. Without a dataset: the positive is a noisy copy of the query."""
    row_len = data_args.packed_row_length
    pairs = []
    if data_args.dataset_format == "synthetic" or not data_args.dataset_path:
        rng = np.random.default_rng(data_args.shuffle_seed + 104729 * dp_rank)
        v = data_args.synthetic_vocab or vocab_size
        for _ in range(512):
            q = rng.integers(0, v, size=int(rng.integers(8, 48)))
            p = q.copy()
            flip = rng.random(len(p)) < 0.2
            p[flip] = rng.integers(0, v, size=int(flip.sum()))
            pairs.append((q, p))
    else:
        tok = lambda s: np.asarray(tokenizer(s, add_special_tokens=False)["input_ids"], dtype=np.int64)  # noqa: E731
        for rec in read_records(data_args.dataset_path):
            pairs.append((tok(rec["query"])[:row_len // 2], tok(rec["positive"])[:row_len // 2]))
        pairs = pairs[dp_rank::dp_world]
    rows, cur, used = [], [], 0
    for q, p in pairs:
        if cur and (used + len(q) + len(p) > row_len or len(cur) >= 2 * pairs_per_row):
            rows.append(pack_documents(cur))
            cur, used = [], 0
        cur += [q, p]
        used += len(q) + len(p)
    if len(cur) >= 4:                       # a row needs at least one negative
        rows.append(pack_documents(cur))
    return rows
