"""Offline-prepared datasets: tokenise and pack once, write numbered shards plus a ``metadata.json`` contract, and
load them back rank-sharded (halo/data/preprocessed/{metadata,preparation,shard_index}.py). Also the coordinated
cache: one rank builds an artifact under a deterministic key, the others wait for it and read it
(halo/data/pipeline/coordinated_map.py, map_cache_key.py).

Shard ``rows_<i>.npz`` holds, per packed row, ``input_ids``, ``labels``, ``position_ids`` (all ``[row_len]``) and the
row's ``cu_seqlens`` (ragged, stored as one concatenated array with offsets). ``metadata.json`` records the row
length, the number of rows per shard, the tokenizer identity and the cache key of the inputs; a loader refuses
metadata it does not understand."""

from __future__ import annotations

import json
import os
import time

import numpy as np
import torch

from halo_b200.checkpoint.atomic import atomic_write_json, staged_path
from halo_b200.data.datasets import cache_key
from halo_b200.data.packing import PackedBatch

FORMAT_VERSION = 1


def write_shards(rows: list[PackedBatch], out_dir: str, rows_per_shard: int = 256, tokenizer_name: str = "",
                 source_key: str = "") -> dict:
    os.makedirs(out_dir, exist_ok=True)
    if not rows:
        raise ValueError("no rows to write")
    row_len = rows[0].n_tokens
    shards = []
    for s in range(0, len(rows), rows_per_shard):
        part = rows[s:s + rows_per_shard]
        if any(r.n_tokens != row_len for r in part):
            raise ValueError("every packed row of a prepared dataset has the same length")
        cu_all = np.concatenate([r.cu_seqlens for r in part])
        cu_off = np.cumsum([0] + [len(r.cu_seqlens) for r in part])
        name = f"rows_{len(shards):05d}.npz"
        with staged_path(os.path.join(out_dir, name)) as tmp:
            with open(tmp, "wb") as f:
                np.savez(f, input_ids=np.stack([r.input_ids.numpy() for r in part]),
                         labels=np.stack([r.labels.numpy() for r in part]),
                         position_ids=np.stack([r.position_ids.numpy() for r in part]), cu=cu_all, cu_off=cu_off)
        shards.append({"file": name, "rows": len(part)})
    meta = {"format_version": FORMAT_VERSION, "row_len": row_len, "n_rows": len(rows), "shards": shards,
            "tokenizer": tokenizer_name, "source_key": source_key}
    atomic_write_json(os.path.join(out_dir, "metadata.json"), meta)      # written last: its presence means complete
    return meta


def read_metadata(path: str) -> dict:
    p = os.path.join(path, "metadata.json")
    if not os.path.isfile(p):
        raise FileNotFoundError(f"{path!r} is not a prepared dataset (no metadata.json: preparation did not finish)")
    meta = json.load(open(p))
    if meta.get("format_version") != FORMAT_VERSION:
        raise ValueError(f"prepared dataset {path!r} has format {meta.get('format_version')}, this build reads {FORMAT_VERSION}")
    return meta


def load_rows(path: str, dp_rank: int = 0, dp_world: int = 1, expect_row_len: int | None = None) -> list[PackedBatch]:
    """Rows ``dp_rank, dp_rank + dp_world, ...`` of the prepared dataset."""
    meta = read_metadata(path)
    if expect_row_len is not None and meta["row_len"] != expect_row_len:
        raise ValueError(f"the dataset was packed to {meta['row_len']} tokens per row, the run asks for {expect_row_len}")
    out, index = [], 0
    for sh in meta["shards"]:
        lo, hi = index, index + sh["rows"]
        index = hi
        mine = [i for i in range(lo, hi) if i % dp_world == dp_rank]
        if not mine:
            continue
        z = np.load(os.path.join(path, sh["file"]))
        for i in mine:
            j = i - lo
            cu = z["cu"][z["cu_off"][j]:z["cu_off"][j + 1]]
            labels = torch.from_numpy(z["labels"][j])
            out.append(PackedBatch(torch.from_numpy(z["input_ids"][j]), torch.from_numpy(z["position_ids"][j]), labels,
                                   cu.astype(np.int64), int((labels != -100).sum())))
    return out


def coordinated_cache(cache_dir: str, key_parts: list, build, rank: int = 0, wait_seconds: float = 4 * 3600,
                      poll_seconds: float = 0.5) -> str:
    """Directory of an artifact identified by ``key_parts``. Rank 0 calls ``build(directory)`` when it does not
    exist yet (and marks it complete); every other rank polls for the completion marker with a deadline. A second
    run with the same inputs finds the artifact and builds nothing."""
    key = cache_key(*key_parts)
    directory = os.path.join(cache_dir, key)
    marker = os.path.join(directory, ".complete")
    if os.path.isfile(marker):
        return directory
    if rank == 0:
        os.makedirs(directory, exist_ok=True)
        build(directory)
        with open(marker, "w") as f:
            f.write(key)
        return directory
    deadline = time.monotonic() + wait_seconds
    while not os.path.isfile(marker):
        if time.monotonic() > deadline:
            raise TimeoutError(f"the artifact {key} was not completed by the building rank within {wait_seconds} s")
        time.sleep(poll_seconds)
    return directory


def main(argv=None) -> int:
    """``python -m halo_b200.data.preprocessed <jsonl or dir> <out_dir> --row-len N [--tokenizer PATH]``"""
    import argparse

    from halo_b200.configs.arguments import DataArguments
    from halo_b200.data.datasets import pack_rows, read_records, tokenize_record

    ap = argparse.ArgumentParser()
    ap.add_argument("src")
    ap.add_argument("out")
    ap.add_argument("--row-len", type=int, required=True)
    ap.add_argument("--tokenizer", default="")
    ap.add_argument("--completion-only", action="store_true")
    a = ap.parse_args(argv)
    tok = None
    if a.tokenizer:
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(a.tokenizer)
    docs = [tokenize_record(r, tok) for r in read_records(a.src)]
    rows = pack_rows(docs, a.row_len, a.completion_only)
    meta = write_shards(rows, a.out, tokenizer_name=a.tokenizer, source_key=cache_key(a.src, a.row_len, a.tokenizer))
    print(f"wrote {meta['n_rows']} rows of {meta['row_len']} tokens to {a.out}")
    _ = DataArguments
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
