"""Shared plumbing of the offline tools: iterate the tensors of a checkpoint one at a time and stream them
into a new one, so a tool never holds more than one shard in memory."""

from __future__ import annotations

import os
import shutil

from halo_b200.checkpoint.load import CheckpointIndex
from halo_b200.checkpoint.writing import INDEX_NAME, SINGLE_NAME, StreamingShardWriter

SIDE_FILES = ("config.json", "generation_config.json", "tokenizer.json", "tokenizer_config.json", "vocab.json",
              "merges.txt", "special_tokens_map.json", "chat_template.jinja", "added_tokens.json")


def tensor_names(directory: str) -> list[str]:
    idx = CheckpointIndex(directory)
    return sorted(idx.weight_map)


def copy_side_files(src: str, dst: str) -> None:
    os.makedirs(dst, exist_ok=True)
    for name in SIDE_FILES:
        p = os.path.join(src, name)
        if os.path.isfile(p):
            shutil.copy2(p, os.path.join(dst, name))


def rewrite(src: str, dst: str, fn, save_dtype=None, max_shard_bytes: int = 5 * 1024**3) -> int:
    """``fn(name, tensor) -> dict[name, tensor]`` maps every tensor of ``src``; the result is written to ``dst``."""
    idx = CheckpointIndex(src)
    writer = StreamingShardWriter(dst, max_shard_bytes, save_dtype)
    n = 0
    for name in sorted(idx.weight_map):
        for out_name, t in fn(name, idx.get(name)).items():
            writer.add(out_name, t)
            n += 1
    writer.finish()
    copy_side_files(src, dst)
    return n


__all__ = ["CheckpointIndex", "StreamingShardWriter", "INDEX_NAME", "SINGLE_NAME", "tensor_names", "copy_side_files", "rewrite"]
