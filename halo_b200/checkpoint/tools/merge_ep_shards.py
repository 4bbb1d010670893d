"""Merge a sharded expert-parallel save (``ep_shard_<rank>/`` directories, each holding that rank's experts
under their global hub names, plus the writer rank's non-expert tensors in the top directory) into one
ordinary hub-layout checkpoint (halo/checkpoint/tools/merge_ep_shards.py).

    python -m halo_b200.checkpoint.tools.merge_ep_shards <sharded_dir> <out_dir>
"""

from __future__ import annotations

import argparse
import os
import re
import sys

from ._io import CheckpointIndex, StreamingShardWriter, copy_side_files

SHARD_DIR = re.compile(r"^ep_shard_(\d+)$")


def merge(src: str, dst: str, max_shard_bytes: int = 5 * 1024**3) -> int:
    shards = sorted(d for d in os.listdir(src) if SHARD_DIR.match(d))
    if not shards:
        raise FileNotFoundError(f"{src!r} holds no ep_shard_<rank> directories")
    writer = StreamingShardWriter(dst, max_shard_bytes)
    seen: set[str] = set()
    sources = [src] + [os.path.join(src, d) for d in shards]
    for directory in sources:
        try:
            idx = CheckpointIndex(directory)
        except FileNotFoundError:
            if directory == src:
                continue      # the top directory may hold only side files
            raise
        for name in sorted(idx.weight_map):
            if name in seen:
                raise ValueError(f"tensor {name!r} appears in more than one shard")
            seen.add(name)
            writer.add(name, idx.get(name))
        idx.close()
    writer.finish()
    copy_side_files(src, dst)
    return len(seen)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("src")
    ap.add_argument("dst")
    args = ap.parse_args(argv)
    n = merge(args.src, args.dst)
    print(f"merged {n} tensors into {args.dst}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
