"""Grow (or cut) the vocabulary rows of ``embed_tokens`` and ``lm_head``; new rows take the mean of the old
ones so that a new token starts as an "average" token (halo/checkpoint/tools/vocab_patch.py).

    python -m halo_b200.checkpoint.tools.patch_vocab <src> <dst> --vocab-size 152064
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from ._io import rewrite

VOCAB_TENSORS = ("model.embed_tokens.weight", "lm_head.weight")


def resize_rows(t: torch.Tensor, rows: int) -> torch.Tensor:
    if rows <= t.shape[0]:
        return t[:rows].contiguous()
    mean = t.float().mean(0, keepdim=True).to(t.dtype)
    return torch.cat([t, mean.expand(rows - t.shape[0], -1)], dim=0).contiguous()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--vocab-size", type=int, required=True)
    a = ap.parse_args(argv)
    rewrite(a.src, a.dst, lambda n, t: {n: resize_rows(t, a.vocab_size) if n in VOCAB_TENSORS else t})
    cfg_path = os.path.join(a.dst, "config.json")
    cfg = json.load(open(cfg_path))
    cfg["vocab_size"] = a.vocab_size
    json.dump(cfg, open(cfg_path, "w"), indent=2)
    print(f"vocabulary is now {a.vocab_size} rows in {a.dst}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
