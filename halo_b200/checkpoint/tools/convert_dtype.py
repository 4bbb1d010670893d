"""Rewrite a checkpoint in another floating-point dtype (bf16 by default), shard by shard.

    python -m halo_b200.checkpoint.tools.convert_dtype <src> <dst> [--dtype bfloat16|float16|float32]
"""

from __future__ import annotations

import argparse
import sys

import torch

from ._io import rewrite


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    args = ap.parse_args(argv)
    n = rewrite(args.src, args.dst, lambda name, t: {name: t}, save_dtype=getattr(torch, args.dtype))
    print(f"wrote {n} tensors as {args.dtype} to {args.dst}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
