"""Fold a low-rank adapter (PEFT layout: ``adapter_config.json`` + ``adapter_model.safetensors``) into a base
checkpoint, streaming one tensor at a time: every ``<module>.weight`` with a ``lora_A`` / ``lora_B`` pair becomes
``W + (alpha / r) * B A``; everything else is copied (the role of halo/checkpoint/tools merge-PEFT tools, including
the streaming form). Routed-expert pairs (one per global expert) fold the same way.

    python -m halo_b200.checkpoint.tools.merge_adapter <base_dir> <adapter_dir> <out_dir>
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
from safetensors import safe_open

from ._io import rewrite

PREFIX = "base_model.model."


def merge(base: str, adapter: str, dst: str, save_dtype=None) -> int:
    cfg = json.load(open(os.path.join(adapter, "adapter_config.json")))
    scale = float(cfg["lora_alpha"]) / int(cfg["r"])
    handle = safe_open(os.path.join(adapter, "adapter_model.safetensors"), "pt")
    keys = set(handle.keys())
    modules = {k[len(PREFIX):-len(".lora_A.weight")] for k in keys if k.endswith(".lora_A.weight")}
    used: set[str] = set()

    def fold(name: str, t: torch.Tensor) -> dict:
        module = name[:-len(".weight")] if name.endswith(".weight") else None
        if module in modules:
            a = handle.get_tensor(f"{PREFIX}{module}.lora_A.weight").float()
            b = handle.get_tensor(f"{PREFIX}{module}.lora_B.weight").float()
            if (b.shape[0], a.shape[1]) != tuple(t.shape):
                raise ValueError(f"adapter of {module} is {tuple(b.shape)} x {tuple(a.shape)}, the weight {tuple(t.shape)}")
            used.add(module)
            return {name: (t.float() + scale * (b @ a)).to(t.dtype)}
        return {name: t}

    n = rewrite(base, dst, fold, save_dtype)
    left = sorted(modules - used)
    if left:
        raise KeyError(f"{len(left)} adapted modules are absent from the base checkpoint, e.g. {left[:3]}")
    return len(used)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("base")
    ap.add_argument("adapter")
    ap.add_argument("dst")
    args = ap.parse_args(argv)
    n = merge(args.base, args.adapter, args.dst)
    print(f"folded {n} adapter pairs into {args.dst}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
