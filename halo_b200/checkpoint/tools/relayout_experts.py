"""Rewrite the expert weights of a checkpoint from one on-disk layout kind to another (per-expert
``gate_proj/up_proj/down_proj`` <-> fused banks <-> interleaved GLU ...): "unfuse experts" and its inverse
(halo/checkpoint/tools/unfuse_experts.py).

    python -m halo_b200.checkpoint.tools.relayout_experts <src> <dst> --from FUSED --to SEPARATE_GLU
"""

from __future__ import annotations

import argparse
import json
import os
import re
import sys

from halo_b200.models.moe_families import LAYOUT_KINDS, from_runtime_banks, to_runtime_banks

from ._io import CheckpointIndex, StreamingShardWriter, copy_side_files

EXPERT_KEY = re.compile(r"^(?P<prefix>.*\.experts\.)(?P<rest>.+)$")


def relayout(src: str, dst: str, kind_from: str, kind_to: str) -> int:
    idx = CheckpointIndex(src)
    cfg = json.load(open(os.path.join(src, "config.json")))
    n_experts = cfg.get("num_experts") or cfg.get("num_local_experts") or cfg.get("n_routed_experts")
    writer = StreamingShardWriter(dst)
    groups: dict[str, dict[str, str]] = {}
    n = 0
    for name in sorted(idx.weight_map):
        m = EXPERT_KEY.match(name)
        if m:
            groups.setdefault(m.group("prefix"), {})[m.group("rest")] = name
        else:
            writer.add(name, idx.get(name))
            n += 1
    for prefix, members in sorted(groups.items()):
        tensors = {rest: idx.get(full) for rest, full in members.items()}
        gate_up, down = to_runtime_banks(kind_from, tensors, n_experts)
        for rest, t in from_runtime_banks(kind_to, gate_up, down).items():
            writer.add(prefix + rest, t.contiguous())
            n += 1
    writer.finish()
    copy_side_files(src, dst)
    return n


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--from", dest="kind_from", required=True, choices=LAYOUT_KINDS)
    ap.add_argument("--to", dest="kind_to", required=True, choices=LAYOUT_KINDS)
    a = ap.parse_args(argv)
    print(f"wrote {relayout(a.src, a.dst, a.kind_from, a.kind_to)} tensors to {a.dst}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
