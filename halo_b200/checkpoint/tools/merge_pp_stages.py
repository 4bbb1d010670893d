"""Merge the per-node directories of one pipeline-parallel save into one checkpoint that ``from_pretrained`` loads.

On an output filesystem the nodes do not share, every node's copy of the checkpoint directory holds only the shard files
its own stages wrote (``model-stage<k>-*.safetensors``) and, on the first stage's node, the merged index and
``config.json``. This tool unions the shard files into one directory, rebuilds ``model.safetensors.index.json`` from the
files actually present (every tensor exactly once, or it refuses), and copies the side files from whichever directory
has them.

    python -m halo_b200.checkpoint.tools.merge_pp_stages <node0_dir> <node1_dir> ... --out <dir>

Counterpart of halo/checkpoint/tools/pp_stage_merge.py:1-89.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import sys

from safetensors import safe_open

from ._io import copy_side_files


def merge(node_dirs: list[str], dst: str, link: bool = False) -> dict:
    os.makedirs(dst, exist_ok=True)
    weight_map: dict[str, str] = {}
    total = 0
    seen_files: dict[str, str] = {}
    for d in node_dirs:
        for f in sorted(os.listdir(d)):
            if not f.endswith(".safetensors"):
                continue
            src = os.path.join(d, f)
            if f in seen_files:
                if os.path.getsize(seen_files[f]) != os.path.getsize(src):
                    raise ValueError(f"{f} exists in {os.path.dirname(seen_files[f])} and {d} with different sizes: the directories "
                                     "are not parts of one save")
                continue                       # the same file seen through a shared mount
            seen_files[f] = src
            with safe_open(src, "pt") as h:
                for name in h.keys():
                    if name in weight_map:
                        raise ValueError(f"tensor {name} is in both {weight_map[name]} and {f}: stages overlap")
                    weight_map[name] = f
                    sl = h.get_slice(name)
                    n = 1
                    for s in sl.get_shape():
                        n *= s
                    total += n * {"BF16": 2, "F16": 2, "F32": 4, "F64": 8, "I64": 8, "I32": 4, "U8": 1, "I8": 1, "F8_E4M3": 1,
                                  "BOOL": 1}.get(sl.get_dtype(), 2)
            out = os.path.join(dst, f)
            if os.path.abspath(out) != os.path.abspath(src):
                if link:
                    if os.path.lexists(out):
                        os.remove(out)
                    os.symlink(os.path.abspath(src), out)
                else:
                    shutil.copyfile(src, out)
    if not weight_map:
        raise FileNotFoundError(f"no safetensors files under {node_dirs}")
    # an index written by the first stage lists every tensor the save intended: all of them must have been found
    for d in node_dirs:
        idx = os.path.join(d, "model.safetensors.index.json")
        if os.path.isfile(idx):
            intended = set(json.load(open(idx))["weight_map"])
            missing = sorted(intended - set(weight_map))
            if missing:
                raise ValueError(f"{len(missing)} tensors of the save are in none of the directories (first: {missing[0]}): "
                                 "a node's directory is missing")
            break
    for d in node_dirs:
        copy_side_files(d, dst)
    with open(os.path.join(dst, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": dict(sorted(weight_map.items()))}, f, indent=2)
    return {"tensors": len(weight_map), "files": len(seen_files), "bytes": total}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("node_dirs", nargs="+")
    ap.add_argument("--out", required=True)
    ap.add_argument("--link", action="store_true", help="symlink the shard files instead of copying them")
    args = ap.parse_args(argv)
    out = merge(args.node_dirs, args.out, args.link)
    print(f"merged {out['tensors']} tensors in {out['files']} files ({out['bytes'] / 1e9:.2f} GB) into {args.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
