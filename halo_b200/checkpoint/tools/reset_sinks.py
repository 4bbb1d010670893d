"""Neutralize (or restore from another checkpoint) the attention sinks of a gpt-oss checkpoint on disk: every
``self_attn.sinks`` tensor is set to almost the most negative finite bf16 value, so the sink takes no softmax mass -
the state a run with ``reset_sinks: true`` trains in, made permanent for serving stacks that cannot apply the policy
themselves (the reference's after-training sink-reset script over halo/models/attention/gpt_oss_sinks.py).

    python -m halo_b200.checkpoint.tools.reset_sinks <src> <dst> [--from-checkpoint DIR]
"""

from __future__ import annotations

import argparse
import sys

import torch

from halo_b200.models.attention_sinks import is_sink_name

from ._io import rewrite


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--from-checkpoint", default="", help="take the sinks of this checkpoint instead of neutralizing them")
    a = ap.parse_args(argv)
    donor = None
    if a.from_checkpoint:
        from halo_b200.checkpoint.load import CheckpointIndex

        donor = CheckpointIndex(a.from_checkpoint)
    touched = []

    def edit(name, t):
        if not is_sink_name(name):
            return {name: t}
        touched.append(name)
        if donor is not None:
            if name not in donor:
                raise KeyError(f"{a.from_checkpoint!r} has no tensor {name!r}")
            return {name: donor.get(name).to(t.dtype)}
        return {name: torch.full_like(t, 0.99 * torch.finfo(torch.bfloat16).min)}

    rewrite(a.src, a.dst, edit)
    if not touched:
        raise SystemExit(f"{a.src!r} holds no attention sinks")
    print(f"{len(touched)} sink tensors {'copied from ' + a.from_checkpoint if donor is not None else 'neutralized'} in {a.dst}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
