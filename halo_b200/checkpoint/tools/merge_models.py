"""Weight-space merges of checkpoints that share an architecture: ``linear`` (weighted average), ``slerp``
(spherical interpolation of two models, per tensor) and ``ties`` (trim each task vector to its largest
entries, elect a sign per coordinate, average the agreeing entries) - the merges of the reference's
halo/checkpoint/tools/merge_models.py. Tensors stream one at a time.

    python -m halo_b200.checkpoint.tools.merge_models --method linear --weights 0.5 0.5 A B --out C
    python -m halo_b200.checkpoint.tools.merge_models --method slerp --t 0.3 A B --out C
    python -m halo_b200.checkpoint.tools.merge_models --method ties --base BASE --density 0.2 A B --out C
"""

from __future__ import annotations

import argparse
import sys

import torch

from ._io import CheckpointIndex, StreamingShardWriter, copy_side_files


def linear(tensors: list[torch.Tensor], weights: list[float]) -> torch.Tensor:
    total = sum(weights)
    return sum(w / total * t.float() for w, t in zip(weights, tensors))


def slerp(a: torch.Tensor, b: torch.Tensor, t: float, eps: float = 1e-8) -> torch.Tensor:
    af, bf = a.float().flatten(), b.float().flatten()
    an, bn = af / (af.norm() + eps), bf / (bf.norm() + eps)
    dot = torch.clamp((an * bn).sum(), -1.0, 1.0)
    if dot.abs() > 0.9995:                       # nearly parallel: plain interpolation is the stable limit
        return ((1 - t) * af + t * bf).view_as(a)
    omega = torch.acos(dot)
    so = torch.sin(omega)
    return (torch.sin((1 - t) * omega) / so * af + torch.sin(t * omega) / so * bf).view_as(a)


def ties(base: torch.Tensor, tensors: list[torch.Tensor], density: float, weights: list[float]) -> torch.Tensor:
    b = base.float()
    deltas = []
    for t, w in zip(tensors, weights):
        d = (t.float() - b) * w
        k = max(1, int(density * d.numel()))
        if k < d.numel():
            thresh = d.abs().flatten().kthvalue(d.numel() - k + 1).values
            d = torch.where(d.abs() >= thresh, d, torch.zeros_like(d))
        deltas.append(d)
    stack = torch.stack(deltas)
    sign = torch.sign(stack.sum(0))
    agree = (torch.sign(stack) == sign) & (stack != 0)
    merged = (stack * agree).sum(0) / agree.sum(0).clamp_min(1)
    return b + merged


def merge(method: str, models: list[str], out: str, weights=None, t: float = 0.5, base: str | None = None,
          density: float = 0.2) -> int:
    idxs = [CheckpointIndex(m) for m in models]
    names = sorted(idxs[0].weight_map)
    for m, i in zip(models[1:], idxs[1:]):
        if sorted(i.weight_map) != names:
            raise ValueError(f"{m!r} does not hold the same tensors as {models[0]!r}")
    weights = list(weights) if weights else [1.0] * len(models)
    if len(weights) != len(models):
        raise ValueError("give one weight per model")
    base_idx = CheckpointIndex(base) if base else None
    if method == "slerp" and len(models) != 2:
        raise ValueError("slerp merges exactly two models")
    if method == "ties" and base_idx is None:
        raise ValueError("ties needs --base")
    writer = StreamingShardWriter(out)
    for name in names:
        ts = [i.get(name) for i in idxs]
        if not ts[0].is_floating_point():
            merged = ts[0]
        elif method == "linear":
            merged = linear(ts, weights)
        elif method == "slerp":
            merged = slerp(ts[0], ts[1], t)
        elif method == "ties":
            merged = ties(base_idx.get(name), ts, density, weights)
        else:
            raise ValueError(f"unknown merge method {method!r}")
        writer.add(name, merged.to(ts[0].dtype))
    writer.finish()
    copy_side_files(models[0], out)
    return len(names)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="merge checkpoints in weight space")
    ap.add_argument("models", nargs="+")
    ap.add_argument("--out", required=True)
    ap.add_argument("--method", default="linear", choices=["linear", "slerp", "ties"])
    ap.add_argument("--weights", type=float, nargs="*")
    ap.add_argument("--t", type=float, default=0.5)
    ap.add_argument("--base")
    ap.add_argument("--density", type=float, default=0.2)
    a = ap.parse_args(argv)
    n = merge(a.method, a.models, a.out, a.weights, a.t, a.base, a.density)
    print(f"merged {n} tensors into {a.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
