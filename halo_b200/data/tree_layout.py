"""Prefix-sharing tree packing: the completions sampled for one prompt become branches of one tree whose trunk - the
prompt - is stored, embedded and attended once instead of once per completion.

A tree is laid out as ``prompt[:-1]`` followed by one segment per completion, each starting with a copy of the prompt's
last token: that token is where the branches diverge (its successor differs per branch), so it must exist once per
branch for every branch's first token to be a next-token target. Positions continue from the trunk inside every
branch; a token attends the trunk and the earlier tokens of its own branch. With ``G`` completions of a ``P``-token
prompt a row holds ``(G - 1) (P - 1)`` fewer tokens than flat packing.

The role of the reference's tree packing (halo/data/tree_layout.py, halo/models/attention/tree_plan.py); the mask
is served by :func:`halo_b200.ops.masked_attention.masked_attention`.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

IGNORE = -100


@dataclass
class TreeLayout:
    input_ids: torch.Tensor        # [T]
    position_ids: torch.Tensor     # [T] int32
    labels: torch.Tensor           # [T] next token along the token's own branch, -100 on the trunk and at branch ends
    cu_seqlens: np.ndarray         # one "document" per tree (rotary / norm bookkeeping only; the mask decides attention)
    allowed: torch.Tensor          # [T, T] bool
    branch_slices: list            # per tree: list of (start, stop) of each branch's completion tokens (copy of the fork token excluded)
    flat_tokens: int               # what flat packing would have taken


def pack_trees(groups: list, completion_masks: list | None = None) -> TreeLayout:
    """``groups``: ``[(prompt_ids, [completion_ids, ...]), ...]``. ``completion_masks``: per group, per completion, a bool
    array that is False where a completion token must not be a target (environment tokens)."""
    ids, pos, labels, cu, slices = [], [], [], [0], []
    segments = []                                     # (trunk_lo, trunk_hi, [(branch_lo, branch_hi), ...])
    flat = 0
    at = 0
    for gi, (prompt, completions) in enumerate(groups):
        prompt = np.asarray(prompt, dtype=np.int64)
        if len(prompt) < 1 or not completions:
            raise ValueError("a tree needs a prompt of at least one token and one completion")
        trunk = prompt[:-1]
        t_lo, t_hi = at, at + len(trunk)
        ids.append(trunk)
        pos.append(np.arange(len(trunk)))
        labels.append(np.full(len(trunk), IGNORE, dtype=np.int64))
        at = t_hi
        branches, own = [], []
        for ci, comp in enumerate(completions):
            comp = np.asarray(comp, dtype=np.int64)
            seg = np.concatenate([prompt[-1:], comp])
            lab = np.full(len(seg), IGNORE, dtype=np.int64)
            lab[:-1] = seg[1:]
            if completion_masks is not None:
                ok = np.asarray(completion_masks[gi][ci], dtype=bool)
                lab[:-1][~ok] = IGNORE
            ids.append(seg)
            pos.append(len(trunk) + np.arange(len(seg)))
            labels.append(lab)
            branches.append((at, at + len(seg)))
            own.append((at + 1, at + len(seg)))
            at += len(seg)
            flat += len(prompt) + len(comp)
        segments.append((t_lo, t_hi, branches))
        slices.append(own)
        cu.append(at)
    T = at
    allowed = torch.zeros(T, T, dtype=torch.bool)
    causal = torch.ones(T, T, dtype=torch.bool).tril_()
    for t_lo, t_hi, branches in segments:
        allowed[t_lo:t_hi, t_lo:t_hi] = causal[t_lo:t_hi, t_lo:t_hi]
        for b_lo, b_hi in branches:
            allowed[b_lo:b_hi, t_lo:t_hi] = True
            allowed[b_lo:b_hi, b_lo:b_hi] = causal[b_lo:b_hi, b_lo:b_hi]
    return TreeLayout(torch.from_numpy(np.concatenate(ids)), torch.from_numpy(np.concatenate(pos).astype(np.int32)),
                      torch.from_numpy(np.concatenate(labels)), np.asarray(cu, dtype=np.int64), allowed, slices, flat)
