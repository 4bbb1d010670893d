"""Block-sparse causal attention: a query attends a few selected *compression blocks* of ``ratio`` keys of its document
plus the keys after its last complete block (the tail), the pattern of the sparse-attention decoder families.

    spans[t]  = (first, visible): the document's first position and how many of its keys query ``t`` may see
    blocks[t] = ``block_topk`` block indices inside the document; only the first ``min(visible // ratio, block_topk)``
                slots are used
    keys(t)   = U_slots { first + block * ratio + 0 .. ratio - 1 }  U  { first + (visible // ratio) * ratio .. first + visible - 1 }

This module states the op with tensor ops (the keys of a chunk of queries are gathered and a dense masked softmax
runs over them; autograd provides the backward) and is the oracle any kernel for it must match. No sm_100a kernel is
built for it yet: on a GPU it runs these ops, chunked so that the gathered keys stay within ``chunk_queries`` rows.
The reference's Triton kernel is halo/kernels/block_sparse_attention.py:138-303.
"""

from __future__ import annotations

import torch


def key_positions(spans: torch.Tensor, blocks: torch.Tensor, ratio: int):
    """``(positions [T, topk * ratio + ratio] int64, valid [T, same] bool)`` of the keys every query attends."""
    T, topk = blocks.shape
    first, visible = spans[:, 0].long(), spans[:, 1].long()
    complete = visible // ratio
    selected = torch.minimum(complete, torch.full_like(complete, topk))
    within = torch.arange(ratio, device=spans.device)
    slot = torch.arange(topk, device=spans.device)
    pos_blocks = first[:, None, None] + blocks.long()[:, :, None] * ratio + within[None, None, :]          # [T, topk, ratio]
    ok_blocks = (slot[None, :] < selected[:, None])[:, :, None].expand(T, topk, ratio)
    pos_tail = first[:, None] + complete[:, None] * ratio + within[None, :]                                  # [T, ratio]
    ok_tail = within[None, :] < (visible - complete * ratio)[:, None]
    pos = torch.cat([pos_blocks.reshape(T, topk * ratio), pos_tail], dim=1)
    ok = torch.cat([ok_blocks.reshape(T, topk * ratio), ok_tail], dim=1)
    return torch.where(ok, pos, torch.zeros_like(pos)), ok


def block_sparse_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, spans: torch.Tensor, blocks: torch.Tensor,
                           ratio: int, scale: float | None = None, chunk_queries: int = 2048) -> torch.Tensor:
    """``q [T, Hq, D]``, ``k`` / ``v [T, Hkv, D]`` (one packed row), ``spans [T, 2]``, ``blocks [T, block_topk]`` ->
    ``[T, Hq, D]``. A query with no visible key returns zeros. Duplicate block indices count twice, as in the
    kernel this restates."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    if Hq % Hkv:
        raise ValueError(f"{Hq} query heads do not group over {Hkv} key/value heads")
    G = Hq // Hkv
    scale = D ** -0.5 if scale is None else scale
    out = []
    for lo in range(0, T, chunk_queries):
        hi = min(lo + chunk_queries, T)
        pos, ok = key_positions(spans[lo:hi], blocks[lo:hi], ratio)
        kk, vv = k[pos], v[pos]                                           # [t, n, Hkv, D]
        qq = q[lo:hi].reshape(hi - lo, Hkv, G, D).float()
        scores = torch.einsum("thgd,tnhd->thgn", qq, kk.float()) * scale
        scores = scores.masked_fill(~ok[:, None, None, :], float("-inf"))
        any_key = ok.any(-1)[:, None, None, None]
        probs = torch.softmax(torch.where(any_key, scores, torch.zeros_like(scores)), dim=-1)
        probs = torch.where(any_key & ok[:, None, None, :], probs, torch.zeros_like(probs))
        out.append(torch.einsum("thgn,tnhd->thgd", probs, vv.float()).reshape(hi - lo, Hq, D).to(q.dtype))
    return torch.cat(out, dim=0)


def dense_reference(q, k, v, spans, blocks, ratio, scale=None):
    """The same attention written as a dense ``[T, T]`` mask (for tests: every selected key marked, then an ordinary
    masked softmax). Duplicate blocks must not occur in inputs compared with this form."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    pos, ok = key_positions(spans, blocks, ratio)
    mask = torch.zeros(T, T, dtype=torch.bool, device=q.device)
    rows = torch.arange(T, device=q.device)[:, None].expand_as(pos)
    mask[rows[ok], pos[ok]] = True
    kk = k.repeat_interleave(Hq // Hkv, dim=1).float()
    vv = v.repeat_interleave(Hq // Hkv, dim=1).float()
    scores = torch.einsum("thd,shd->hts", q.float(), kk) * (D ** -0.5 if scale is None else scale)
    scores = scores.masked_fill(~mask[None], float("-inf"))
    probs = torch.nan_to_num(torch.softmax(scores, dim=-1), nan=0.0)
    return torch.einsum("hts,shd->thd", probs, vv).to(q.dtype)
