"""Attention under an arbitrary boolean ``[Q, K]`` mask (the sparse-index attention of the DSA families, tree
attention over shared prefixes, windows): tiles of queries over the keys, with a closed-form backward that keeps no
probabilities - a tile's scores are recomputed, :func:`halo_b200.ops.streams.masked_softmax_backward` turns them into
the probabilities and the score cotangent in one pass (its sm_100a kernel on CUDA), and three products give the
gradients.

    out = softmax(mask(q k^T * scale)) v        per head, GQA by head grouping
    delta = sum(out * d_out)                    (row-wise)
    d_scores = P * (d_out v^T - delta) * scale;   d_v = P^T d_out;   d_q = d_scores k;   d_k = d_scores^T q

The products are plain batched GEMMs (library), the element-wise half is the kernel. Memory per tile:
``heads x tile x K`` fp32 scores, bounded by ``scores_per_tile``. A query whose mask row is empty returns zeros.
The reference's masked-matmul attention: halo/models/attention/masked_matmul.py.
"""

from __future__ import annotations

import torch

from .streams import masked_softmax_backward

SCORES_PER_TILE = 1 << 26


def masked_attention_reference(q, k, v, allowed, scale=None, sinks=None, softcap=0.0):
    """``q [Q, Hq, D]``, ``k`` / ``v [K, Hkv, D]``, ``allowed [Q, K]`` bool -> ``[Q, Hq, D]`` (plain autograd form)."""
    Hq, Hkv, D = q.shape[1], k.shape[1], q.shape[2]
    kk, vv = (t.repeat_interleave(Hq // Hkv, dim=1).float() for t in (k, v))
    scores = torch.einsum("qhd,khd->hqk", q.float(), kk) * (D ** -0.5 if scale is None else scale)
    if softcap:
        scores = softcap * torch.tanh(scores / softcap)
    scores = scores.masked_fill(~allowed[None], float("-inf"))
    if sinks is not None:
        joined = torch.cat([scores, sinks.float()[:, None, None].expand(-1, scores.shape[1], 1)], dim=-1)
        probs = torch.softmax(joined, dim=-1)[..., :-1]
    else:
        probs = torch.nan_to_num(torch.softmax(scores, dim=-1), nan=0.0)
    return torch.einsum("hqk,khd->qhd", probs, vv).to(q.dtype)


def _tiles(n_queries: int, n_keys: int, heads: int, budget: int):
    step = max(8, budget // max(1, heads * n_keys) // 8 * 8)
    return [(lo, min(lo + step, n_queries)) for lo in range(0, n_queries, step)]


class _MaskedAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, allowed, scale, budget, sinks=None, softcap=0.0):
        Q, Hq, D = q.shape
        K, Hkv = k.shape[0], k.shape[1]
        G = Hq // Hkv
        kh = k.permute(1, 0, 2)                                             # [Hkv, K, D]
        vh = v.permute(1, 0, 2)
        out = torch.empty_like(q)
        lse = torch.empty((Hq, Q), dtype=torch.float32, device=q.device)
        for lo, hi in _tiles(Q, K, Hq, budget):
            qt = q[lo:hi].permute(1, 0, 2).reshape(Hkv, G * (hi - lo), D)    # heads of a group share their keys
            scores = torch.bmm(qt.float(), kh.float().transpose(1, 2)).reshape(Hq, hi - lo, K) * scale
            if softcap:
                scores = softcap * torch.tanh(scores / softcap)             # tanh soft-capping of the scaled scores (Gemma 2)
            scores = scores.masked_fill(~allowed[lo:hi][None], float("-inf"))
            tile_lse = torch.logsumexp(scores, dim=-1)
            if sinks is not None:
                # an attention sink: one learned logit per head joins every softmax (and takes its share of the mass)
                tile_lse = torch.logaddexp(tile_lse, sinks.float()[:, None].expand_as(tile_lse))
            tile_lse = torch.where(torch.isinf(tile_lse), torch.zeros_like(tile_lse), tile_lse)     # empty rows: exp(-inf - 0) = 0
            probs = torch.exp(scores - tile_lse[..., None])
            o = torch.bmm(probs.reshape(Hkv, G * (hi - lo), K), vh.float()).reshape(Hq, hi - lo, D)
            out[lo:hi] = o.permute(1, 0, 2).to(q.dtype)
            lse[:, lo:hi] = tile_lse
        ctx.save_for_backward(q, k, v, allowed, out, lse, sinks if sinks is not None else q.new_zeros(0))
        ctx.meta = (scale, budget, sinks is not None, softcap)
        return out

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, allowed, out, lse, sinks = ctx.saved_tensors
        scale, budget, has_sinks, softcap = ctx.meta
        Q, Hq, D = q.shape
        K, Hkv = k.shape[0], k.shape[1]
        G = Hq // Hkv
        kh, vh = k.permute(1, 0, 2).float(), v.permute(1, 0, 2).float()
        dq = torch.empty_like(q)
        dk = torch.zeros((Hkv, K, D), dtype=torch.float32, device=q.device)
        dv = torch.zeros((Hkv, K, D), dtype=torch.float32, device=q.device)
        delta = (out.float() * d_out.float()).sum(-1).t().contiguous()       # [Hq, Q]
        for lo, hi in _tiles(Q, K, Hq, budget):
            n = hi - lo
            qt = q[lo:hi].permute(1, 0, 2).reshape(Hkv, G * n, D).float()
            gt = d_out[lo:hi].permute(1, 0, 2).reshape(Hkv, G * n, D).float()
            raw = torch.bmm(qt, kh.transpose(1, 2)).reshape(Hq, n, K).contiguous()           # unscaled scores
            upstream = torch.bmm(gt, vh.transpose(1, 2)).reshape(Hq, n, K).contiguous()      # d_out v^T
            if softcap:
                # the softmax saw cap * tanh(raw * scale / cap): its backward runs on the capped scores (scale 1) and
                # the chain rule through the cap multiplies by (1 - tanh^2) * scale
                t = torch.tanh(raw * (scale / softcap))
                probs, d_scores = masked_softmax_backward(t * softcap, allowed[lo:hi], lse[:, lo:hi].contiguous(), 1.0, upstream,
                                                          delta[:, lo:hi].contiguous(), True, torch.float32)
                d_scores = d_scores * ((1.0 - t * t) * scale)
            else:
                probs, d_scores = masked_softmax_backward(raw, allowed[lo:hi], lse[:, lo:hi].contiguous(), scale, upstream,
                                                          delta[:, lo:hi].contiguous(), True, torch.float32)
            probs, d_scores = probs.reshape(Hkv, G * n, K), d_scores.reshape(Hkv, G * n, K)
            dv += torch.bmm(probs.transpose(1, 2), gt)
            dk += torch.bmm(d_scores.transpose(1, 2), qt)
            dq[lo:hi] = torch.bmm(d_scores, kh).reshape(Hq, n, D).permute(1, 0, 2).to(q.dtype)
        dsinks = None
        if has_sinks:
            # the sink's probability is exp(sink - lse) and its "value" is zero: d sink = -sum_q p_sink * delta
            dsinks = -(torch.exp(sinks.float()[:, None] - lse) * delta).sum(-1).to(sinks.dtype)
        return dq, dk.permute(1, 0, 2).to(k.dtype), dv.permute(1, 0, 2).to(v.dtype), None, None, None, dsinks, None


def masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, allowed: torch.Tensor, scale: float | None = None,
                     scores_per_tile: int = SCORES_PER_TILE, sinks: torch.Tensor | None = None, softcap: float = 0.0) -> torch.Tensor:
    """``q [Q, Hq, D]``, ``k`` / ``v [K, Hkv, D]``, ``allowed [Q, K]`` bool -> ``[Q, Hq, D]``. ``sinks [Hq]``: one learned
    logit per head that joins every row's softmax without a value (attention sinks). ``softcap``: the scaled scores pass
    through ``softcap * tanh(. / softcap)`` before the mask."""
    if q.shape[1] % k.shape[1]:
        raise ValueError(f"{q.shape[1]} query heads do not group over {k.shape[1]} key/value heads")
    if tuple(allowed.shape) != (q.shape[0], k.shape[0]):
        raise ValueError(f"mask {tuple(allowed.shape)} where queries and keys give {(q.shape[0], k.shape[0])}")
    scale = q.shape[2] ** -0.5 if scale is None else scale
    return _MaskedAttention.apply(q, k, v, allowed.bool(), float(scale), scores_per_tile, sinks, float(softcap or 0.0))


def tree_mask(parent: torch.Tensor) -> torch.Tensor:
    """``allowed[i, j]`` = token ``j`` lies on token ``i``'s root-to-leaf path (itself included), for a packed tree
    given as ``parent[i]`` (-1 at a root; a parent precedes its children). Completions that share a prompt are
    branches of one tree: the prompt is stored and attended once."""
    n = parent.shape[0]
    allowed = torch.eye(n, dtype=torch.bool, device=parent.device)
    for i in range(n):
        p = int(parent[i])
        if p >= 0:
            if p >= i:
                raise ValueError("a parent must precede its children")
            allowed[i] |= allowed[p]
    return allowed


def window_mask(cu_seqlens, window: int, device=None) -> torch.Tensor:
    """Causal attention inside each packed document, limited to the last ``window`` keys."""
    cu = [int(x) for x in cu_seqlens]
    n = cu[-1]
    pos = torch.arange(n, device=device)
    doc = torch.bucketize(pos, torch.tensor(cu[1:], device=device), right=True)
    same = doc[:, None] == doc[None, :]
    return same & (pos[None, :] <= pos[:, None]) & (pos[None, :] > pos[:, None] - window)
