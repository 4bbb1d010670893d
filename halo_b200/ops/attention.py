"""Causal attention over packed rows (documents delimited by ``cu_seqlens``), grouped-query heads.

On a GPU the tcgen05 flash kernels run (forward + the two deterministic backward kernels); the
tile work lists are built once per batch on the host from ``cu_seqlens`` and ordered heaviest
first. On CPU tensors a plain fp32 per-document softmax attention runs, which is also the oracle
of the GPU tests.

Stands where the reference resolves an attention backend (FA4 / FA2 varlen) for packed rows
(halo/models/attention/selection.py:383-462, halo/models/attention/packed_position_ids.py).
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib

HEAD_DIM = 128
# 1: 128-key tiles, output rescaled in registers, one CTA per SM
# 2: 64-key tiles, output accumulated in TMEM with lazy rescale, two CTAs per SM
# 3: as 2, with the probabilities written to tensor memory (tcgen05.st) and read from there by the P V product
FWD_VARIANT = int(os.environ.get("HALO_ATTN_FWD_VARIANT", "3"))


def _launch_fwd(L, q, k, v, o, lse, plan, T, n_heads, n_kv_heads, scale, dev, sinks=None):
    if sinks is not None:
        # the sink logit joins the denominator in the forward kernel's last step (with or without a window)
        work = plan.bwd_q
        rc = L.halo_attn_fwd3_sinks(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(work),
            _lib.c_int(work.shape[0]), _lib.c_ll(T), _lib.c_int(n_heads), _lib.c_int(n_kv_heads),
            _lib.c_int(HEAD_DIM), _lib.c_ll(_ld(q)), _lib.c_ll(_ld(k)), _lib.c_ll(_ld(v)), _lib.c_ll(_ld(o)),
            _lib.c_float(scale), _lib.c_int(plan.window), _lib.ptr(sinks), _lib.ptr(_lib.status_word(dev)),
            _lib.stream_ptr(dev))
        _lib.check(rc, "halo_attn_fwd3_sinks")
        return
    if plan.window:
        work = plan.bwd_q
        rc = L.halo_attn_fwd3_window(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(work),
            _lib.c_int(work.shape[0]), _lib.c_ll(T), _lib.c_int(n_heads), _lib.c_int(n_kv_heads),
            _lib.c_int(HEAD_DIM), _lib.c_ll(_ld(q)), _lib.c_ll(_ld(k)), _lib.c_ll(_ld(v)), _lib.c_ll(_ld(o)),
            _lib.c_float(scale), _lib.c_int(plan.window), _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(dev))
        _lib.check(rc, "halo_attn_fwd3_window")
        return
    if FWD_VARIANT == 3:
        work, fn, what = plan.bwd_q, L.halo_attn_fwd3, "halo_attn_fwd3"
    elif FWD_VARIANT == 2:
        work, fn, what = plan.bwd_q, L.halo_attn_fwd2, "halo_attn_fwd2"
    else:
        work, fn, what = plan.fwd, L.halo_attn_fwd, "halo_attn_fwd"
    rc = fn(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(work),
        _lib.c_int(work.shape[0]), _lib.c_ll(T), _lib.c_int(n_heads), _lib.c_int(n_kv_heads),
        _lib.c_int(HEAD_DIM), _lib.c_ll(_ld(q)), _lib.c_ll(_ld(k)), _lib.c_ll(_ld(v)), _lib.c_ll(_ld(o)),
        _lib.c_float(scale), _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(dev),
    )
    _lib.check(rc, what)


def _launch_bwd(L, q, k, v, o, do, lse, delta, dq, dk, dv, plan, T, n_heads, n_kv_heads, scale, dev):
    args = [
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(do), _lib.ptr(lse), _lib.ptr(delta),
        _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv),
        _lib.ptr(plan.bwd_kv), _lib.c_int(plan.bwd_kv.shape[0]),
        _lib.ptr(plan.bwd_q), _lib.c_int(plan.bwd_q.shape[0]),
        _lib.c_ll(T), _lib.c_int(n_heads), _lib.c_int(n_kv_heads), _lib.c_int(HEAD_DIM),
        _lib.c_ll(_ld(q)), _lib.c_ll(_ld(k)), _lib.c_ll(_ld(v)), _lib.c_ll(_ld(o)), _lib.c_ll(_ld(do)),
        _lib.c_ll(_ld(dq)), _lib.c_ll(_ld(dk)), _lib.c_ll(_ld(dv)), _lib.c_float(scale)]
    if plan.window:
        rc = L.halo_attn_bwd_window(*args, _lib.c_int(plan.window), _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(dev))
        _lib.check(rc, "halo_attn_bwd_window")
        return
    rc = L.halo_attn_bwd(*args, _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(dev))
    _lib.check(rc, "halo_attn_bwd")


@dataclass
class AttentionPlan:
    """Tile work lists for one packed batch (device int32 tensors of shape [n, 4])."""

    cu_seqlens: np.ndarray  # host int64 [n_docs + 1]
    total: int
    fwd: torch.Tensor | None = None
    bwd_kv: torch.Tensor | None = None
    bwd_q: torch.Tensor | None = None
    max_seqlen: int = 0
    window: int = 0         # > 0: sliding-window attention (a query sees the last ``window`` keys up to itself)

    @property
    def n_docs(self) -> int:
        return len(self.cu_seqlens) - 1


def build_plan(cu_seqlens, device: torch.device | str | None = None, q_lo: int = 0, window: int = 0) -> AttentionPlan:
    """``cu_seqlens``: increasing offsets ``[0, len0, len0+len1, ...]`` of the packed documents.

    ``window > 0``: sliding-window attention. The lists are cut to the window - a query tile starts at the first key tile its
    first row can see, a key tile's queries end ``window - 1`` rows after its last key - so the work (and the time) of a long
    document grows with ``window``, not with the document's length.

    ``q_lo``: rows below it are keys only (the foreign prefix of a context-parallel chunk): no query tile is
    listed for them, and the dK/dV lists start their query range at ``q_lo``. The caller keeps the query and
    output-gradient rows below ``q_lo`` at zero, so the rows of a tile that straddles ``q_lo`` add nothing."""
    cu = np.asarray(cu_seqlens.cpu() if isinstance(cu_seqlens, torch.Tensor) else cu_seqlens, dtype=np.int64)
    if cu.ndim != 1 or len(cu) < 1 or cu[0] != 0 or np.any(np.diff(cu) < 0):
        raise ValueError("cu_seqlens must start at 0 and be non-decreasing")
    total = int(cu[-1])
    if window and q_lo:
        raise ValueError("a sliding window together with a key-only prefix is not supported")
    plan = AttentionPlan(cu_seqlens=cu, total=total, window=int(window))
    lens = np.diff(cu)
    plan.max_seqlen = int(lens.max()) if len(lens) else 0
    device = torch.device(device) if device is not None else None
    fwd, bkv, bq = [], [], []
    for start, end in zip(cu[:-1], cu[1:]):
        n = int(end - start)
        if n == 0:
            continue
        if int(end) <= q_lo:
            continue                      # a document that lies wholly in the prefix has no local queries
        for i in range((n + 127) // 128):
            q0 = int(start) + 128 * i
            last = min(q0 + 128, int(end))
            if window:
                # the first key tile the tile's first row sees, aligned to 64 rows from the document's start
                k_first = int(start) + max(0, q0 - window + 1 - int(start)) // 64 * 64
                bq.append((q0, k_first, (last - k_first + 63) // 64, int(end)))
                fwd.append((q0, k_first, (last - k_first + 127) // 128, int(end)))
                # queries that see the key tile end window - 1 rows after its last key
                q_stop = min(int(end), q0 + 127 + window)
                bkv.append((q0, q0, (q_stop - q0 + 63) // 64, int(end)))
                continue
            if last > q_lo:
                fwd.append((q0, int(start), i + 1, int(end)))
                # dQ: 64-key sub-tiles up to the tile's last visible key
                bq.append((q0, int(start), (last - int(start) + 63) // 64, int(end)))
            # dK/dV: 64-query sub-tiles from the key tile's first row (or the first local query) to the document end
            qb = max(q0, (q_lo - int(start)) // 64 * 64 + int(start)) if q_lo > q0 else q0
            bkv.append((q0, qb, (int(end) - qb + 63) // 64, int(end)))

    plan.host_lists = {"fwd": fwd, "bwd_kv": bkv, "bwd_q": bq}          # the lists as built, for inspection and tests
    if device is None or device.type != "cuda":
        return plan

    def to_dev(rows, key):
        if not rows:
            return torch.zeros((0, 4), dtype=torch.int32, device=device)
        arr = np.asarray(rows, dtype=np.int32)
        arr = arr[np.argsort(-arr[:, key], kind="stable")]
        return torch.from_numpy(arr).to(device, non_blocking=True)

    plan.fwd = to_dev(fwd, 2)
    plan.bwd_q = to_dev(bq, 2)
    plan.bwd_kv = to_dev(bkv, 2)
    return plan


def attention_reference(q, k, v, cu_seqlens, n_heads, n_kv_heads, scale=None, window: int = 0, sinks=None):
    """fp32 oracle. q: [T, Hq*D]; k, v: [T, Hkv*D]; returns [T, Hq*D] in q's dtype. ``window > 0``: a query sees the last
    ``window`` keys up to itself. ``sinks [Hq]``: one logit per head that joins every row's softmax and carries no value."""
    T = q.shape[0]
    D = q.shape[1] // n_heads
    scale = scale if scale is not None else D**-0.5
    qf = q.float().reshape(T, n_heads, D)
    kf = k.float().reshape(T, n_kv_heads, D)
    vf = v.float().reshape(T, n_kv_heads, D)
    rep = n_heads // n_kv_heads
    out = torch.zeros_like(qf)
    cu = [int(x) for x in cu_seqlens]
    for s, e in zip(cu[:-1], cu[1:]):
        if e == s:
            continue
        qq = qf[s:e].transpose(0, 1)  # [H, n, D]
        kk = kf[s:e].transpose(0, 1).repeat_interleave(rep, dim=0)
        vv = vf[s:e].transpose(0, 1).repeat_interleave(rep, dim=0)
        sc = (qq @ kk.transpose(1, 2)) * scale
        n = e - s
        mask = torch.ones(n, n, dtype=torch.bool, device=q.device).tril()
        if window:
            mask &= ~torch.ones(n, n, dtype=torch.bool, device=q.device).tril(-int(window))
        sc = sc.masked_fill(~mask, float("-inf"))
        if sinks is not None:
            sc = torch.cat([sc, sinks.float()[:, None, None].expand(-1, n, 1)], dim=-1)
            out[s:e] = (torch.softmax(sc, dim=-1)[..., :n] @ vv).transpose(0, 1)
        else:
            out[s:e] = (torch.softmax(sc, dim=-1) @ vv).transpose(0, 1)
    return out.reshape(T, n_heads * D).to(q.dtype)


def _sink_grad(sinks, lse, delta):
    """Gradient of the sink logits from what the backward kernels leave behind: the sink's probability in row t of head
    h is exp(sink_h - lse[h, t]) and its value vector is zero, so dS_sink = -P_sink * delta with delta = rowsum(dO * O)."""
    return -(torch.exp(sinks[:, None] - lse) * delta).sum(dim=1)


def _ld(t: torch.Tensor) -> int:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError("attention operands must be 2-D with contiguous rows")
    return t.stride(0)


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, plan: AttentionPlan, n_heads: int, n_kv_heads: int, scale: float, sinks=None):
        T = q.shape[0]
        o = torch.empty((T, n_heads * HEAD_DIM), dtype=torch.bfloat16, device=q.device)
        lse = torch.empty((n_heads, T), dtype=torch.float32, device=q.device)
        _launch_fwd(_lib.lib(), q, k, v, o, lse, plan, T, n_heads, n_kv_heads, scale, q.device, sinks)
        ctx.save_for_backward(q, k, v, o, lse, sinks)
        ctx.plan, ctx.n_heads, ctx.n_kv_heads, ctx.scale = plan, n_heads, n_kv_heads, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, sinks = ctx.saved_tensors
        plan = ctx.plan
        T = q.shape[0]
        do = do.contiguous()
        dq = torch.empty((T, ctx.n_heads * HEAD_DIM), dtype=torch.bfloat16, device=q.device)
        dkv = torch.empty((T, 2 * ctx.n_kv_heads * HEAD_DIM), dtype=torch.bfloat16, device=q.device)
        dk = dkv[:, : ctx.n_kv_heads * HEAD_DIM]
        dv = dkv[:, ctx.n_kv_heads * HEAD_DIM :]
        delta = torch.empty((ctx.n_heads, T), dtype=torch.float32, device=q.device)
        L = _lib.lib()
        _launch_bwd(L, q, k, v, o, do, lse, delta, dq, dk, dv, plan, T, ctx.n_heads, ctx.n_kv_heads, ctx.scale, q.device)
        dsinks = _sink_grad(sinks, lse, delta) if sinks is not None and ctx.needs_input_grad[7] else None
        return dq, dk, dv, None, None, None, None, dsinks


PADDED_HEAD_DIMS = (64,)


def _pad_heads(t, n, D):
    """[T, n*D] -> [T, n*128] with each head's columns D..127 zero."""
    return torch.nn.functional.pad(t.reshape(t.shape[0], n, D), (0, HEAD_DIM - D)).reshape(t.shape[0], n * HEAD_DIM)


def flash_attention(q, k, v, plan: AttentionPlan, n_heads: int, n_kv_heads: int, scale: float | None = None, sinks=None):
    """q: [T, Hq*D]; k, v: [T, Hkv*D] (row-strided views are fine); returns [T, Hq*D]. ``sinks [Hq]``: one logit per head
    that joins every row's softmax (and gets a gradient). D is 128; heads of 64 run on the same kernels with columns
    64..127 of every head zero (scores and outputs are unchanged by zero columns; the tensor work is that of 128-wide
    heads, memory stays linear in the row length)."""
    D = q.shape[1] // n_heads
    scale = float(scale if scale is not None else D**-0.5)
    if not q.is_cuda:
        return attention_reference(q, k, v, plan.cu_seqlens, n_heads, n_kv_heads, scale, window=plan.window, sinks=sinks)
    if D in PADDED_HEAD_DIMS and q.dtype == torch.bfloat16:
        o = flash_attention(_pad_heads(q, n_heads, D), _pad_heads(k, n_kv_heads, D), _pad_heads(v, n_kv_heads, D), plan,
                            n_heads, n_kv_heads, scale, sinks)
        return o.reshape(-1, n_heads, HEAD_DIM)[:, :, :D].reshape(-1, n_heads * D)
    if D != HEAD_DIM:
        raise NotImplementedError("the sm_100a flash kernels are built for head_dim 128 (and 64, zero-padded)")
    if plan.fwd is None:
        raise ValueError("the attention plan was built without a CUDA device")
    if sinks is not None:
        sinks = sinks.float().contiguous()
    return _FlashAttention.apply(q, k, v, plan, n_heads, n_kv_heads, scale, sinks)


class _RopeAttention(torch.autograd.Function):
    """q/k norm + RoPE + flash attention on the fused ``qkv`` projection, as one autograd node.

    The backward writes dq / dk (through the rotation and norm) and dv straight into the columns
    of one ``dqkv`` buffer, so no gradient is sliced, zero-filled or re-added by autograd.
    """

    @staticmethod
    def forward(ctx, qkv, wq, wk, table, plan, n_heads, n_kv_heads, eps, use_norm, scale, sinks=None):
        T = qkv.shape[0]
        dev = qkv.device
        L = _lib.lib()
        q = torch.empty((T, n_heads * HEAD_DIM), dtype=torch.bfloat16, device=dev)
        k = torch.empty((T, n_kv_heads * HEAD_DIM), dtype=torch.bfloat16, device=dev)
        rstd = torch.empty(T * (n_heads + n_kv_heads), dtype=torch.float32, device=dev)
        rc = L.halo_qknorm_rope_fwd(
            _lib.ptr(qkv), _lib.ptr(wq), _lib.ptr(wk), _lib.ptr(table), _lib.ptr(q), _lib.ptr(k), _lib.ptr(rstd),
            _lib.c_ll(T), _lib.c_int(n_heads), _lib.c_int(n_kv_heads), _lib.c_int(HEAD_DIM), _lib.c_float(eps),
            _lib.c_int(1 if use_norm else 0), _lib.stream_ptr(dev),
        )
        _lib.check(rc, "halo_qknorm_rope_fwd")
        v = qkv[:, (n_heads + n_kv_heads) * HEAD_DIM :]
        o = torch.empty((T, n_heads * HEAD_DIM), dtype=torch.bfloat16, device=dev)
        lse = torch.empty((n_heads, T), dtype=torch.float32, device=dev)
        _launch_fwd(L, q, k, v, o, lse, plan, T, n_heads, n_kv_heads, scale, dev, sinks)
        ctx.save_for_backward(qkv, wq, wk, table, q, k, o, lse, rstd, sinks)
        ctx.meta = (plan, n_heads, n_kv_heads, use_norm, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, wq, wk, table, q, k, o, lse, rstd, sinks = ctx.saved_tensors
        plan, n_heads, n_kv_heads, use_norm, scale = ctx.meta
        T = qkv.shape[0]
        dev = qkv.device
        L = _lib.lib()
        do = do.contiguous()
        v = qkv[:, (n_heads + n_kv_heads) * HEAD_DIM :]
        dqkv = torch.empty_like(qkv)
        dv = dqkv[:, (n_heads + n_kv_heads) * HEAD_DIM :]
        dq = torch.empty_like(q)
        dk = torch.empty_like(k)
        delta = torch.empty((n_heads, T), dtype=torch.float32, device=dev)
        _launch_bwd(L, q, k, v, o, do, lse, delta, dq, dk, dv, plan, T, n_heads, n_kv_heads, scale, dev)
        blocks = L.halo_qknorm_rope_bwd_blocks(_lib.c_ll(T), _lib.c_int(n_heads + n_kv_heads))
        partial = torch.empty((max(blocks, 1), 256), dtype=torch.float32, device=dev)
        dw = torch.zeros(256, dtype=torch.float32, device=dev)
        rc = L.halo_qknorm_rope_bwd(
            _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(qkv), _lib.ptr(wq), _lib.ptr(wk), _lib.ptr(table), _lib.ptr(rstd),
            _lib.ptr(dqkv), _lib.ptr(partial), _lib.ptr(dw), _lib.c_void_p(0), _lib.c_int(0), _lib.c_ll(T),
            _lib.c_int(n_heads), _lib.c_int(n_kv_heads), _lib.c_int(HEAD_DIM), _lib.c_int(1 if use_norm else 0),
            _lib.stream_ptr(dev),
        )
        _lib.check(rc, "halo_qknorm_rope_bwd")
        dwq = dw[:128].to(wq.dtype) if use_norm else None
        dwk = dw[128:].to(wk.dtype) if use_norm else None
        dsinks = _sink_grad(sinks, lse, delta) if sinks is not None and ctx.needs_input_grad[10] else None
        return dqkv, dwq, dwk, None, None, None, None, None, None, None, dsinks


def rope_attention(qkv, wq, wk, table, plan, n_heads, n_kv_heads, eps=1e-6, use_norm=True, scale=None, sinks=None):
    """``attention(rope(norm(q)), rope(norm(k)), v)`` from the fused projection ``qkv``; ``sinks [Hq]`` as in
    :func:`flash_attention`."""
    D = qkv.shape[1] // (n_heads + 2 * n_kv_heads)
    scale = float(scale if scale is not None else D**-0.5)
    per_head_norm = not use_norm or wq is None or wq.numel() == D
    if qkv.is_cuda and D == HEAD_DIM and qkv.dtype == torch.bfloat16 and 2 * table.shape[1] == D and per_head_norm:
        return _RopeAttention.apply(qkv.contiguous(), wq, wk, table, plan, n_heads, n_kv_heads, eps, use_norm, scale,
                                    None if sinks is None else sinks.float().contiguous())
    from .rope import qk_norm_rope_reference

    q, k = qk_norm_rope_reference(qkv, wq, wk, table, n_heads, n_kv_heads, eps, use_norm)
    v = qkv[:, (n_heads + n_kv_heads) * D :]
    if qkv.is_cuda and (D == HEAD_DIM or D in PADDED_HEAD_DIMS) and qkv.dtype == torch.bfloat16:
        # partial rotary / whole-width q-k norm / 64-wide heads: these run as tensor ops (the fused kernel norms and turns
        # whole 128-wide heads one by one), attention itself on the kernel
        return flash_attention(q, k, v, plan, n_heads, n_kv_heads, scale, sinks)
    return attention_reference(q, k, v, plan.cu_seqlens, n_heads, n_kv_heads, scale, window=plan.window, sinks=sinks)
