"""Per-head q/k RMSNorm fused with rotate-half rotary embedding (the Qwen3 attention prologue).

``qk_norm_rope(qkv, wq, wk, table, ...)`` takes the fused projection ``[T, (Hq + 2 Hkv) * D]`` and
returns rotated ``q [T, Hq*D]`` and ``k [T, Hkv*D]``; ``v`` stays a strided view of ``qkv`` that the
attention kernel reads in place. The cos/sin table is computed once per batch from the packed
``position_ids`` and shared by every layer.

Stands where the reference applies Liger RoPE (or eager rotate-half under context parallelism,
halo/distributed/context_parallel/ulysses_attention.py:63-76) after the HF q_norm / k_norm modules.
"""

from __future__ import annotations

import torch

from . import _lib

HEAD_DIM = 128


def rope_table(position_ids: torch.Tensor, head_dim: int, theta: float) -> torch.Tensor:
    """``[T, head_dim/2, 2]`` fp32 (cos, sin), each rounded to bf16 as the HF module does."""
    pos = position_ids.reshape(-1)
    T = pos.shape[0]
    half = head_dim // 2
    if not pos.is_cuda:
        inv = theta ** (-torch.arange(0, half, dtype=torch.float32) * 2.0 / head_dim)
        ang = pos.float()[:, None] * inv[None, :]
        return torch.stack([ang.cos().bfloat16().float(), ang.sin().bfloat16().float()], dim=-1)
    table = torch.empty((T, half, 2), dtype=torch.float32, device=pos.device)
    pos32 = pos.to(torch.int32).contiguous()
    rc = _lib.lib().halo_rope_table(
        _lib.ptr(pos32), _lib.c_ll(T), _lib.c_int(head_dim), _lib.c_float(theta), _lib.ptr(table),
        _lib.stream_ptr(pos.device),
    )
    _lib.check(rc, "halo_rope_table")
    return table


def qk_norm_rope_reference(qkv, wq, wk, table, n_heads, n_kv_heads, eps, use_norm=True):
    T = qkv.shape[0]
    D = qkv.shape[1] // (n_heads + 2 * n_kv_heads)
    q = qkv[:, : n_heads * D].reshape(T, n_heads, D)
    k = qkv[:, n_heads * D : (n_heads + n_kv_heads) * D].reshape(T, n_kv_heads, D)
    cos = torch.cat([table[..., 0], table[..., 0]], dim=-1)[:, None, :].to(qkv.dtype)
    sin = torch.cat([table[..., 1], table[..., 1]], dim=-1)[:, None, :].to(qkv.dtype)

    def norm(x, w):
        if not use_norm:
            return x
        xf = x.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        return w * (xf * rstd).to(x.dtype)

    def rot(x):
        x1, x2 = x[..., : D // 2], x[..., D // 2 :]
        return (x * cos) + (torch.cat([-x2, x1], dim=-1) * sin)

    return rot(norm(q, wq)).reshape(T, n_heads * D), rot(norm(k, wk)).reshape(T, n_kv_heads * D)


class _QKNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, wq, wk, table, n_heads, n_kv_heads, eps, use_norm):
        T = qkv.shape[0]
        q = torch.empty((T, n_heads * HEAD_DIM), dtype=qkv.dtype, device=qkv.device)
        k = torch.empty((T, n_kv_heads * HEAD_DIM), dtype=qkv.dtype, device=qkv.device)
        rstd = torch.empty(T * (n_heads + n_kv_heads), dtype=torch.float32, device=qkv.device)
        rc = _lib.lib().halo_qknorm_rope_fwd(
            _lib.ptr(qkv), _lib.ptr(wq), _lib.ptr(wk), _lib.ptr(table), _lib.ptr(q), _lib.ptr(k), _lib.ptr(rstd),
            _lib.c_ll(T), _lib.c_int(n_heads), _lib.c_int(n_kv_heads), _lib.c_int(HEAD_DIM), _lib.c_float(eps),
            _lib.c_int(1 if use_norm else 0), _lib.stream_ptr(qkv.device),
        )
        _lib.check(rc, "halo_qknorm_rope_fwd")
        ctx.save_for_backward(qkv, wq, wk, table, rstd)
        ctx.meta = (n_heads, n_kv_heads, use_norm)
        return q, k

    @staticmethod
    def backward(ctx, dq, dk):
        qkv, wq, wk, table, rstd = ctx.saved_tensors
        n_heads, n_kv_heads, use_norm = ctx.meta
        T = qkv.shape[0]
        L = _lib.lib()
        dqkv = torch.empty_like(qkv)
        blocks = L.halo_qknorm_rope_bwd_blocks(_lib.c_ll(T), _lib.c_int(n_heads + n_kv_heads))
        partial = torch.empty((max(blocks, 1), 256), dtype=torch.float32, device=qkv.device)
        dw = torch.zeros(256, dtype=torch.float32, device=qkv.device)
        rc = L.halo_qknorm_rope_bwd(
            _lib.ptr(dq.contiguous()), _lib.ptr(dk.contiguous()), _lib.ptr(qkv), _lib.ptr(wq), _lib.ptr(wk),
            _lib.ptr(table), _lib.ptr(rstd), _lib.ptr(dqkv), _lib.ptr(partial), _lib.ptr(dw), _lib.c_void_p(0),
            _lib.c_int(0), _lib.c_ll(T), _lib.c_int(n_heads), _lib.c_int(n_kv_heads), _lib.c_int(HEAD_DIM),
            _lib.c_int(1 if use_norm else 0), _lib.stream_ptr(qkv.device),
        )
        _lib.check(rc, "halo_qknorm_rope_bwd")
        # the v columns of dqkv are left for the attention backward's dv, which the caller adds
        dqkv[:, (n_heads + n_kv_heads) * HEAD_DIM :].zero_()
        dwq = dw[:128].to(wq.dtype) if use_norm else None
        dwk = dw[128:].to(wk.dtype) if use_norm else None
        return dqkv, dwq, dwk, None, None, None, None, None


def qk_norm_rope(qkv, wq, wk, table, n_heads, n_kv_heads, eps=1e-6, use_norm=True):
    D = qkv.shape[1] // (n_heads + 2 * n_kv_heads)
    if not qkv.is_cuda or D != HEAD_DIM or qkv.dtype != torch.bfloat16:
        return qk_norm_rope_reference(qkv, wq, wk, table, n_heads, n_kv_heads, eps, use_norm)
    return _QKNormRope.apply(qkv.contiguous(), wq, wk, table, n_heads, n_kv_heads, eps, use_norm)
