"""Per-head q/k RMSNorm fused with rotate-half rotary embedding (the Qwen3 attention prologue).

``qk_norm_rope(qkv, wq, wk, table, ...)`` takes the fused projection ``[T, (Hq + 2 Hkv) * D]`` and
returns rotated ``q [T, Hq*D]`` and ``k [T, Hkv*D]``; ``v`` stays a strided view of ``qkv`` that the
attention kernel reads in place. The cos/sin table is computed once per batch from the packed
``position_ids`` and shared by every layer.

Stands where the reference applies Liger RoPE (or eager rotate-half under context parallelism,
halo/distributed/context_parallel/ulysses_attention.py:63-76) after the HF q_norm / k_norm modules.
"""

from __future__ import annotations

import json
import math

import torch

from . import _lib

HEAD_DIM = 128


def scaled_inverse_frequencies(head_dim: int, theta: float, scaling: dict, max_positions: int = 0):
    """Inverse frequencies ``[head_dim/2]`` (fp32, CPU) and the factor applied to cos / sin for a Hugging Face
    ``rope_scaling`` entry: ``linear`` (positions divided by ``factor``), ``llama3`` (low frequencies divided by
    ``factor``, a smooth ramp between the two wavelength bounds) and ``yarn`` (per-frequency blend of interpolation
    and extrapolation, with the attention temperature folded into cos / sin)."""
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    half = head_dim // 2
    inv = theta ** (-torch.arange(0, half, dtype=torch.float32) * 2.0 / head_dim)
    if kind == "default":
        return inv, 1.0
    factor = float(scaling["factor"])
    if kind == "linear":
        return inv / factor, 1.0
    if kind == "llama3":
        low, high = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        old = float(scaling["original_max_position_embeddings"])
        wavelen = 2.0 * math.pi / inv
        smooth = (old / wavelen - low) / (high - low)
        blended = (1.0 - smooth) * inv / factor + smooth * inv
        out = torch.where(wavelen > old / low, inv / factor, inv)
        mid = (wavelen <= old / low) & (wavelen >= old / high)
        return torch.where(mid, blended, out), 1.0
    if kind == "yarn":
        old = float(scaling.get("original_max_position_embeddings") or max_positions)
        beta_fast, beta_slow = float(scaling.get("beta_fast") or 32.0), float(scaling.get("beta_slow") or 1.0)
        mscale, mscale_all = scaling.get("mscale"), scaling.get("mscale_all_dim")

        def temperature(scale, m=1.0):
            return 1.0 if scale <= 1.0 else 0.1 * m * math.log(scale) + 1.0

        attention_factor = scaling.get("attention_factor")
        if attention_factor is None:
            attention_factor = (temperature(factor, mscale) / temperature(factor, mscale_all)
                                if mscale and mscale_all else temperature(factor))

        def correction_dim(rotations):
            return head_dim * math.log(old / (rotations * 2.0 * math.pi)) / (2.0 * math.log(theta))

        lo, hi = correction_dim(beta_fast), correction_dim(beta_slow)
        if scaling.get("truncate", True):
            lo, hi = math.floor(lo), math.ceil(hi)
        lo, hi = max(lo, 0), min(hi, head_dim - 1)
        if lo == hi:
            hi += 0.001
        ramp = ((torch.arange(half, dtype=torch.float32) - lo) / (hi - lo)).clamp(0, 1)
        extrapolation_share = 1.0 - ramp
        return (inv / factor) * (1.0 - extrapolation_share) + inv * extrapolation_share, float(attention_factor)
    raise ValueError(f"rope scaling of type {kind!r} is not built (known: default, linear, llama3, yarn)")


_SCALED_CACHE: dict = {}


def rope_table(position_ids: torch.Tensor, head_dim: int, theta: float, scaling: dict | None = None,
               max_positions: int = 0, round_bf16: bool = True) -> torch.Tensor:
    """``[T, head_dim/2, 2]`` fp32 (cos, sin), each rounded to bf16 as the HF module does for a bf16 model
    (``round_bf16=False``: an fp32 model keeps them exact, as HF does there). With ``scaling`` the frequencies come
    from :func:`scaled_inverse_frequencies` (built once per configuration, kept on the device)."""
    pos = position_ids.reshape(-1)
    T = pos.shape[0]
    half = head_dim // 2
    if scaling:
        key = (head_dim, theta, json.dumps(scaling, sort_keys=True), max_positions, str(pos.device))
        if key not in _SCALED_CACHE:
            inv, factor = scaled_inverse_frequencies(head_dim, theta, scaling, max_positions)
            _SCALED_CACHE[key] = (inv.to(pos.device), factor)
        inv, factor = _SCALED_CACHE[key]
        ang = pos.float()[:, None] * inv[None, :]
        cos, sin = ang.cos() * factor, ang.sin() * factor
        if round_bf16:
            cos, sin = cos.bfloat16().float(), sin.bfloat16().float()
        return torch.stack([cos, sin], dim=-1)
    if not pos.is_cuda:
        inv = theta ** (-torch.arange(0, half, dtype=torch.float32) * 2.0 / head_dim)
        ang = pos.float()[:, None] * inv[None, :]
        if not round_bf16:
            return torch.stack([ang.cos(), ang.sin()], dim=-1)
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
    R = 2 * table.shape[1]               # rotated dims of a head: all of them, or the leading part (partial rotary)
    q = qkv[:, : n_heads * D].reshape(T, n_heads, D)
    k = qkv[:, n_heads * D : (n_heads + n_kv_heads) * D].reshape(T, n_kv_heads, D)
    cos = torch.cat([table[..., 0], table[..., 0]], dim=-1)[:, None, :].to(qkv.dtype)
    sin = torch.cat([table[..., 1], table[..., 1]], dim=-1)[:, None, :].to(qkv.dtype)

    def norm(x, w):
        if not use_norm:
            return x
        xf = x.float()
        if w.numel() == x.shape[1] * x.shape[2]:
            # one norm over the whole projection (all heads together), as OLMoE does, instead of one per head
            flat = xf.reshape(T, -1)
            rstd = torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + eps)
            return (w * (flat * rstd).to(x.dtype)).reshape(x.shape)
        rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        return w * (xf * rstd).to(x.dtype)

    def rot(x):
        xr, rest = x[..., :R], x[..., R:]
        x1, x2 = xr[..., : R // 2], xr[..., R // 2 :]
        turned = (xr * cos) + (torch.cat([-x2, x1], dim=-1) * sin)
        return turned if R == D else torch.cat([turned, rest], dim=-1)

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
    whole_width_norm = use_norm and wq is not None and wq.numel() != D
    if not qkv.is_cuda or D != HEAD_DIM or qkv.dtype != torch.bfloat16 or 2 * table.shape[1] != D or whole_width_norm:
        return qk_norm_rope_reference(qkv, wq, wk, table, n_heads, n_kv_heads, eps, use_norm)
    return _QKNormRope.apply(qkv.contiguous(), wq, wk, table, n_heads, n_kv_heads, eps, use_norm)
