"""Multi-head latent attention (DeepSeek-V2 / V3, Mistral 4): queries pass through a low-rank bottleneck with its own RMSNorm,
keys and values are expanded from one shared latent vector per token, and the rotary embedding acts on a separate
slice of every query head and on ONE key slice shared by all heads.

    q      = q_b( norm( q_a(x) ) )                   [T, heads, nope + rope]      (or one plain q_proj)
    c, kr  = split( kv_a(x) )                        [T, latent], [T, rope]
    kn, v  = split( kv_b( norm(c) ) )                [T, heads, nope], [T, heads, v_dim]
    k      = concat( kn, rotate(kr) broadcast over heads ),   q = concat( q_nope, rotate(q_rope) )

The projections run on the framework's GEMM; attention itself goes through the masked-attention op (query tiles
under the causal mask of the packed documents) with the values zero-padded to the key width, because the flash
kernel is built for equal query / key / value widths of 128. Training, evaluation and cached generation (the cache
holds the expanded keys and padded values, not the latent vectors) on unsliced rows; no tensor or context parallelism
for this block.
(The role of the DeepSeek branch of halo/models/attention and ``family_specs.py``'s ``deepseek_v4`` entry.)"""

from __future__ import annotations

import math

import torch
from torch import nn

from halo_b200.ops import gemm
from halo_b200.ops.norm import rms_norm


def rotate(x: torch.Tensor, table: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """``x [T, heads, R]``, ``table [T, R/2, 2]`` (cos, sin). ``interleaved``: the pairs are stored (even, odd) and come
    out in halves, as the released checkpoints expect."""
    if interleaved:
        x = x.reshape(*x.shape[:-1], -1, 2).transpose(-1, -2).reshape(x.shape)
    half = x.shape[-1] // 2
    cos, sin = table[..., 0][:, None, :].to(x.dtype), table[..., 1][:, None, :].to(x.dtype)
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


class LatentAttention(nn.Module):
    def __init__(self, cfg, dtype, device, tp_size: int = 1, layer_idx: int = 0):
        super().__init__()
        if tp_size > 1:
            raise ValueError("latent attention is not cut over tensor-parallel ranks")
        self.cfg = cfg
        H, Hq = cfg.hidden_size, cfg.num_attention_heads
        self.nope, self.rope_dim, self.v_dim = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        self.qk_dim = self.nope + self.rope_dim

        def matrix(rows, cols):
            return nn.Parameter(torch.empty(rows, cols, dtype=dtype, device=device))

        if cfg.q_lora_rank:
            self.q_a_proj = matrix(cfg.q_lora_rank, H)
            self.q_a_norm = nn.Parameter(torch.ones(cfg.q_lora_rank, dtype=dtype, device=device))
            self.q_b_proj = matrix(Hq * self.qk_dim, cfg.q_lora_rank)
        else:
            self.q_proj = matrix(Hq * self.qk_dim, H)
        self.kv_a_proj = matrix(cfg.kv_lora_rank + self.rope_dim, H)
        self.kv_a_norm = nn.Parameter(torch.ones(cfg.kv_lora_rank, dtype=dtype, device=device))
        self.kv_b_proj = matrix(Hq * (self.nope + self.v_dim), cfg.kv_lora_rank)
        self.o_proj = matrix(H, Hq * self.v_dim)
        if cfg.index_topk:
            # sparse attention: a small indexer ranks the keys of every query and attention sees the best ``index_topk``.
            # The ranking is a hard choice (no gradient reaches these tensors through the loss), so they are held fixed
            if not cfg.q_lora_rank:
                raise ValueError("the indexer reads the low-rank query state: it needs q_lora_rank > 0")
            Hi, Di = cfg.index_n_heads, cfg.index_head_dim
            self.indexer_wq_b = matrix(Hi * Di, cfg.q_lora_rank)
            self.indexer_wk = matrix(Di, H)
            self.indexer_k_norm = nn.Parameter(torch.ones(Di, dtype=dtype, device=device))
            self.indexer_k_norm_bias = nn.Parameter(torch.zeros(Di, dtype=dtype, device=device))
            self.indexer_weights_proj = matrix(Hi, H)
            for p in (self.indexer_wq_b, self.indexer_wk, self.indexer_k_norm, self.indexer_k_norm_bias, self.indexer_weights_proj):
                p.requires_grad_(False)
        self.window, self.sinks, self.lora, self.lowp = 0, None, None, ""
        # yarn: the softmax temperature grows with the context extension (squared: it scales q and k); Mistral 4 keeps
        # the plain scale and stretches its queries by position instead (``ctx.query_scale``)
        self.scale = self.qk_dim ** -0.5
        rs = cfg.rope_scaling or {}
        if cfg.family not in ("mistral4", "glm_moe_dsa") and rs.get("rope_type", rs.get("type", "default")) != "default" and rs.get("mscale_all_dim"):
            factor = float(rs["factor"])
            m = 1.0 if factor <= 1.0 else 0.1 * float(rs["mscale_all_dim"]) * math.log(factor) + 1.0
            self.scale *= m * m

    @torch.no_grad()
    def selected_keys(self, h, q_low, rope, mask):
        """``[T, T]`` bool: for every query, the ``index_topk`` visible keys with the highest indexer score

            score[s, t] = sum over indexer heads of  weight[s, head] * relu(q[s, head] . k[t]) / sqrt(width)

        (all visible keys when there are fewer). The indexer turns the LEADING ``rope`` dims of its queries and of its one
        key per token, pairs stored in halves."""
        cfg = self.cfg
        T, Hi, Di, R = h.shape[0], cfg.index_n_heads, cfg.index_head_dim, self.rope_dim
        q = gemm.linear(q_low, self.indexer_wq_b).reshape(T, Hi, Di)
        k = torch.nn.functional.layer_norm(gemm.linear(h, self.indexer_wk).float(), (Di,), self.indexer_k_norm.float(),
                                           self.indexer_k_norm_bias.float(), 1e-6).to(h.dtype)
        q = torch.cat([rotate(q[..., :R], rope, False), q[..., R:]], dim=-1)
        k = torch.cat([rotate(k[:, None, :R], rope, False)[:, 0], k[:, R:]], dim=-1)
        weights = gemm.linear(h, self.indexer_weights_proj).float() * Hi ** -0.5
        scores = torch.relu(torch.einsum("shd,td->sht", q.float(), k.float()) * Di ** -0.5)
        ranked = torch.einsum("sht,sh->st", scores, weights).masked_fill(~mask, float("-inf"))
        top = ranked.topk(min(cfg.index_topk, T), dim=-1).indices
        return torch.zeros_like(mask).scatter_(1, top, True) & mask

    def forward(self, h, ctx):
        from halo_b200.ops.masked_attention import masked_attention, window_mask

        cfg = self.cfg
        if ctx.cp is not None or ctx.tp is not None:
            raise NotImplementedError("latent attention runs on unsliced rows")
        T, Hq = h.shape[0], cfg.num_attention_heads
        q_low = None
        if cfg.q_lora_rank:
            q_low = rms_norm(gemm.linear(h, self.q_a_proj), self.q_a_norm, cfg.rms_norm_eps)
            q = gemm.linear(q_low, self.q_b_proj)
        else:
            q = gemm.linear(h, self.q_proj)
        q = q.reshape(T, Hq, self.qk_dim)
        latent = gemm.linear(h, self.kv_a_proj)
        c, k_rope = latent[:, :cfg.kv_lora_rank], latent[:, cfg.kv_lora_rank:]
        kv = gemm.linear(rms_norm(c.contiguous(), self.kv_a_norm, cfg.rms_norm_eps), self.kv_b_proj).reshape(T, Hq, self.nope + self.v_dim)
        k_nope, v = kv[..., :self.nope], kv[..., self.nope:]
        q_rope = rotate(q[..., self.nope:], ctx.rope, cfg.rope_interleave)
        k_rope = rotate(k_rope.reshape(T, 1, self.rope_dim), ctx.rope, cfg.rope_interleave).expand(-1, Hq, -1)
        q = torch.cat([q[..., :self.nope], q_rope], dim=-1)
        k = torch.cat([k_nope, k_rope], dim=-1)
        if getattr(ctx, "query_scale", None) is not None:
            q = q * ctx.query_scale[:, None, None].to(q.dtype)
        if self.v_dim < self.qk_dim:
            v = torch.nn.functional.pad(v, (0, self.qk_dim - self.v_dim))       # the op takes one width; the pad is sliced off below
        cache = ctx.kv_cache
        if cache is not None:
            # generation: the expanded keys and padded values of this layer go to the cache; a decode step reads it
            li = cache.write(k.reshape(T, Hq * self.qk_dim), v.reshape(T, Hq * self.qk_dim))
            if cache.mode != "prefill":
                if cfg.index_topk and cache.k.shape[2] > cfg.index_topk:
                    raise NotImplementedError(f"cached decoding past index_topk ({cfg.index_topk}) keys: the indexer's key cache is "
                                              "not built; up to that length every key is selected and decoding is exact")
                o = cache.attend(li, q.reshape(T, Hq * self.qk_dim), Hq, scale=self.scale).reshape(T, Hq, self.qk_dim)
                return gemm.linear(o[..., :self.v_dim].reshape(T, Hq * self.v_dim), self.o_proj)
        mask = getattr(ctx, "attention_mask", None)
        if mask is None:
            if getattr(ctx, "causal", None) is None:
                ctx.causal = window_mask(ctx.plan.cu_seqlens, T, device=h.device)     # shared by the layers
            mask = ctx.causal
        elif mask.device != h.device:
            mask = ctx.attention_mask = mask.to(h.device)
        if cfg.index_topk:
            mask = self.selected_keys(h, q_low, ctx.rope, mask)
        o = masked_attention(q, k, v.contiguous(), mask, scale=self.scale)[..., :self.v_dim]
        return gemm.linear(o.reshape(T, Hq * self.v_dim), self.o_proj)
