"""Sampling from the training model itself: batched generation with a key/value cache, for on-policy rollouts,
evaluation prompts and the example generations logged during training.

Prefill packs all prompts into ONE varlen row and runs the training kernels unchanged (flash attention over the
packed documents, grouped expert GEMMs); each layer's rotated keys and values are scattered into a padded cache
``[layers, batch, max_len, kv_heads, head_dim]`` on the way. A decode step feeds one token per sequence: the
projections, the router and the expert products are the same ops at ``T = batch``, and attention reads the cache -
one query row against its sequence's cached keys - with the decode kernel of ``csrc/decode_attention.cu`` (all query
heads of a key/value head in one CTA, the cache streamed once; batched tensor ops on CPU).
Sampling (temperature, top-k, nucleus) runs on the device in fp32 with a generator seeded per call; the sampled
token's log-probability under the *unmodified* distribution is returned for importance ratios.

The role of the reference's generation CLI and vLLM-backed rollouts
(halo/entrypoints/generation.py, halo/trainers/grpo/online.py), served here by the resident weights.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from halo_b200.ops import gemm
from halo_b200.ops.norm import rms_norm


@dataclass
class SamplingParams:
    max_new_tokens: int = 128
    temperature: float = 1.0          # 0 = greedy
    top_k: int = 0                    # 0 = off
    top_p: float = 1.0                # 1 = off
    stop_token_ids: tuple[int, ...] = ()
    seed: int | None = None


@dataclass
class Generation:
    prompt_ids: np.ndarray
    token_ids: np.ndarray             # generated tokens, the stop token included when one ended the sequence
    logprobs: np.ndarray              # log p(token) under the model's distribution at temperature 1
    finish_reason: str = "length"     # "stop" | "length"
    extra: dict = field(default_factory=dict)


class KVCache:
    """Padded per-sequence cache of rotated keys and values, filled layer by layer during a forward pass."""

    def __init__(self, n_layers: int, batch: int, max_len: int, n_kv_heads: int, head_dim: int, dtype, device):
        shape = (n_layers, batch, max_len, n_kv_heads, head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.lengths = torch.zeros(batch, dtype=torch.long, device=device)
        self.mode = "prefill"
        self._layer = 0
        self._rows = self._cols = None
        self._conv: dict[int, torch.Tensor] = {}      # layer index -> [batch, taps - 1, hidden]: a conv mixer's recent inputs
        self.recurrent: dict[int, torch.Tensor] = {}  # layer index -> [batch, heads, dk, dv]: a linear-attention layer's state

    def begin_prefill(self, seq_of_token: torch.Tensor, pos_of_token: torch.Tensor, lengths: torch.Tensor) -> None:
        self.mode, self._layer = "prefill", 0
        self._rows, self._cols = seq_of_token, pos_of_token
        self._prefill_lengths = lengths

    def end_prefill(self) -> None:
        self.lengths.copy_(self._prefill_lengths)

    def begin_decode(self) -> None:
        self.mode, self._layer = "decode", 0
        self._rows = torch.arange(self.lengths.shape[0], device=self.lengths.device)
        self._cols = self.lengths.clone()

    def end_decode(self) -> None:
        self.lengths += 1

    def conv_state(self, layer: int, depth: int, like: torch.Tensor) -> torch.Tensor:
        """The last ``depth`` inputs of a short-convolution layer per sequence, oldest first (zeros before a sequence's start)."""
        st = self._conv.get(layer)
        if st is None:
            st = self._conv[layer] = torch.zeros(self.k.shape[1], depth, like.shape[-1], dtype=like.dtype, device=like.device)
        return st

    def recurrent_state(self, layer: int, heads: int, dk: int, dv: int) -> torch.Tensor:
        st = self.recurrent.get(layer)
        if st is None:
            st = self.recurrent[layer] = torch.zeros(self.k.shape[1], heads, dk, dv, dtype=torch.float32, device=self.k.device)
        return st

    def store_conv_tail(self, layer: int, depth: int, x: torch.Tensor) -> None:
        """Prefill: keep every prompt's last ``depth`` rows of ``x [T, hidden]`` (packed prompts) for the decode steps."""
        st = self.conv_state(layer, depth, x)
        st.zero_()
        slot = self._cols - (self._prefill_lengths[self._rows] - depth)
        keep = slot >= 0
        st[self._rows[keep], slot[keep]] = x[keep]

    def write(self, k: torch.Tensor, v: torch.Tensor) -> int:
        """Store this layer's keys / values ``[T, kv_heads * head_dim]``; returns the layer's index."""
        li = self._layer
        self._layer += 1
        Hkv, D = self.k.shape[-2:]
        self.k[li][self._rows, self._cols] = k.reshape(-1, Hkv, D)
        self.v[li][self._rows, self._cols] = v.reshape(-1, Hkv, D)
        return li

    def attend(self, li: int, q: torch.Tensor, n_heads: int, scale: float | None = None, window: int = 0,
               sinks: torch.Tensor | None = None, softcap: float = 0.0) -> torch.Tensor:
        """One query per sequence ``[B, heads * head_dim]`` against keys ``0 .. lengths[b]`` (the token just written
        included); ``window`` limits it to the last ``window`` of them and ``sinks [heads]`` adds one value-less logit
        per head to the softmax - both run as tensor operations."""
        B = q.shape[0]
        Hkv, D = self.k.shape[-2:]
        G = n_heads // Hkv
        if q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128) and G <= 16 and not window and sinks is None and not softcap:
            # the decode kernel streams the cache once and reads the lengths on the device (no host synchronisation)
            from halo_b200.ops import _lib

            qc = q.contiguous()
            out = torch.empty_like(qc)
            rc = _lib.lib().halo_decode_attention(
                _lib.ptr(qc), _lib.ptr(self.k[li]), _lib.ptr(self.v[li]), _lib.ptr(self._cols), _lib.ptr(out), _lib.c_int(B),
                _lib.c_int(n_heads), _lib.c_int(Hkv), _lib.c_int(D), _lib.c_ll(self.k.shape[2]),
                _lib.c_float(scale if scale is not None else D ** -0.5), _lib.stream_ptr(q.device))
            _lib.check(rc, "halo_decode_attention")
            return out
        upto = int(self._cols.max().item()) + 1
        k, v = self.k[li, :, :upto], self.v[li, :, :upto]                 # [B, S, Hkv, D]
        qh = q.reshape(B, Hkv, G, D).float()
        scores = torch.einsum("bhgd,bshd->bhgs", qh, k.float()) * (scale if scale is not None else D ** -0.5)
        if softcap:
            scores = softcap * torch.tanh(scores / softcap)
        visible = torch.arange(upto, device=q.device)[None, :] <= self._cols[:, None]        # [B, S]
        if window:
            visible = visible & (torch.arange(upto, device=q.device)[None, :] > self._cols[:, None] - window)
        scores = scores.masked_fill(~visible[:, None, None, :], float("-inf"))
        if sinks is not None:
            sink = sinks.float().reshape(1, Hkv, G, 1).expand(B, -1, -1, -1)
            probs = torch.softmax(torch.cat([scores, sink], dim=-1), dim=-1)[..., :-1]
        else:
            probs = torch.softmax(scores, dim=-1)
        out = torch.einsum("bhgs,bshd->bhgd", probs, v.float())
        return out.reshape(B, n_heads * D).to(q.dtype)


def cached_attention(attn, h, ctx):
    """The attention block's forward while a :class:`KVCache` is attached to the context (called by
    :class:`halo_b200.models.qwen3.Attention`)."""
    from halo_b200.ops import attention as attn_ops
    from halo_b200.ops.rope import qk_norm_rope

    cfg, cache = attn.cfg, ctx.kv_cache
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    qkv = attn._qkv(h)
    q, k = qk_norm_rope(qkv, attn.q_norm, attn.k_norm, attn.rope_of(ctx), Hq, Hkv, cfg.rms_norm_eps, cfg.use_qk_norm)
    v = qkv[:, (Hq + Hkv) * D:]
    li = cache.write(k, v)
    special = attn.window or attn.sinks is not None or attn.scale is not None or attn.softcap
    if special and cache.mode == "prefill":
        o = attn.masked_core(q, k, v, ctx)
    elif special:
        o = cache.attend(li, q, Hq, scale=attn.scale, window=attn.window, sinks=attn.sinks, softcap=attn.softcap)
    elif cache.mode == "prefill":
        if q.is_cuda and D != 128:
            o = attn_ops.attention_reference(q, k, v, ctx.plan.cu_seqlens, Hq, Hkv)
        else:
            o = attn_ops.flash_attention(q, k, v, ctx.plan, Hq, Hkv)
    else:
        o = cache.attend(li, q, Hq)
    return attn._out(o)


def _sample(logits: torch.Tensor, params: SamplingParams, generator) -> tuple[torch.Tensor, torch.Tensor]:
    """``logits [B, V]`` fp32 -> (token ``[B]``, its log-probability under softmax(logits))."""
    logp = torch.log_softmax(logits, dim=-1)
    if params.temperature <= 0.0:
        tok = logits.argmax(-1)
        return tok, logp.gather(-1, tok[:, None]).squeeze(-1)
    scaled = logits / params.temperature
    if params.top_k and params.top_k < scaled.shape[-1]:
        kth = scaled.topk(params.top_k, dim=-1).values[:, -1:]
        scaled = scaled.masked_fill(scaled < kth, float("-inf"))
    if params.top_p < 1.0:
        sorted_logits, order = scaled.sort(dim=-1, descending=True)
        probs = torch.softmax(sorted_logits, dim=-1)
        before = probs.cumsum(-1) - probs                      # mass strictly ahead of each token
        drop = before >= params.top_p                          # the first token past the nucleus is kept
        sorted_logits = sorted_logits.masked_fill(drop, float("-inf"))
        scaled = torch.full_like(scaled, float("-inf")).scatter(-1, order, sorted_logits)
    tok = torch.multinomial(torch.softmax(scaled, dim=-1), 1, generator=generator).squeeze(-1)
    return tok, logp.gather(-1, tok[:, None]).squeeze(-1)


class Generator:
    """Batched sampling from a model built by :func:`halo_b200.models.qwen3.build_model` (single rank: the model's
    expert transport must be local)."""

    def __init__(self, model, eos_token_id: int | None = None, pad_token_id: int = 0):
        if getattr(model.transport, "n_ranks", 1) != 1 or model.tensor_parallel is not None or model.context_parallel is not None:
            raise ValueError("generation runs on an unsharded copy of the model (one rank holds every expert)")
        if model.cfg.hc_mult > 1:
            raise ValueError("generation is built for the plain residual decoder")
        self.model, self.eos, self.pad = model, eos_token_id, pad_token_id

    def _logits(self, trunk_rows: torch.Tensor) -> torch.Tensor:
        m = self.model
        h = rms_norm(trunk_rows, m.norm, m.cfg.rms_norm_eps)
        if m.cfg.final_logit_softcapping:
            return m.capped_logits(h)
        w = m.head_weight()
        return gemm.matmul(h, w, out_dtype=torch.float32) if h.is_cuda else h.float() @ w.float().t()

    @torch.no_grad()
    def generate(self, prompts: list, params: SamplingParams | None = None, record_routing: bool = False) -> list[Generation]:
        """``record_routing``: also return, per sequence, the experts every processed token was routed to
        (``extra["routing"]``: int16 ``[moe layers, prompt + generated - 1, top_k]``, ``extra["routing_layers"]``: their
        layer indices) so that training can replay the sampler's routing."""
        from halo_b200.models.qwen3 import ForwardContext

        params = params or SamplingParams()
        m, cfg = self.model, self.model.cfg
        dev = next(m.parameters()).device
        prompts = [np.asarray(p, dtype=np.int64).reshape(-1) for p in prompts]
        if not prompts or any(len(p) == 0 for p in prompts):
            raise ValueError("every prompt needs at least one token")
        B = len(prompts)
        lens = np.array([len(p) for p in prompts])
        stops = set(params.stop_token_ids) | ({self.eos} if self.eos is not None else set())
        # latent attention caches the expanded keys (one per query head, no-rotary + rotary dims) and zero-padded values
        kv_heads, width = ((cfg.num_attention_heads, cfg.qk_nope_head_dim + cfg.qk_rope_head_dim) if cfg.kv_lora_rank
                           else (cfg.num_key_value_heads, cfg.head_dim))
        cache = KVCache(len(m.layers), B, int(lens.max()) + params.max_new_tokens, kv_heads, width, next(m.parameters()).dtype, dev)
        generator = None
        if params.seed is not None:
            generator = torch.Generator(device=dev).manual_seed(params.seed)
        # ---- prefill: one packed row through the training kernels ------------------------------------------------
        ids = torch.from_numpy(np.concatenate(prompts)).to(dev)
        pos = torch.from_numpy(np.concatenate([np.arange(n) for n in lens])).to(dev)
        seq = torch.from_numpy(np.repeat(np.arange(B), lens)).to(dev)
        cu = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)).to(dev)
        trace: dict | None = {} if record_routing else None
        ctx = m.make_context(pos, cu)
        ctx.kv_cache = cache
        ctx.routing_trace = trace
        cache.begin_prefill(seq, pos, torch.from_numpy(lens).to(dev))
        trunk = m.trunk_states(ids, ctx)
        cache.end_prefill()
        logits = self._logits(trunk[(cu[1:] - 1).long()])
        # ---- decode --------------------------------------------------------------------------------------------
        tokens = torch.full((B, params.max_new_tokens), self.pad, dtype=torch.long, device=dev)
        logps = torch.zeros((B, params.max_new_tokens), dtype=torch.float32, device=dev)
        n_generated = torch.zeros(B, dtype=torch.long, device=dev)
        done = torch.zeros(B, dtype=torch.bool, device=dev)
        stopped = torch.zeros(B, dtype=torch.bool, device=dev)
        stop_t = torch.tensor(sorted(stops), dtype=torch.long, device=dev) if stops else None
        for step in range(params.max_new_tokens):
            tok, lp = _sample(logits, params, generator)
            tok = torch.where(done, torch.full_like(tok, self.pad), tok)
            tokens[:, step] = tok
            logps[:, step] = torch.where(done, torch.zeros_like(lp), lp)
            n_generated += (~done).long()
            if stop_t is not None:
                hit = torch.isin(tok, stop_t) & ~done
                stopped |= hit
                done |= hit
            if bool(done.all()) or step + 1 == params.max_new_tokens:
                break
            cache.begin_decode()
            dctx = ForwardContext(None, m.rope(cache.lengths), m.transport)
            dctx.rope_local = m.rope_local(cache.lengths)
            dctx.query_scale = m.query_scale(cache.lengths)
            dctx.positions = cache.lengths
            dctx.kv_cache = cache
            dctx.routing_trace = trace
            trunk = m.trunk_states(tok, dctx)
            cache.end_decode()
            logits = self._logits(trunk)
        n_cpu, tok_cpu, lp_cpu, stop_cpu = n_generated.cpu().numpy(), tokens.cpu().numpy(), logps.cpu().numpy(), stopped.cpu().numpy()
        outs = [Generation(prompts[b], tok_cpu[b, :n_cpu[b]].copy(), lp_cpu[b, :n_cpu[b]].copy(), "stop" if stop_cpu[b] else "length")
                for b in range(B)]
        if trace:
            layers = sorted(trace)
            # per layer: the prefill's [T, k] rows (packed by sequence), then one [B, k] row per decode step
            prefill = np.stack([trace[li][0].cpu().numpy() for li in layers])                       # [L, T, k]
            decode = np.stack([np.stack([t.cpu().numpy() for t in trace[li][1:]]) if len(trace[li]) > 1
                               else np.zeros((0, B, prefill.shape[-1]), dtype=prefill.dtype) for li in layers])   # [L, steps, B, k]
            offsets = np.concatenate([[0], np.cumsum(lens)])
            for b, g in enumerate(outs):
                fed = max(int(n_cpu[b]) - 1, 0)                      # generated tokens that were fed back (all but the last)
                rows = np.concatenate([prefill[:, offsets[b]:offsets[b + 1]], decode[:, :fed, b]], axis=1)
                g.extra["routing"], g.extra["routing_layers"] = rows.astype(np.int16), layers
        return outs
