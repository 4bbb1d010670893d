"""Gated delta-rule linear attention (the ``linear_attention`` layers of Qwen3-Next): a per-head matrix state that
decays, forgets what it held under the incoming key and writes the new value there,

    S_t = g_t S_{t-1} + k_t (beta_t (v_t - (g_t S_{t-1})^T k_t))^T,        o_t = S_t^T q_t,

behind a short causal convolution (with SiLU) over the concatenated q / k / v channels, and in front of an RMSNorm that is
gated by a fourth projection ``z``. ``g_t = exp(-exp(A_log) * softplus(a_t + time_step))`` and ``beta_t = sigmoid(b_t)``
come from a second small projection. Queries and keys are L2-normalised per head; a key head serves
``value_heads / key_heads`` value heads.

Training runs the recurrence chunk by chunk (chunks of ``CHUNK`` tokens that never straddle a document). With the
cumulative log-decay ``c_i`` inside a chunk and the state ``S_0`` at its start,

    (I + A) U = beta V - beta e^c K S_0,      A_ij = beta_i e^{c_i - c_j} (k_i . k_j)   for j < i,

so everything that does not depend on ``S_0`` (the triangular solve against ``beta V`` and ``beta e^c K``, the masked
``q k^T`` block) is computed for ALL chunks of the row at once, and the sequential part is four small products per
chunk. Documents advance side by side: step ``r`` handles the ``r``-th chunk of every document that has one, so the loop
is as long as the longest document, not as the row. All of it is tensor operations under autograd, in fp32.

While sampling, the cache holds each sequence's last ``kernel - 1`` convolution inputs and its matrix state: prefill
leaves every prompt's final state there, a decode step is one application of the recurrence.

Whole rows only (a cut row would cut both the convolution and the recurrence).
(The role of the reference's Qwen3-Next / Qwen3.5 linear-attention families, halo/models/families and
halo/models/segment_markers.py.)"""

from __future__ import annotations

import torch
from torch import nn

from halo_b200.ops import gemm

from .short_conv import segment_causal_conv

CHUNK = 64


def _chunk_layout(lengths: list[int], chunk: int, device):
    """Chunks that never straddle a document. Returns ``src [N, C]`` (token index of every slot, ``T`` for padding),
    ``slot_of_token [T]`` (flat slot index), and per step ``r`` the pair ``(documents active, their chunk ids)``."""
    src, steps, start, n_chunks = [], [], 0, 0
    T = sum(lengths)
    for d, n in enumerate(lengths):
        for r in range((n + chunk - 1) // chunk):
            lo = start + r * chunk
            hi = min(lo + chunk, start + n)
            src.append(list(range(lo, hi)) + [T] * (chunk - (hi - lo)))
            while len(steps) <= r:
                steps.append(([], []))
            steps[r][0].append(d)
            steps[r][1].append(n_chunks)
            n_chunks += 1
        start += n
    src_t = torch.tensor(src, dtype=torch.long, device=device)
    flat = src_t.reshape(-1)
    slot_of_token = torch.empty(T + 1, dtype=torch.long, device=device)
    slot_of_token[flat] = torch.arange(flat.numel(), device=device)
    steps_t = [(torch.tensor(a, dtype=torch.long, device=device), torch.tensor(b, dtype=torch.long, device=device)) for a, b in steps]
    return src_t, slot_of_token[:T], steps_t


def chunked_gated_delta_rule(q, k, v, log_g, beta, lengths: list[int], chunk: int = CHUNK):
    """``q, k [T, H, dk]`` (normalised, ``q`` scaled), ``v [T, H, dv]``, ``log_g, beta [T, H]``; documents of ``lengths``
    tokens back to back. Returns ``(o [T, H, dv], final state per document [n_docs, H, dk, dv])``, fp32."""
    T, H, dk = k.shape
    dv = v.shape[-1]
    dev = q.device
    src, slot_of_token, steps = _chunk_layout(lengths, chunk, dev)
    N, C = src.shape

    def chunks(x):          # [T, H, ...] -> [N, H, C, ...] with a neutral row (zeros) in the padded slots
        padded = torch.cat([x.float(), torch.zeros_like(x[:1], dtype=torch.float32)], dim=0)
        return padded[src].transpose(1, 2)

    qc, kc, vc = chunks(q), chunks(k), chunks(v)                        # [N, H, C, d]
    bc, lg = chunks(beta), chunks(log_g)                                # [N, H, C]
    c = lg.cumsum(dim=-1)
    lower = torch.ones(C, C, dtype=torch.bool, device=dev).tril()       # j <= i
    diff = (c[..., :, None] - c[..., None, :]).masked_fill(~lower, float("-inf"))
    decay = diff.exp()                                                  # e^{c_i - c_j} for j <= i, else 0
    a = bc[..., :, None] * decay * (kc @ kc.transpose(-1, -2))
    a = a.masked_fill(torch.eye(C, dtype=torch.bool, device=dev), 0.0)  # strictly lower
    rhs = torch.cat([bc[..., None] * vc, (bc * c.exp())[..., None] * kc], dim=-1)
    x = torch.linalg.solve_triangular(a + torch.eye(C, device=dev), rhs, upper=False, unitriangular=True)
    u_free, w = x[..., :dv], x[..., dv:]                                # U = u_free - w S_0
    m = decay * (qc @ kc.transpose(-1, -2))                             # e^{c_i - c_j} (q_i . k_j), j <= i
    q_dec = qc * c.exp()[..., None]
    total = c[..., -1]                                                  # log-decay over the whole chunk
    k_dec = kc * (total[..., None] - c).exp()[..., None]

    state = torch.zeros(len(lengths), H, dk, dv, dtype=torch.float32, device=dev)
    outs = torch.zeros(N, H, C, dv, dtype=torch.float32, device=dev)
    for docs, ids in steps:
        s0 = state[docs]
        u = u_free[ids] - w[ids] @ s0
        outs = outs.index_copy(0, ids, q_dec[ids] @ s0 + m[ids] @ u)
        state = state.index_copy(0, docs, total[ids].exp()[..., None, None] * s0 + k_dec[ids].transpose(-1, -2) @ u)
    o = outs.transpose(1, 2).reshape(N * C, H, dv)[slot_of_token]
    return o, state


def recurrent_gated_delta_step(state, q, k, v, log_g, beta):
    """One token per sequence: ``state [B, H, dk, dv]`` (fp32), ``q, k [B, H, dk]``, ``v [B, H, dv]``, ``log_g, beta [B, H]``."""
    s = state * log_g.float().exp()[..., None, None]
    held = torch.einsum("bhkv,bhk->bhv", s, k.float())
    s = s + k.float()[..., :, None] * ((v.float() - held) * beta.float()[..., None])[..., None, :]
    return torch.einsum("bhkv,bhk->bhv", s, q.float()), s


def _l2norm(x):
    return x * torch.rsqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


class GatedDeltaNet(nn.Module):
    def __init__(self, cfg, dtype, device, tp_size: int = 1, layer_idx: int = 0):
        super().__init__()
        if tp_size > 1:
            raise ValueError("the gated delta-rule mixer is not cut over tensor-parallel ranks")
        self.cfg, self.layer_idx = cfg, layer_idx
        H = cfg.hidden_size
        self.Hk, self.Hv, self.dk, self.dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
        if self.Hv % self.Hk:
            raise ValueError("linear_num_value_heads must be a multiple of linear_num_key_heads")
        key_dim, value_dim = self.Hk * self.dk, self.Hv * self.dv

        def param(*shape):
            return nn.Parameter(torch.empty(*shape, dtype=dtype, device=device))

        # the hub's own row order. Qwen3-Next: two projections grouped per key head (its q, k, and its value heads' v and
        # z; b and a likewise). Qwen3.5: one projection per role, heads in flat order
        self.per_role = cfg.family == "qwen3_5_moe_text"
        if self.per_role:
            self.gdn_in_proj_qkv = param(2 * key_dim + value_dim, H)
            self.gdn_in_proj_z = param(value_dim, H)
            self.gdn_in_proj_b = param(self.Hv, H)
            self.gdn_in_proj_a = param(self.Hv, H)
        else:
            self.gdn_in_proj_qkvz = param(2 * key_dim + 2 * value_dim, H)
            self.gdn_in_proj_ba = param(2 * self.Hv, H)
        self.gdn_conv = param(2 * key_dim + value_dim, 1, cfg.linear_conv_kernel_dim)
        self.gdn_time_step = param(self.Hv)
        self.gdn_A_log = param(self.Hv)
        self.gdn_norm = param(self.dv)
        self.gdn_out_proj = param(H, value_dim)
        self.window, self.sinks, self.lora, self.lowp = 0, None, None, ""

    def forward(self, h, ctx):
        if ctx.cp is not None or ctx.tp is not None:
            raise NotImplementedError("the gated delta-rule mixer runs on unsliced rows")
        cfg, T = self.cfg, h.shape[0]
        Hk, Hv, dk, dv = self.Hk, self.Hv, self.dk, self.dv
        r = Hv // Hk
        if self.per_role:
            mixed = gemm.linear(h, self.gdn_in_proj_qkv)
            z = gemm.linear(h, self.gdn_in_proj_z)
            b, a = gemm.linear(h, self.gdn_in_proj_b), gemm.linear(h, self.gdn_in_proj_a)
        else:
            qkvz = gemm.linear(h, self.gdn_in_proj_qkvz).reshape(T, Hk, 2 * dk + 2 * r * dv)
            q, k, v, z = qkvz.split([dk, dk, r * dv, r * dv], dim=-1)
            ba = gemm.linear(h, self.gdn_in_proj_ba).reshape(T, Hk, 2 * r)
            b, a = ba[..., :r].reshape(T, Hv), ba[..., r:].reshape(T, Hv)
            mixed = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=-1)
        K = cfg.linear_conv_kernel_dim
        taps = self.gdn_conv[:, 0, :]
        cache = ctx.kv_cache
        decode = cache is not None and cache.mode != "prefill"
        if decode:
            recent = cache.conv_state(self.layer_idx, K - 1, mixed)
            window = torch.cat([recent, mixed[:, None, :]], dim=1)
            conv = (window * taps.to(mixed.dtype).t()[None]).sum(dim=1)
            recent.copy_(window[:, 1:])
        else:
            conv = segment_causal_conv(mixed, taps, ctx.positions)
            if cache is not None:
                cache.store_conv_tail(self.layer_idx, K - 1, mixed)
        conv = torch.nn.functional.silu(conv)
        q, k, v = conv.split([Hk * dk, Hk * dk, Hv * dv], dim=-1)
        q = _l2norm(q.reshape(T, Hk, dk).float()).repeat_interleave(r, dim=1) * dk ** -0.5
        k = _l2norm(k.reshape(T, Hk, dk).float()).repeat_interleave(r, dim=1)
        v = v.reshape(T, Hv, dv)
        beta = torch.sigmoid(b)
        log_g = -self.gdn_A_log.float().exp() * torch.nn.functional.softplus(a.float() + self.gdn_time_step.float())
        if decode:
            o, new_state = recurrent_gated_delta_step(cache.recurrent_state(self.layer_idx, Hv, dk, dv), q, k, v, log_g, beta)
            cache.recurrent[self.layer_idx] = new_state
        else:
            if getattr(ctx, "doc_lengths", None) is None:
                cu = ctx.plan.cu_seqlens
                ctx.doc_lengths = [int(n) for n in (cu[1:] - cu[:-1]).tolist()]      # once per batch, shared by the layers
            o, final = chunked_gated_delta_rule(q, k, v, log_g, beta, ctx.doc_lengths)
            if cache is not None:
                cache.recurrent[self.layer_idx] = final.detach()
        o = o.to(h.dtype)
        # RMSNorm per value head, then the SiLU gate of the fourth projection
        of = o.float()
        normed = (of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps)).to(h.dtype)
        gated = (self.gdn_norm * normed).float() * torch.nn.functional.silu(z.reshape(T, Hv, dv).float())
        return gemm.linear(gated.to(h.dtype).reshape(T, Hv * dv), self.gdn_out_proj)
