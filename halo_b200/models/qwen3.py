"""Pre-norm decoder (Qwen3 / Qwen3-MoE, and the Qwen2, Llama, Mistral and Mixtral variants of it that the
configuration's family switches select) over packed rows, with every hot op on the sm_100a kernels.

The model consumes one flattened token stream ``[T]`` per rank (documents delimited by
``cu_seqlens``), as the packing collator produces it. Parameter names follow the Hugging Face
modules so checkpoints convert by renaming only; the three projections of attention are stored
fused (``qkv_proj``), as are ``gate`` / ``up`` (``gate_up_proj``), and routed experts are stacked
``[E_local, 2F, H]`` / ``[E_local, H, F]`` exactly like the Hugging Face runtime layout.

Per layer:  x -> RMSNorm -> qkv GEMM -> q/k-norm + RoPE + flash attention -> o GEMM -> +residual
            -> RMSNorm -> (router GEMM -> top-k -> dispatch -> grouped SwiGLU FFN -> combine |
            dense SwiGLU FFN) -> +residual.
The output head is fused with the loss (no logits plane).

Behavioural counterpart of the reference's patched Hugging Face models
(halo/distributed/expert_parallel/moe_layer/layer.py:67-80, 301-342;
halo/distributed/expert_parallel/moe_layer/routing.py:105-150).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from halo_b200.ops import attention as attn_ops
from halo_b200.ops import gemm
from halo_b200.ops import moe as moe_ops
from halo_b200.ops import _lib
from halo_b200.ops.cross_entropy import fused_linear_cross_entropy, linear_logprobs
from halo_b200.ops.norm import add_rms_norm, rms_norm
from halo_b200.ops.rope import rope_table

from .config import ModelConfig
from .recompute import recompute, recompute_second_half


def _rounded(t, fmt: str):
    """``t`` rounded to the block-scaled format ``fmt`` along its last axis (straight-through gradient); itself
    when no format is set."""
    if not fmt:
        return t
    from halo_b200.ops.lowp import fake_quant

    return fake_quant(t, fmt)


def _linear(x, weight, fmt: str = ""):
    return gemm.linear(_rounded(x, fmt), _rounded(weight, fmt))


class _SwiGLULinear(torch.autograd.Function):
    """act = silu(x Wg^T) * (x Wu^T) with the activation in the GEMM epilogue; recompute-free backward."""

    @staticmethod
    def forward(ctx, x, w_gate_up, grad_mode=True):
        act, pre = gemm.swiglu_matmul(x, w_gate_up, save_pre=grad_mode and any(ctx.needs_input_grad))
        ctx.save_for_backward(x, w_gate_up, pre)
        return act

    @staticmethod
    def backward(ctx, dact):
        x, w, pre = ctx.saved_tensors
        F = w.shape[0] // 2
        dact = dact.contiguous()
        if x.is_cuda:
            dpre = torch.empty_like(pre)
            rc = _lib.lib().halo_swiglu_bwd(_lib.ptr(pre), _lib.ptr(dact), _lib.ptr(dpre), _lib.c_ll(pre.shape[0]),
                                            _lib.c_int(F), _lib.stream_ptr(x.device))
            _lib.check(rc, "halo_swiglu_bwd")
        else:
            g, u = pre[:, :F].float(), pre[:, F:].float()
            s = torch.sigmoid(g)
            d = dact.float()
            dpre = torch.cat([d * u * s * (1 + g * (1 - s)), d * g * s], dim=-1).to(pre.dtype)
        dx = gemm.matmul(dpre, w, b_t=False) if ctx.needs_input_grad[0] else None
        dw = gemm.matmul(dpre, x, a_t=True, b_t=False) if ctx.needs_input_grad[1] else None
        return dx, dw, None


class _RouterLinear(torch.autograd.Function):
    """fp32 router logits from bf16 operands (fp32 accumulate, fp32 result)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return gemm.matmul(x, w, out_dtype=torch.float32)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        gb = g.to(x.dtype)
        # pad the expert dimension of the gradient to a multiple of 8 rows only when needed
        dx = gemm.matmul(gb, w, b_t=False) if ctx.needs_input_grad[0] else None
        dw = gemm.matmul(gb, x, a_t=True, b_t=False) if ctx.needs_input_grad[1] else None
        return dx, dw


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, tp_size: int = 1, layer_idx: int = 0):
        super().__init__()
        self.cfg = cfg
        # the window of this layer: families that alternate windowed and full layers name each layer's kind
        kinds = cfg.layer_types
        self.window = cfg.sliding_window if (not kinds or layer_idx >= len(kinds) or kinds[layer_idx] == "sliding_attention") else 0
        if (cfg.attention_sinks or cfg.output_bias or self.window or cfg.attn_logit_softcapping
                or (cfg.query_pre_attn_scalar or cfg.head_dim) != cfg.head_dim) and tp_size > 1:
            raise ValueError("attention sinks, an output-projection bias, a sliding window and a configured softmax scale are not "
                             "cut over tensor-parallel ranks")
        H, D = cfg.hidden_size, cfg.head_dim
        # under tensor parallelism a rank holds 1/tp of the query and of the key/value heads
        self.n_heads, self.n_kv_heads = cfg.num_attention_heads // tp_size, cfg.num_key_value_heads // tp_size
        self.qkv_proj = nn.Parameter(torch.empty((self.n_heads + 2 * self.n_kv_heads) * D, H, dtype=dtype, device=device))
        self.o_proj = nn.Parameter(torch.empty(H, self.n_heads * D, dtype=dtype, device=device))
        if tp_size > 1:
            self.qkv_proj.tp_kind, self.o_proj.tp_kind = "qkv", "o"
        # Qwen2 puts a bias on q / k / v (not on o); under tensor parallelism it is cut like the rows it belongs to
        if cfg.attention_bias:
            self.qkv_bias = nn.Parameter(torch.zeros((self.n_heads + 2 * self.n_kv_heads) * D, dtype=dtype, device=device))
            if tp_size > 1:
                self.qkv_bias.tp_kind = "qkv_bias"
        else:
            self.register_parameter("qkv_bias", None)
        # a configured softmax scale (Gemma's query_pre_attn_scalar); None = head_dim ** -0.5, which the flash kernel uses
        qpas = cfg.query_pre_attn_scalar
        self.scale = float(qpas) ** -0.5 if qpas and qpas != D else None
        self.softcap = float(cfg.attn_logit_softcapping or 0.0)
        self.o_bias = nn.Parameter(torch.zeros(H, dtype=dtype, device=device)) if cfg.output_bias else None
        self.sinks = nn.Parameter(torch.zeros(self.n_heads, dtype=dtype, device=device)) if cfg.attention_sinks else None
        self.lora = None          # halo_b200.peft.lora.LoraSet when low-rank adapters are attached
        self.lowp = ""            # block-scaled format the projections are rounded to (quantisation-aware training)
        if cfg.use_qk_norm:
            if cfg.qk_norm_whole_width and tp_size > 1:
                raise ValueError("a q / k norm over all heads cannot be cut over tensor-parallel ranks")
            wq, wk = (self.n_heads * D, self.n_kv_heads * D) if cfg.qk_norm_whole_width else (D, D)
            self.q_norm = nn.Parameter(torch.ones(wq, dtype=dtype, device=device))
            self.k_norm = nn.Parameter(torch.ones(wk, dtype=dtype, device=device))
        else:
            self.register_parameter("q_norm", None)
            self.register_parameter("k_norm", None)

    def rope_of(self, ctx):
        """The rotary table of this layer: windowed layers of a family with a local rotary base have their own."""
        local = getattr(ctx, "rope_local", None)
        return local if (self.window and local is not None) else ctx.rope

    def _biased(self, qkv):
        return qkv if self.qkv_bias is None else qkv + self.qkv_bias

    def _masked(self, qkv, ctx):
        """Attention under an explicit ``[T, T]`` mask through the masked-attention op: the context's own mask (tree
        packing: completions that share a stored-once prompt), the sliding window of this layer, or plain causal
        attention with sink logits. The flash kernel serves none of them; meant for rows of a few thousand tokens."""
        from halo_b200.ops.rope import qk_norm_rope

        cfg = self.cfg
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        q, k = qk_norm_rope(qkv, self.q_norm, self.k_norm, self.rope_of(ctx), Hq, Hkv, cfg.rms_norm_eps, cfg.use_qk_norm)
        v = qkv[:, (Hq + Hkv) * D:]
        return self.masked_core(q, k, v, ctx)

    def masked_core(self, q, k, v, ctx):
        """``q [T, Hq*D]``, ``k`` / ``v [T, Hkv*D]`` (normed and rotated) under this layer's mask."""
        from halo_b200.ops.masked_attention import masked_attention, window_mask

        cfg = self.cfg
        if ctx.cp is not None or ctx.tp is not None:
            raise NotImplementedError("windowed / sink / explicitly masked attention is built for unsliced rows")
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        mask = getattr(ctx, "attention_mask", None)
        T = q.shape[0]
        if self.window:
            if getattr(ctx, "window", None) is None:
                ctx.window = window_mask(ctx.plan.cu_seqlens, self.window, device=q.device)     # shared by the layers
                if mask is not None:
                    ctx.window = ctx.window & mask.to(q.device)
            mask = ctx.window
        elif mask is None:
            # a full layer that is here for its sinks: the causal mask of the packed documents, shared by such layers
            if getattr(ctx, "causal", None) is None:
                ctx.causal = window_mask(ctx.plan.cu_seqlens, T, device=q.device)
            mask = ctx.causal
        elif mask.device != q.device:
            mask = ctx.attention_mask = mask.to(q.device)
        o = masked_attention(q.reshape(T, Hq, D), k.reshape(T, Hkv, D), v.reshape(T, Hkv, D), mask, scale=self.scale, sinks=self.sinks,
                             softcap=self.softcap)
        return o.reshape(T, Hq * D)

    def _qkv(self, h):
        qkv = self._biased(_linear(h, self.qkv_proj, self.lowp))
        if self.lora is not None:
            q, kv = self.n_heads * self.cfg.head_dim, self.n_kv_heads * self.cfg.head_dim
            qkv = self.lora.add_fused(h, qkv, [("q_proj", 0, q), ("k_proj", q, q + kv), ("v_proj", q + kv, q + 2 * kv)])
        return qkv

    def _out(self, o):
        y = _linear(o, self.o_proj, self.lowp)
        if self.lora is not None and "o_proj" in self.lora:
            y = y + self.lora.delta("o_proj", o)
        return y if self.o_bias is None else y + self.o_bias

    def forward(self, h, ctx):
        cfg = self.cfg
        if ctx.kv_cache is not None:
            # generation: keys / values go to the cache, a decode step attends the cache
            from halo_b200.inference.generate import cached_attention

            return cached_attention(self, h, ctx)
        if ctx.tp is not None:
            # token shards -> whole row, a slice of the heads, partial output summed back into token shards
            from halo_b200.parallel.tensor_parallel import gather_seq, row_parallel_linear

            qkv = self._biased(gemm.linear(gather_seq(h, ctx.tp), self.qkv_proj))
            o = attn_ops.rope_attention(qkv, self.q_norm, self.k_norm, ctx.rope, ctx.plan, self.n_heads, self.n_kv_heads,
                                        cfg.rms_norm_eps, cfg.use_qk_norm)
            return row_parallel_linear(o, self.o_proj, ctx.tp)
        qkv = self._qkv(h)
        if ((self.window or self.sinks is not None or self.scale is not None) and not self.softcap and qkv.is_cuda
                and qkv.dtype == torch.bfloat16 and ctx.cp is None and getattr(ctx, "attention_mask", None) is None
                and (cfg.head_dim == attn_ops.HEAD_DIM or cfg.head_dim in attn_ops.PADDED_HEAD_DIMS)):
            # windows, sinks and a configured softmax scale on the flash kernels: work lists cut to the window and its left
            # edge masked in the kernels, the sink logit added to the denominator in the forward's last step, the scale a
            # kernel argument
            plan = ctx.window_plan(self.window) if self.window else ctx.plan
            o = attn_ops.rope_attention(qkv, self.q_norm, self.k_norm, self.rope_of(ctx), plan, cfg.num_attention_heads,
                                        cfg.num_key_value_heads, cfg.rms_norm_eps, cfg.use_qk_norm, scale=self.scale,
                                        sinks=self.sinks)
            return self._out(o)
        if (self.window or self.sinks is not None or self.scale is not None or self.softcap
                or getattr(ctx, "attention_mask", None) is not None):
            return self._out(self._masked(qkv, ctx))
        if ctx.cp is not None:
            # context parallel: this rank holds one chunk of the row; keys and values of straddling documents
            # come from the lower ranks
            from halo_b200.ops.rope import qk_norm_rope
            from halo_b200.parallel.context_parallel import cp_attention

            cp, layout = ctx.cp
            q, k = qk_norm_rope(qkv, self.q_norm, self.k_norm, ctx.rope, cfg.num_attention_heads,
                                cfg.num_key_value_heads, cfg.rms_norm_eps, cfg.use_qk_norm)
            v = qkv[:, (cfg.num_attention_heads + cfg.num_key_value_heads) * cfg.head_dim:]
            o = cp_attention(q, k, v, layout, ctx.plan, cp.group, cp.exchange, cfg.num_attention_heads,
                             cfg.num_key_value_heads)
        else:
            o = attn_ops.rope_attention(qkv, self.q_norm, self.k_norm, ctx.rope, ctx.plan, cfg.num_attention_heads,
                                        cfg.num_key_value_heads, cfg.rms_norm_eps, cfg.use_qk_norm)
        return self._out(o)


class GatedAttention(Attention):
    """Attention whose output is multiplied by ``sigmoid(gate)`` before the output projection (Qwen3-Next). The gate comes
    out of the query projection: its rows are, per head, the head's query rows then its gate rows - the hub's own order,
    kept at run time so that the checkpoint's ``q_proj`` loads as one block in front of ``k_proj`` and ``v_proj``.
    Unsliced rows and heads only; low-rank adapters on ``q_proj`` are refused by the adapter code."""

    def __init__(self, cfg: ModelConfig, dtype, device, tp_size: int = 1, layer_idx: int = 0):
        if tp_size > 1 or cfg.attention_bias:
            raise ValueError("gated attention is built without a q / k / v bias and is not cut over tensor-parallel ranks")
        super().__init__(cfg, dtype, device, tp_size, layer_idx)
        H, D = cfg.hidden_size, cfg.head_dim
        self.qkv_proj = nn.Parameter(torch.empty((2 * self.n_heads + 2 * self.n_kv_heads) * D, H, dtype=dtype, device=device))
        self._gate = None

    def _qkv(self, h):
        D, Hq = self.cfg.head_dim, self.n_heads
        wide = self._biased(_linear(h, self.qkv_proj, self.lowp))
        qg = wide[:, :2 * Hq * D].reshape(-1, Hq, 2 * D)
        self._gate = qg[..., D:].reshape(-1, Hq * D)
        qkv = torch.cat([qg[..., :D].reshape(-1, Hq * D), wide[:, 2 * Hq * D:]], dim=-1)
        if self.lora is not None:
            q, kv = Hq * D, self.n_kv_heads * D
            # the query block carries no adapter here (its projection also makes the gate): its range passes through
            qkv = self.lora.add_fused(h, qkv, [("q_proj", 0, q), ("k_proj", q, q + kv), ("v_proj", q + kv, q + 2 * kv)])
        return qkv

    def _out(self, o):
        gate, self._gate = self._gate, None
        return super()._out(o * torch.sigmoid(gate.float()).to(o.dtype))


class DenseMLP(nn.Module):
    def __init__(self, hidden: int, width: int, dtype, device, tp_size: int = 1):
        super().__init__()
        width //= tp_size
        self.tp_size = tp_size
        self.gate_up_proj = nn.Parameter(torch.empty(2 * width, hidden, dtype=dtype, device=device))
        self.down_proj = nn.Parameter(torch.empty(hidden, width, dtype=dtype, device=device))
        if tp_size > 1:
            self.gate_up_proj.tp_kind, self.down_proj.tp_kind = "gate_up", "down"
        self.lora = None          # halo_b200.peft.lora.LoraSet when low-rank adapters are attached
        self.lowp = ""            # block-scaled format of quantisation-aware training
        self.activation = "silu"  # "gelu_tanh": Gemma's gate; runs as tensor ops between the two GEMMs

    def forward(self, h, ctx=None):
        if self.activation != "silu":
            if self.tp_size > 1 or self.lowp:
                raise NotImplementedError("the tanh-GELU gate is built for unsliced, full-precision feed-forward blocks")
            width = self.gate_up_proj.shape[0] // 2
            pre = gemm.linear(h, self.gate_up_proj)
            if self.lora is not None:
                pre = self.lora.add_fused(h, pre, [("gate_proj", 0, width), ("up_proj", width, 2 * width)])
            act = torch.nn.functional.gelu(pre[:, :width], approximate="tanh") * pre[:, width:]
            y = gemm.linear(act, self.down_proj)
            return y + self.lora.delta("down_proj", act) if self.lora is not None and "down_proj" in self.lora else y
        if self.lowp and self.lora is None and self.tp_size == 1:
            act = _SwiGLULinear.apply(_rounded(h, self.lowp), _rounded(self.gate_up_proj, self.lowp), torch.is_grad_enabled())
            return _linear(act, self.down_proj, self.lowp)
        if self.lora is not None:
            # the low-rank terms join the pre-activation, so the activation runs as its own kernel here
            from halo_b200.ops.activation import swiglu

            width = self.gate_up_proj.shape[0] // 2
            pre = self.lora.add_fused(h, gemm.linear(h, self.gate_up_proj), [("gate_proj", 0, width), ("up_proj", width, 2 * width)])
            act = swiglu(pre)
            y = gemm.linear(act, self.down_proj)
            return y + self.lora.delta("down_proj", act) if "down_proj" in self.lora else y
        if self.tp_size > 1:
            from halo_b200.parallel.tensor_parallel import gather_seq, row_parallel_linear

            act = _SwiGLULinear.apply(gather_seq(h, ctx.tp), self.gate_up_proj, torch.is_grad_enabled())
            return row_parallel_linear(act, self.down_proj, ctx.tp)
        return gemm.linear(_SwiGLULinear.apply(h, self.gate_up_proj, torch.is_grad_enabled()), self.down_proj)


class SparseMoE(nn.Module):
    """Router + routed experts (+ optional shared expert). Expert tensors hold only this rank's
    experts ``[E_local, ...]`` when expert parallelism is on."""

    def __init__(self, cfg: ModelConfig, dtype, device, n_local_experts: int, router_dtype=None, etp=None):
        super().__init__()
        self.cfg = cfg
        self.etp = etp            # ExpertTensorParallel: every expert's width is cut over its group
        H, F = cfg.hidden_size, cfg.moe_intermediate_size
        if etp is not None:
            etp.check(cfg)
            F //= etp.size
        self.gate = nn.Parameter(torch.empty(cfg.num_experts, H, dtype=router_dtype or dtype, device=device))
        self.experts_gate_up = nn.Parameter(torch.empty(n_local_experts, 2 * F, H, dtype=dtype, device=device))
        self.experts_down = nn.Parameter(torch.empty(n_local_experts, H, F, dtype=dtype, device=device))
        self.experts_gate_up.is_expert = True
        self.experts_down.is_expert = True
        if etp is not None:
            self.experts_gate_up.etp_kind, self.experts_down.etp_kind = "gate_up", "down"
        if cfg.shared_expert_intermediate_size:
            self.shared_expert = DenseMLP(H, cfg.shared_expert_intermediate_size, dtype, device)
            self.shared_gate = (nn.Parameter(torch.empty(1, H, dtype=dtype, device=device))
                                if cfg.shared_expert_gate else None)
        else:
            self.shared_expert = None
            self.shared_gate = None
        # auxiliary-loss-free balancing: a per-expert bias that only ranks experts (never a parameter,
        # saved as a sidecar by the balancing callback)
        self.register_buffer("selection_bias", None, persistent=False)
        # families that ship a selection bias with the checkpoint (it ranks experts, never weights them): stored, not trained
        if cfg.router_bias:
            self.e_score_correction_bias = nn.Parameter(torch.zeros(cfg.num_experts, dtype=torch.float32, device=device),
                                                        requires_grad=False)
        else:
            self.register_parameter("e_score_correction_bias", None)
        # gpt-oss: a trained bias on the router's logits, and per-expert bias vectors around a clamped GLU
        self.gate_bias = (nn.Parameter(torch.zeros(cfg.num_experts, dtype=router_dtype or dtype, device=device))
                          if cfg.router_logit_bias else None)
        if cfg.expert_bias or cfg.expert_activation != "swiglu":
            if etp is not None:
                raise ValueError("experts with bias vectors / a clamped GLU are not cut inside an expert (expert tensor "
                                 "parallelism); expert parallelism holds whole experts and is fine")
            self.experts_gate_up_bias = nn.Parameter(torch.zeros(n_local_experts, 2 * F, dtype=dtype, device=device))
            self.experts_down_bias = nn.Parameter(torch.zeros(n_local_experts, H, dtype=dtype, device=device))
            self.experts_gate_up_bias.is_expert = self.experts_down_bias.is_expert = True
        else:
            self.experts_gate_up_bias = self.experts_down_bias = None
        self.expert_lora = None       # halo_b200.peft.lora.ExpertLora when the routed experts carry adapters
        self.lowp = ""                # block-scaled format of quantisation-aware training (banks and dispatched rows)
        self.load_counter = None      # (ExpertLoadCounter, layer index) when load metrics are on
        self.last_routing = None
        self.layer_index = -1         # global index of the decoder layer this block belongs to (set by the layer)

    def forward(self, h, ctx):
        cfg = self.cfg
        gate_w = self.gate if self.gate.dtype == h.dtype else self.gate.to(h.dtype)
        logits = _RouterLinear.apply(h, gate_w) if h.is_cuda else (h.float() @ self.gate.float().t())
        if self.gate_bias is not None:
            logits = logits + self.gate_bias.float()
        bias = self.selection_bias
        if self.e_score_correction_bias is not None:
            bias = self.e_score_correction_bias if bias is None else self.e_score_correction_bias + bias
        forced, partial = None, False
        if isinstance(ctx.replay_topk, dict):
            partial = True
            # routing replay keyed by layer (safe under recomputation): the sampler's expert choice per token, -1 where
            # the sampler never routed the token - there this forward routes for itself
            forced = ctx.replay_topk.get(self.layer_index)
        elif ctx.replay_topk is not None:
            forced = ctx.replay_topk.pop(0)
        if forced is not None:
            idx = forced.to(logits.device)
            if partial:                   # merged on the device: no host read of "is anything missing"
                with torch.no_grad():
                    own, _ = (moe_ops.router_grouped_topk(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob, bias, cfg.n_group,
                                                          cfg.topk_group, cfg.routed_scaling_factor, cfg.score_function, cfg.norm_topk_eps)
                              if cfg.grouped_routing else
                              moe_ops.router_topk(logits.detach(), cfg.num_experts_per_tok, cfg.norm_topk_prob, bias))
                idx = torch.where(idx < 0, own.to(idx.dtype), idx)
            idx = idx.to(torch.int32)
            probs = torch.sigmoid(logits.float()) if cfg.score_function == "sigmoid" else torch.softmax(logits.float(), dim=-1)
            w = probs.gather(-1, idx.long())
            if cfg.norm_topk_prob:
                w = w / (w.sum(-1, keepdim=True) + (cfg.norm_topk_eps if cfg.grouped_routing else 0.0))
            w = w * cfg.routed_scaling_factor
        elif cfg.grouped_routing:
            idx, w = moe_ops.router_grouped_topk(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob, bias, cfg.n_group,
                                                 cfg.topk_group, cfg.routed_scaling_factor, cfg.score_function, cfg.norm_topk_eps)
        else:
            idx, w = moe_ops.router_topk(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob, self.selection_bias)
        if self.load_counter is not None and not getattr(ctx, "output_unused", False):
            counter, layer_index = self.load_counter
            counter.add(layer_index, idx)     # first pass only: a recomputation replays the same routing
        if ctx.record_routing is not None:
            ctx.record_routing.append((logits, idx))
        if getattr(ctx, "routing_trace", None) is not None:
            ctx.routing_trace.setdefault(self.layer_index, []).append(idx.detach())
        bank_gate_up, bank_down = self.experts_gate_up, self.experts_down
        if self.expert_lora is not None:
            bank_gate_up, bank_down = self.expert_lora.effective_banks(bank_gate_up, bank_down)
        h_experts = h
        if self.lowp:
            bank_gate_up, bank_down, h_experts = (_rounded(t, self.lowp) for t in (bank_gate_up, bank_down, h))
        if self.experts_gate_up_bias is not None:
            from halo_b200.ops.biased_glu_experts import GLU_ALPHA, biased_glu_experts

            if h_experts.is_cuda and h_experts.dtype == torch.bfloat16:
                # grouped products with the bias / clamped-GLU row kernels between them; dispatches over expert-parallel
                # ranks like the plain experts
                out = moe_ops.moe_experts(h_experts, idx, w, bank_gate_up, bank_down, ctx.transport,
                                          skip_output=getattr(ctx, "output_unused", False),
                                          glu=(self.experts_gate_up_bias, self.experts_down_bias, cfg.glu_limit, GLU_ALPHA))
            else:
                if bank_gate_up.shape[0] != cfg.num_experts:
                    raise NotImplementedError("experts with bias vectors / a clamped GLU dispatch over expert-parallel "
                                              "ranks on GPUs only")
                out = biased_glu_experts(h_experts, idx, w, bank_gate_up, self.experts_gate_up_bias, bank_down,
                                         self.experts_down_bias, cfg.glu_limit)
        elif self.etp is not None:
            # every rank of the group routes the same tokens through its slice of each expert; the partial outputs
            # are summed in token space (and the partial input / routing-weight gradients on the way back)
            from halo_b200.parallel.expert_tensor_parallel import copy_to_group, sum_from_group

            part = moe_ops.moe_experts(copy_to_group(h, self.etp), idx, copy_to_group(w, self.etp), self.experts_gate_up,
                                       self.experts_down, ctx.transport)
            out = sum_from_group(part, self.etp)
        else:
            out = moe_ops.moe_experts(h_experts, idx, w, bank_gate_up, bank_down, ctx.transport,
                                      skip_output=getattr(ctx, "output_unused", False))
        if self.shared_expert is not None:
            sh = self.shared_expert(h)
            if self.shared_gate is not None:
                sh = sh * torch.sigmoid(h.float() @ self.shared_gate.float().t()).to(h.dtype)
            out = out + sh
        return out


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, idx: int, dtype, device, n_local_experts: int, router_dtype=None, tp_size: int = 1,
                 etp=None):
        super().__init__()
        H = cfg.hidden_size
        self.input_layernorm = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.post_attention_layernorm = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        if cfg.layer_is_conv(idx):
            from .short_conv import ShortConv

            self.self_attn = ShortConv(cfg, dtype, device, tp_size, idx)
        elif cfg.layer_is_linear_attention(idx):
            from .gated_delta_net import GatedDeltaNet

            self.self_attn = GatedDeltaNet(cfg, dtype, device, tp_size, idx)
        elif cfg.attn_output_gate:
            self.self_attn = GatedAttention(cfg, dtype, device, tp_size, idx)
        elif cfg.kv_lora_rank:
            from .latent_attention import LatentAttention

            self.self_attn = LatentAttention(cfg, dtype, device, tp_size, idx)
        else:
            self.self_attn = Attention(cfg, dtype, device, tp_size, idx)
        if cfg.layer_is_moe(idx):
            # attention-only tensor parallelism for MoE layers: router and experts see this rank's token shard
            self.mlp = SparseMoE(cfg, dtype, device, n_local_experts, router_dtype, etp)
            self.mlp.layer_index = idx
        else:
            self.mlp = DenseMLP(H, cfg.intermediate_size, dtype, device, tp_size)
            self.mlp.activation = cfg.hidden_activation
        # Gemma: each block's output is normed as well before it joins the residual (``post_attention_layernorm`` is then
        # the norm of the attention OUTPUT, and the feed-forward block has its own pair)
        self.sandwich = cfg.sandwich_norms
        if self.sandwich:
            if cfg.hc_mult > 1:
                raise ValueError("output norms and hyper-connections are not combined")
            self.pre_feedforward_layernorm = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
            self.post_feedforward_layernorm = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.eps = cfg.rms_norm_eps
        # "full": the whole layer is re-run in the backward pass; "mlp": the attention half keeps its
        # activations (about 30 KB per token) and only the feed-forward half is re-run; "none": nothing is re-run
        self.recompute_policy = "full"

    def forward(self, x, ctx):
        if self.sandwich:
            return self.mlp_half(self.attention_half(x, ctx), ctx)
        h = rms_norm(x, self.input_layernorm, self.eps)
        a = self.self_attn(h, ctx)
        h2, x2 = add_rms_norm(a, x, self.post_attention_layernorm, self.eps)
        m = self.mlp(h2, ctx)
        return x2 + m

    def attention_half(self, x, ctx):
        a = self.self_attn(rms_norm(x, self.input_layernorm, self.eps), ctx)
        return x + (rms_norm(a, self.post_attention_layernorm, self.eps) if self.sandwich else a)

    def mlp_half(self, x2, ctx):
        if self.sandwich:
            m = self.mlp(rms_norm(x2, self.pre_feedforward_layernorm, self.eps), ctx)
            return x2 + rms_norm(m, self.post_feedforward_layernorm, self.eps)
        return x2 + self.mlp(rms_norm(x2, self.post_attention_layernorm, self.eps), ctx)


class HyperConnectedLayer(DecoderLayer):
    """The same two blocks on ``N`` residual streams ``[T, N, H]``: each block reads the streams collapsed by its
    hyper-connection and its output is mixed back into all of them."""

    def __init__(self, cfg: ModelConfig, idx: int, dtype, device, n_local_experts: int, router_dtype=None, tp_size: int = 1,
                 etp=None):
        super().__init__(cfg, idx, dtype, device, n_local_experts, router_dtype, tp_size, etp)
        from .hyper_connections import GatedResidual, HyperConnection

        self.gated = cfg.hc_kind == "gated"
        if self.gated:
            args = (cfg.hidden_size, cfg.hc_mult, cfg.hc_mix_rank, cfg.rms_norm_eps, dtype, device)
            self.attn_hc = GatedResidual(*args, seed=2 * idx)
            self.ffn_hc = GatedResidual(*args, seed=2 * idx + 1)
        elif cfg.hc_kind == "mhc":
            args = (cfg.hidden_size, cfg.hc_mult, cfg.hc_sinkhorn_iters, cfg.hc_eps, cfg.rms_norm_eps, device)
            self.attn_hc = HyperConnection(*args)
            self.ffn_hc = HyperConnection(*args)
        else:
            raise ValueError(f"hc_kind {cfg.hc_kind!r}: known kinds are 'mhc' and 'gated'")

    def _around(self, hc, block, streams):
        """``block`` on the collapsed streams, its output spread back over them."""
        if self.gated:
            from halo_b200.ops.streams import inject_streams

            collapsed, gates = hc(streams)
            return inject_streams(block(collapsed), streams, gates.to(streams.dtype))
        from .hyper_connections import mixed

        post, comb, collapsed = hc(streams)
        return mixed(block(collapsed), streams, post, comb)

    def attention_half(self, streams, ctx):
        return self._around(self.attn_hc, lambda x: self.self_attn(rms_norm(x, self.input_layernorm, self.eps), ctx), streams)

    def mlp_half(self, streams, ctx):
        return self._around(self.ffn_hc, lambda x: self.mlp(rms_norm(x, self.post_attention_layernorm, self.eps), ctx), streams)

    def forward(self, streams, ctx):
        return self.mlp_half(self.attention_half(streams, ctx), ctx)


class ForwardContext:
    """Per-batch state shared by all layers: attention plan, rotary table, expert transport."""

    def __init__(self, plan, rope, transport, record_routing=None, replay_topk=None, cp=None, tp=None):
        self.plan = plan
        self.tp = tp                 # TensorParallel when activations are token-sharded over a tensor-parallel group
        self.cp = cp                 # (ContextParallel, CPLayout) when the row is cut over a context-parallel group
        self.rope = rope
        self.transport = transport
        self.record_routing = record_routing
        self.replay_topk = replay_topk
        self.output_unused = False   # set while a layer is re-run only to rebuild its graph
        self.kv_cache = None         # halo_b200.inference.generate.KVCache while sampling
        self.attention_mask = None   # bool [T, T]: an explicit mask (tree packing) served by the masked-attention op
        self.rope_local = None       # rotary table of the windowed layers when their base differs (Gemma 3)
        self.query_scale = None      # [T] fp32: per-position stretch of the queries (Mistral 4), else None
        self.positions = None        # [T]: each token's index inside its document (the segment marks of convolution mixers)
        self._window_plans = {}      # window size -> attention plan cut to that window (built on first use)

    def window_plan(self, window: int):
        plan = self._window_plans.get(window)
        if plan is None:
            dev = self.plan.fwd.device if self.plan.fwd is not None else None
            plan = self._window_plans[window] = attn_ops.build_plan(self.plan.cu_seqlens, dev, window=window)
        return plan


class Qwen3Model(nn.Module):
    """Causal LM. ``forward`` returns the loss when ``labels`` are given, else final hidden states."""

    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device=None, transport=None,
                 gradient_checkpointing: bool = True, router_dtype=None, layer_range: tuple[int, int] | None = None,
                 has_embed: bool = True, has_head: bool = True, tensor_parallel=None, expert_tensor_parallel=None):
        super().__init__()
        self.cfg = cfg
        self.transport = transport or moe_ops.LocalTransport()
        if cfg.is_moe and cfg.num_experts % self.transport.n_ranks:
            raise ValueError(
                f"num_experts ({cfg.num_experts}) is not divisible by expert_parallel_size ({self.transport.n_ranks})")
        n_local = cfg.num_experts // self.transport.n_ranks if cfg.is_moe else 0
        self.gradient_checkpointing = gradient_checkpointing
        self.context_parallel = None      # halo_b200.parallel.context_parallel.ContextParallel when cp > 1
        self.tensor_parallel = tensor_parallel    # halo_b200.parallel.tensor_parallel.TensorParallel when tp > 1
        self.expert_tensor_parallel = expert_tensor_parallel
        tp_size = tensor_parallel.size if tensor_parallel is not None else 1
        if tp_size > 1:
            from halo_b200.parallel.tensor_parallel import check_divisibility

            check_divisibility(cfg, tp_size)
        lo, hi = layer_range or (0, cfg.num_hidden_layers)
        self.layer_range = (lo, hi)
        H = cfg.hidden_size
        self.embed_tokens = nn.Parameter(torch.empty(cfg.vocab_size, H, dtype=dtype, device=device)) if has_embed else None
        if cfg.hc_mult > 1 and (tp_size > 1 or (lo, hi) != (0, cfg.num_hidden_layers)):
            raise ValueError("hyper-connected models (hc_mult > 1) are built for data / expert parallel layouts: turn tensor "
                             "and pipeline parallelism off")
        layer_cls = HyperConnectedLayer if cfg.hc_mult > 1 else DecoderLayer
        self.layers = nn.ModuleList(
            [layer_cls(cfg, i, dtype, device, n_local, router_dtype, tp_size, expert_tensor_parallel) for i in range(lo, hi)])
        if cfg.hc_mult > 1 and has_head and cfg.hc_kind == "mhc":
            from .hyper_connections import HyperHead

            self.hc_head = HyperHead(H, cfg.hc_mult, cfg.hc_eps, cfg.rms_norm_eps, device)
        else:
            self.hc_head = None
        if cfg.num_nextn_predict_layers:
            if cfg.num_nextn_predict_layers != 1 or cfg.hc_mult > 1 or tp_size > 1 or (lo, hi) != (0, cfg.num_hidden_layers):
                raise ValueError("the multi-token-prediction head is built as one block on an unsliced, single-stage, "
                                 "plain-residual model")
            if cfg.mtp_objective not in ("joint", "detached"):
                raise ValueError(f"mtp_objective {cfg.mtp_objective!r}: known objectives are 'joint' and 'detached'")
            from .mtp import MTPHead

            self.mtp = MTPHead(cfg, dtype, device, n_local, router_dtype)
        else:
            self.mtp = None
        self.norm = nn.Parameter(torch.ones(H, dtype=dtype, device=device)) if has_head else None
        if has_head and not (cfg.tie_word_embeddings and has_embed):
            self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, H, dtype=dtype, device=device))
        else:
            self.register_parameter("lm_head", None)
        self.has_head = has_head
        # optional hook ``gate(params)`` called before a group of parameters is first read in a step;
        # an optimizer that updates parameters asynchronously uses it to order the reads
        self.param_gate = None
        self.layer_hooks = None          # halo_b200.parallel.zero3.Zero3Layers when the layers' matrices are sharded over the ranks

    # ---- initialisation ----------------------------------------------------------------------
    @torch.no_grad()
    def init_weights(self, seed: int = 0) -> None:
        """N(0, initializer_range) for matrices, ones for norms; per-tensor generators keyed by the
        global parameter name so any sharding of the experts draws the same values."""
        std = self.cfg.initializer_range
        from halo_b200.optim.adamw_bf16 import param_name_hash

        first = self.layer_range[0]
        for module in self.modules():
            if hasattr(module, "reset_parameters") and module is not self:
                module.reset_parameters()          # hyper-connections: the plain residual model's function
        for name, p in self.named_parameters():
            if "_hc." in name or name.startswith("hc_head."):
                continue
            if p.dim() == 1 or name.endswith("bias"):
                p.fill_(0.0 if name.endswith(("bias", "sinks")) else 1.0)
                continue
            dev = p.device
            if first and name.startswith("layers."):
                # a pipeline stage numbers its layers from 0: key the draw by the layer's global index
                _, li, rest = name.split(".", 2)
                name = f"layers.{int(li) + first}.{rest}"
            base = (seed * 1000003 + param_name_hash(name)) % (2**62)
            if getattr(p, "is_expert", False):
                # one generator per (parameter, global expert): any sharding draws the same values
                e0 = self.transport.rank * p.shape[0]
                etp = self.expert_tensor_parallel if getattr(p, "etp_kind", None) is not None else None
                for le in range(p.shape[0]):
                    g = torch.Generator(device=dev).manual_seed(base + e0 + le)
                    if etp is None:
                        p[le].normal_(0.0, std, generator=g)
                    else:
                        # draw the unsliced expert (same values under any width cut) and keep this rank's slice
                        from halo_b200.parallel.expert_tensor_parallel import slice_expert_bank

                        full_shape = ((p.shape[1] * etp.size, p.shape[2]) if p.etp_kind == "gate_up"
                                      else (p.shape[1], p.shape[2] * etp.size))
                        full = torch.empty(full_shape, dtype=p.dtype, device=dev).normal_(0.0, std, generator=g)
                        p[le].copy_(slice_expert_bank(p.etp_kind, full[None], etp.rank, etp.size)[0])
            elif getattr(p, "tp_kind", None) is not None:
                # draw the unsliced tensor (same values under any tensor-parallel width) and keep this rank's slice
                from halo_b200.parallel.tensor_parallel import slice_for_rank

                tp = self.tensor_parallel
                full_shape = {"qkv": (self.cfg.qkv_dim, *p.shape[1:]), "qkv_bias": (self.cfg.qkv_dim,), "o": (p.shape[0], p.shape[1] * tp.size),
                              "gate_up": (p.shape[0] * tp.size, p.shape[1]), "down": (p.shape[0], p.shape[1] * tp.size)}[p.tp_kind]
                g = torch.Generator(device=dev).manual_seed(base)
                full = torch.empty(full_shape, dtype=p.dtype, device=dev).normal_(0.0, std, generator=g)
                p.copy_(slice_for_rank(p.tp_kind, full, self.cfg, tp.rank, tp.size))
            else:
                g = torch.Generator(device=dev).manual_seed(base)
                p.normal_(0.0, std, generator=g)

    # ---- forward -----------------------------------------------------------------------------
    def make_context(self, position_ids, cu_seqlens, record_routing=None, replay_topk=None) -> ForwardContext:
        """``cu_seqlens`` always describes the whole packed row; under context parallelism ``position_ids``
        (like the token ids) are this rank's chunk of it."""
        dev = position_ids.device
        rope = self.rope(position_ids)
        if self.context_parallel is not None:
            layout, plan = self.context_parallel.layout_and_plan(cu_seqlens)
            return ForwardContext(plan, rope, self.transport, record_routing, replay_topk, (self.context_parallel, layout))
        plan = attn_ops.build_plan(cu_seqlens, device=dev)
        ctx = ForwardContext(plan, rope, self.transport, record_routing, replay_topk, tp=self.tensor_parallel)
        ctx.rope_local = self.rope_local(position_ids)
        ctx.query_scale = self.query_scale(position_ids)
        ctx.positions = position_ids.reshape(-1)
        return ctx

    def query_scale(self, position_ids):
        """``1 + beta * log(1 + floor(position / period))`` per token, or None for families without it."""
        beta, period = self.cfg.query_scale_beta, self.cfg.query_scale_period
        if not beta or not period:
            return None
        return 1.0 + beta * torch.log1p(torch.floor(position_ids.reshape(-1).float() / period))

    def rope_local(self, position_ids):
        """The windowed layers' own table (their rotary base, no scaling), or None when they share the full layers'."""
        if not self.cfg.rope_local_theta:
            return None
        exact = next(self.parameters()).dtype == torch.float32 and not position_ids.is_cuda
        return rope_table(position_ids, self.cfg.head_dim, self.cfg.rope_local_theta, None, self.cfg.max_position_embeddings,
                          round_bf16=not exact)

    def rope(self, position_ids):
        """cos / sin table of these positions, in the rounding of the model's dtype."""
        exact = next(self.parameters()).dtype == torch.float32 and not position_ids.is_cuda
        rotated = int(self.cfg.head_dim * self.cfg.partial_rotary_factor)      # partial rotary: the leading dims of a head
        return rope_table(position_ids, rotated, self.cfg.rope_theta, self.cfg.rope_scaling,
                          self.cfg.max_position_embeddings, round_bf16=not exact)

    def _gate(self, params):
        if self.param_gate is not None:
            self.param_gate(params)

    def embed(self, input_ids):
        self._gate([self.embed_tokens])
        x = torch.nn.functional.embedding(input_ids.reshape(-1), self.embed_tokens)
        if self.cfg.embedding_multiplier != 1.0:
            x = x * torch.tensor(self.cfg.embedding_multiplier, dtype=x.dtype, device=x.device)     # rounded to the model's dtype first
        return x

    def run_layers(self, x, ctx):
        hooks = self.layer_hooks          # sharded layer parameters: gathered around each layer's passes
        for i, layer in enumerate(self.layers):
            self._gate(layer.parameters())
            policy = layer.recompute_policy if (self.gradient_checkpointing and torch.is_grad_enabled()) else "none"
            if hooks is not None and torch.is_grad_enabled():
                if not self.gradient_checkpointing:
                    raise RuntimeError("sharded layer parameters are gathered per layer pass: training needs per-layer "
                                       "recomputation (gradient_checkpointing: true)")
                if policy != "mlp":
                    policy = "full"
            if policy == "full":
                x = recompute(layer, x, ctx, hooks, i)
            elif policy == "mlp":
                x = recompute_second_half(layer.attention_half, layer.mlp_half, x, ctx, hooks, i)
            elif hooks is not None:
                hooks.before_layer(i, backward=False)
                try:
                    x = layer(x, ctx)
                finally:
                    hooks.after_layer(i, backward=False)
            else:
                x = layer(x, ctx)
        return x

    def head_weight(self):
        w = self.lm_head if self.lm_head is not None else self.embed_tokens
        self._gate([w, self.norm])
        return w

    def trunk_states(self, input_ids, ctx):
        """The last layer's output, before the final norm (``[T, H]``)."""
        x = self.embed(input_ids)
        if self.cfg.hc_mult > 1:
            x = x.unsqueeze(1).expand(-1, self.cfg.hc_mult, -1).contiguous()      # every stream starts as the embedding
        x = self.run_layers(x, ctx)
        if self.hc_head is not None:
            x = self.hc_head(x)
        elif self.cfg.hc_mult > 1:
            x = x.float().mean(1).to(x.dtype)          # the gated variant reads the streams' mean
        return x

    def hidden_states(self, input_ids, position_ids, cu_seqlens, ctx=None):
        ctx = ctx or self.make_context(position_ids.reshape(-1), cu_seqlens)
        return rms_norm(self.trunk_states(input_ids, ctx), self.norm, self.cfg.rms_norm_eps)

    def mtp_states(self, trunk, input_ids, ctx):
        """The multi-token-prediction head's normed states for the shared output head."""
        nxt = torch.roll(input_ids.reshape(-1), -1)
        emb = torch.nn.functional.embedding(nxt, self.embed_tokens)
        if self.cfg.mtp_objective == "detached":
            trunk, emb = trunk.detach(), emb.detach()
        self._gate(self.mtp.parameters())
        return self.mtp(trunk, emb, ctx, self.gradient_checkpointing and torch.is_grad_enabled())

    def forward(self, input_ids, position_ids, cu_seqlens, labels=None, normalizer=None, ctx=None):
        """``labels`` are next-token targets already aligned with ``input_ids`` positions
        (-100 = not scored). Returns the summed CE divided by ``normalizer`` (default: scored tokens)."""
        if self.mtp is None or labels is None:
            h = self.hidden_states(input_ids, position_ids, cu_seqlens, ctx)
            if labels is None:
                return h
            if self.cfg.final_logit_softcapping:
                return self._capped_cross_entropy(h, labels.reshape(-1), normalizer)
            return fused_linear_cross_entropy(h, self.head_weight(), labels.reshape(-1), normalizer)
        from .mtp import shifted_targets

        if self.cfg.final_logit_softcapping:
            raise NotImplementedError("a multi-token-prediction head beside soft-capped logits is not built")
        ctx = ctx or self.make_context(position_ids.reshape(-1), cu_seqlens)
        trunk = self.trunk_states(input_ids, ctx)
        flat = labels.reshape(-1)
        if normalizer is None:
            normalizer = (flat != -100).sum().clamp(min=1)      # both terms share the next-token count
        w = self.head_weight()
        loss = fused_linear_cross_entropy(rms_norm(trunk, self.norm, self.cfg.rms_norm_eps), w, flat, normalizer)
        head_w = w.detach() if self.cfg.mtp_objective == "detached" else w
        head_loss = fused_linear_cross_entropy(self.mtp_states(trunk, input_ids, ctx), head_w, shifted_targets(flat, cu_seqlens),
                                               normalizer)
        self.last_mtp_loss = head_loss.detach()
        return loss + self.cfg.mtp_loss_weight * head_loss

    def token_logprobs(self, input_ids, position_ids, cu_seqlens, labels, want_entropy=False, ctx=None):
        h = self.hidden_states(input_ids, position_ids, cu_seqlens, ctx)
        if self.cfg.final_logit_softcapping:
            return self._capped_logprobs(h, labels.reshape(-1), want_entropy)
        return linear_logprobs(h, self.head_weight(), labels.reshape(-1), want_entropy=want_entropy)

    # ---- soft-capped output logits (Gemma 2): row chunks of logits through cap * tanh(. / cap), as tensor ops --------
    def capped_logits(self, h):
        cap = self.cfg.final_logit_softcapping
        z = h.float() @ self.head_weight().float().t()
        return cap * torch.tanh(z / cap) if cap else z

    def _capped_cross_entropy(self, h, labels, normalizer, chunk_rows: int = 4096):
        total = h.new_zeros((), dtype=torch.float32)
        count = (labels != -100).sum().clamp_min(1) if normalizer is None else normalizer
        for lo in range(0, h.shape[0], chunk_rows):
            total = total + torch.nn.functional.cross_entropy(self.capped_logits(h[lo:lo + chunk_rows]), labels[lo:lo + chunk_rows],
                                                              ignore_index=-100, reduction="sum")
        return total / count

    def _capped_logprobs(self, h, labels, want_entropy, chunk_rows: int = 4096):
        outs, ents = [], []
        for lo in range(0, h.shape[0], chunk_rows):
            logp = torch.log_softmax(self.capped_logits(h[lo:lo + chunk_rows]), dim=-1)
            lab = labels[lo:lo + chunk_rows]
            picked = logp.gather(-1, lab.clamp_min(0)[:, None]).squeeze(-1)
            outs.append(torch.where(lab == -100, torch.zeros_like(picked), picked))
            if want_entropy:
                ents.append(-(logp.exp() * logp).sum(-1).detach())
        return torch.cat(outs), (torch.cat(ents) if want_entropy else None)


def attention_half_bytes_per_token(cfg: ModelConfig, itemsize: int = 2) -> int:
    """Activation bytes per token that a layer keeps under the "mlp" recompute policy: normed input, fused
    QKV (before and after rotary + QK-norm), attention output, projected output, residual sum, softmax statistics."""
    q = cfg.num_attention_heads * cfg.head_dim
    return itemsize * (3 * cfg.hidden_size + 2 * cfg.qkv_dim + q) + 4 * cfg.num_attention_heads


def plan_recompute(model, tokens_per_step: int, free_bytes: int, reserve_bytes: int = 8 << 30, group=None) -> int:
    """Give as many layers as fit in ``free_bytes - reserve_bytes`` the lighter "mlp" policy (from the last layer
    backwards: those activations live shortest). Every rank of ``group`` adopts the smallest count any rank can
    afford, so all ranks run the same collectives. Returns the number of layers that were lightened.

    The role of the reference's measured ``gradient_checkpointing_plan: auto``
    (halo/models/gradient_checkpointing_plan.py)."""
    per_layer = attention_half_bytes_per_token(model.cfg, next(model.parameters()).element_size()) * tokens_per_step
    n = max(0, min(len(model.layers), int((free_bytes - reserve_bytes) // max(per_layer, 1))))
    if getattr(model, "layer_hooks", None) is not None and next(model.parameters()).is_cuda:
        # sharded layer parameters under the lighter policy: the attention half's saved references are read through the
        # parameters bound in the backward window, which holds for the tensor-op path the multi-process CPU tests run;
        # the GPU ops have not been run in that combination, so a plan does not choose it there by itself (setting
        # layer.recompute_policy = "mlp" by hand still takes it)
        n = 0
    if group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()):
        t = torch.tensor([n], dtype=torch.int64, device=next(model.parameters()).device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN, group=group)
        n = int(t.item())
    for i, layer in enumerate(model.layers):
        layer.recompute_policy = "mlp" if i >= len(model.layers) - n else "full"
    return n


def apply_lowp_compute(model, fmt: str) -> int:
    """Quantisation-aware training: every attention, dense feed-forward and routed-expert product rounds its operands
    to the block-scaled format ``fmt`` along the contraction axis (straight-through gradients; the master weights stay
    bf16). The router, the norms, the embedding and the output head keep full precision. Returns the number of
    modules switched (the reference's low-precision apply, halo/model_loading/parallel/lowp_compute.py)."""
    from halo_b200.ops.lowp import BLOCK_SIZE, FORMATS

    if fmt not in FORMATS:
        raise ValueError(f"unknown low-precision format {fmt!r}; known: {FORMATS}")
    bs = BLOCK_SIZE[fmt]
    widths = {model.cfg.hidden_size, model.cfg.num_attention_heads * model.cfg.head_dim}
    widths.add(model.cfg.moe_intermediate_size if model.cfg.is_moe else model.cfg.intermediate_size)
    if not all(model.cfg.layer_is_moe(i) for i in range(model.cfg.num_hidden_layers)):
        widths.add(model.cfg.intermediate_size)
    if model.cfg.shared_expert_intermediate_size:
        widths.add(model.cfg.shared_expert_intermediate_size)
    bad = sorted(w for w in widths if w % bs)
    if bad:
        raise ValueError(f"{fmt} scales blocks of {bs} along the contraction axis; the widths {bad} are no multiples of it")
    n = 0
    for module in model.modules():
        if isinstance(module, (Attention, DenseMLP, SparseMoE)):
            module.lowp = fmt
            n += 1
    return n


def build_model(cfg: ModelConfig, device="cpu", dtype=None, transport=None, seed: int = 0,
                gradient_checkpointing: bool = True, init: bool = True, **kw) -> Qwen3Model:
    device = torch.device(device)
    dtype = dtype or (torch.bfloat16 if device.type == "cuda" else torch.float32)
    model = Qwen3Model(cfg, dtype=dtype, device=device, transport=transport,
                       gradient_checkpointing=gradient_checkpointing, **kw)
    if init:
        model.init_weights(seed)
    return model
