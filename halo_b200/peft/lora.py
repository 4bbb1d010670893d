"""Low-rank adapters (LoRA) for the decoder: frozen base weights, trainable ``B A`` pairs on the named projections.

Targets use the hub's projection names. ``q_proj`` / ``k_proj`` / ``v_proj`` / ``o_proj`` / ``gate_proj`` /
``up_proj`` / ``down_proj`` adapt the attention and the dense (and shared-expert) feed-forward projections through the
low-rank path ``y += scale * (x A^T) B^T`` - the frozen product stays on the tcgen05 GEMM and skips its weight
gradient, the two skinny products are plain library GEMMs. ``experts.gate_proj`` / ``experts.up_proj`` /
``experts.down_proj`` adapt the routed experts: every local expert owns its pair, and the grouped expert products run
on the effective banks ``W + scale * B A`` (one batched product per bank and pass), so dispatch, grouped GEMMs and
combine are the ones of full fine-tuning while the optimizer sees only the pairs. ``all-linear`` names all ten.

Adapters are written in the PEFT layout (``adapter_config.json`` + ``adapter_model.safetensors`` with
``base_model.model.<hub module>.lora_A.weight`` names), expert pairs one per global expert, so
``peft.PeftModel.from_pretrained`` reads the attention / dense part and
:mod:`halo_b200.checkpoint.tools.merge_adapter` folds all of it into a base checkpoint.

The role of the reference's PEFT set-up and expert-LoRA peel (halo/model_loading/parallel/peft_setup.py:39-120,
halo/models/moe/expert_lora_spec.py).
"""

from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F

DENSE_TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
EXPERT_TARGETS = ("experts.gate_proj", "experts.up_proj", "experts.down_proj")
ADAPTER_WEIGHTS = "adapter_model.safetensors"
ADAPTER_CONFIG = "adapter_config.json"


@dataclass
class LoraSpec:
    r: int = 16
    alpha: float = 32.0
    dropout: float = 0.0
    target_modules: list[str] = field(default_factory=lambda: ["q_proj", "k_proj", "v_proj", "o_proj"])

    def __post_init__(self):
        if isinstance(self.target_modules, str):
            self.target_modules = [self.target_modules]
        if "all-linear" in self.target_modules:
            self.target_modules = list(DENSE_TARGETS + EXPERT_TARGETS)
        unknown = [t for t in self.target_modules if t not in DENSE_TARGETS + EXPERT_TARGETS]
        if unknown:
            raise ValueError(f"unknown LoRA targets {unknown}; known: {list(DENSE_TARGETS + EXPERT_TARGETS)} or 'all-linear'")
        if self.r <= 0:
            raise ValueError("the LoRA rank must be positive")
        if not 0.0 <= self.dropout < 1.0:
            raise ValueError("LoRA dropout must lie in [0, 1)")

    @property
    def scale(self) -> float:
        return self.alpha / self.r

    @property
    def dense_targets(self) -> list[str]:
        return [t for t in self.target_modules if t in DENSE_TARGETS]

    @property
    def expert_targets(self) -> list[str]:
        return [t.split(".", 1)[1] for t in self.target_modules if t in EXPERT_TARGETS]

    def peft_config(self, base_model: str = "") -> dict:
        return {"peft_type": "LORA", "task_type": "CAUSAL_LM", "base_model_name_or_path": base_model, "r": self.r,
                "lora_alpha": self.alpha, "lora_dropout": self.dropout, "bias": "none", "fan_in_fan_out": False,
                "inference_mode": True, "target_modules": self.dense_targets,
                "halo_expert_target_modules": self.expert_targets}

    @classmethod
    def from_peft_config(cls, d: dict) -> "LoraSpec":
        targets = list(d.get("target_modules") or []) + [f"experts.{t}" for t in d.get("halo_expert_target_modules") or []]
        return cls(r=int(d["r"]), alpha=float(d["lora_alpha"]), dropout=float(d.get("lora_dropout", 0.0)), target_modules=targets)


def _init_pair(a: torch.Tensor, b: torch.Tensor, seed: int) -> None:
    """PEFT's default: ``A`` uniform with the Kaiming bound of ``a = sqrt(5)`` (that is ``1 / sqrt(fan_in)``), ``B`` zero, so
    the adapted model starts as the base model."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    bound = 1.0 / math.sqrt(a.shape[-1])
    a.copy_((torch.rand(a.shape, generator=g, dtype=torch.float32) * 2.0 - 1.0).mul_(bound).to(a.dtype))
    b.zero_()


class LoraSet(nn.Module):
    """The pairs of one module's projections: ``A[target]`` is ``[r, in]``, ``B[target]`` is ``[out, r]``."""

    def __init__(self, spec: LoraSpec, shapes: dict[str, tuple[int, int]], dtype, device, seed: int):
        super().__init__()
        self.scale, self.p_drop = spec.scale, spec.dropout
        self.A, self.B = nn.ParameterDict(), nn.ParameterDict()
        for i, (target, (n_out, n_in)) in enumerate(shapes.items()):
            a = torch.empty(spec.r, n_in, dtype=dtype, device=device)
            b = torch.empty(n_out, spec.r, dtype=dtype, device=device)
            with torch.no_grad():
                _init_pair(a, b, seed * 131 + i)
            self.A[target], self.B[target] = nn.Parameter(a), nn.Parameter(b)

    def __contains__(self, target: str) -> bool:
        return target in self.A

    def delta(self, target: str, x: torch.Tensor) -> torch.Tensor:
        if self.p_drop and self.training:
            x = F.dropout(x, self.p_drop)
        return F.linear(F.linear(x, self.A[target]), self.B[target]) * self.scale

    def add_fused(self, x: torch.Tensor, y: torch.Tensor, parts: list[tuple[str, int, int]]) -> torch.Tensor:
        """``y`` is a fused projection of ``x`` whose column ranges ``parts`` belong to separate hub projections."""
        if not any(t in self for t, _, _ in parts):
            return y
        return torch.cat([y[:, lo:hi] + self.delta(t, x) if t in self else y[:, lo:hi] for t, lo, hi in parts], dim=-1)


class ExpertLora(nn.Module):
    """One pair per local expert and target: ``A_<t>`` is ``[E_local, r, in]``, ``B_<t>`` ``[E_local, out, r]``."""

    def __init__(self, spec: LoraSpec, n_local: int, first_expert: int, hidden: int, width: int, dtype, device, seed: int):
        super().__init__()
        self.scale = spec.scale
        self.targets = spec.expert_targets
        shapes = {"gate_proj": (width, hidden), "up_proj": (width, hidden), "down_proj": (hidden, width)}
        for ti, target in enumerate(("gate_proj", "up_proj", "down_proj")):
            if target not in self.targets:
                continue
            n_out, n_in = shapes[target]
            a = torch.empty(n_local, spec.r, n_in, dtype=dtype, device=device)
            b = torch.empty(n_local, n_out, spec.r, dtype=dtype, device=device)
            with torch.no_grad():
                for le in range(n_local):     # keyed by the global expert: any expert-parallel width draws the same pairs
                    _init_pair(a[le], b[le], (seed * 131 + ti) * 100003 + first_expert + le)
            pa, pb = nn.Parameter(a), nn.Parameter(b)
            pa.is_expert = pb.is_expert = True
            setattr(self, f"A_{target}", pa)
            setattr(self, f"B_{target}", pb)

    def _delta(self, target: str) -> torch.Tensor:
        return torch.bmm(getattr(self, f"B_{target}"), getattr(self, f"A_{target}")) * self.scale

    def effective_banks(self, gate_up: torch.Tensor, down: torch.Tensor):
        """``(W_gate_up + delta, W_down + delta)``: the banks the grouped products run on."""
        width = gate_up.shape[1] // 2
        if "gate_proj" in self.targets or "up_proj" in self.targets:
            zero = None
            halves = []
            for target in ("gate_proj", "up_proj"):
                if target in self.targets:
                    halves.append(self._delta(target))
                else:
                    zero = zero if zero is not None else gate_up.new_zeros(gate_up.shape[0], width, gate_up.shape[2])
                    halves.append(zero)
            gate_up = gate_up + torch.cat(halves, dim=1)
        if "down_proj" in self.targets:
            down = down + self._delta("down_proj")
        return gate_up, down


def apply_lora(model, spec: LoraSpec, seed: int = 0) -> dict:
    """Freeze every base parameter and attach the adapters ``spec`` names. Returns parameter counts."""
    if getattr(model, "tensor_parallel", None) is not None or getattr(model, "expert_tensor_parallel", None) is not None:
        raise ValueError("LoRA adapters are built for unsliced projections: turn tensor / expert-tensor parallelism off")
    if getattr(model, "lora_spec", None) is not None:
        raise ValueError("the model already carries adapters")
    cfg = model.cfg
    attention_targets = sorted(set(spec.dense_targets) & {"q_proj", "k_proj", "v_proj", "o_proj"})
    if getattr(cfg, "kv_lora_rank", 0) and attention_targets:
        raise ValueError(f"targets {attention_targets}: latent attention has no such projections (its low-rank bottlenecks are "
                         f"already adapters of a kind); target the feed-forward blocks or the routed experts")
    if getattr(cfg, "attn_output_gate", False) and "q_proj" in attention_targets:
        raise ValueError("target q_proj: this family's query projection also produces the output gate (rows interleaved per head); "
                         "target k_proj / v_proj / o_proj, the feed-forward blocks or the routed experts")
    for p in model.parameters():
        p.requires_grad_(False)
    ref = next(model.parameters())
    dtype, device = ref.dtype, ref.device
    H, D = cfg.hidden_size, cfg.head_dim
    q_rows, kv_rows = cfg.num_attention_heads * D, cfg.num_key_value_heads * D
    dense = set(spec.dense_targets)
    first_layer = model.layer_range[0]
    tr = model.transport
    found_experts = False
    for li, layer in enumerate(model.layers):
        gi = li + first_layer
        shapes = {t: s for t, s in (("q_proj", (q_rows, H)), ("k_proj", (kv_rows, H)), ("v_proj", (kv_rows, H)),
                                    ("o_proj", (H, q_rows))) if t in dense}
        if hasattr(layer.self_attn, "conv_taps") or hasattr(layer.self_attn, "gdn_conv"):
            shapes = {}            # a convolution / linear-attention mixer has no q / k / v / o projections: attention targets skip the layer
        layer.self_attn.lora = LoraSet(spec, shapes, dtype, device, seed * 7919 + gi * 4 + 0) if shapes else None
        mlps = []
        if hasattr(layer.mlp, "experts_gate_up"):
            found_experts = True
            if spec.expert_targets:
                n_local = layer.mlp.experts_gate_up.shape[0]
                layer.mlp.expert_lora = ExpertLora(spec, n_local, tr.rank * n_local, H, cfg.moe_intermediate_size, dtype,
                                                   device, seed * 7919 + gi * 4 + 1)
            if layer.mlp.shared_expert is not None:
                mlps.append((layer.mlp.shared_expert, cfg.shared_expert_intermediate_size, 2))
        else:
            mlps.append((layer.mlp, cfg.intermediate_size, 3))
        for mlp, width, salt in mlps:
            shapes = {t: s for t, s in (("gate_proj", (width, H)), ("up_proj", (width, H)), ("down_proj", (H, width)))
                      if t in dense}
            mlp.lora = LoraSet(spec, shapes, dtype, device, seed * 7919 + gi * 4 + salt) if shapes else None
    if spec.expert_targets and not found_experts:
        raise ValueError(f"targets {['experts.' + t for t in spec.expert_targets]} name routed experts, but the model has none")
    model.lora_spec = spec
    trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)
    if trainable == 0:
        raise ValueError(f"targets {spec.target_modules} match no projection of this model")
    return {"trainable": trainable, "frozen": sum(p.numel() for p in model.parameters() if not p.requires_grad)}


# ---- PEFT-layout names ------------------------------------------------------------------------------------------
def _module_adapters(model):
    """Yields ``(hub module path, A [r, in], B [out, r])`` for every pair, expert pairs per LOCAL expert with their
    global index in the path."""
    from halo_b200.checkpoint.hub_layout import MOE_HUB_NAMES

    cfg = model.cfg
    block, gate_name, up_name, down_name = MOE_HUB_NAMES.get(cfg.family, MOE_HUB_NAMES["qwen3_moe"])
    expert_names = {"gate_proj": gate_name, "up_proj": up_name, "down_proj": down_name}
    first_layer = model.layer_range[0]
    for li, layer in enumerate(model.layers):
        pre = f"model.layers.{li + first_layer}."
        lora = getattr(layer.self_attn, "lora", None)
        if lora is not None:
            for t in lora.A:
                yield pre + f"self_attn.{t}", lora.A[t], lora.B[t]
        if hasattr(layer.mlp, "experts_gate_up"):
            shared = getattr(layer.mlp.shared_expert, "lora", None) if layer.mlp.shared_expert is not None else None
            if shared is not None:
                for t in shared.A:
                    yield pre + f"mlp.shared_expert.{t}", shared.A[t], shared.B[t]
            ex = getattr(layer.mlp, "expert_lora", None)
            if ex is not None:
                n_local = layer.mlp.experts_gate_up.shape[0]
                e0 = model.transport.rank * n_local
                for t in ex.targets:
                    a, b = getattr(ex, f"A_{t}"), getattr(ex, f"B_{t}")
                    for le in range(n_local):
                        yield pre + f"{block}.experts.{e0 + le}.{expert_names[t]}", a[le], b[le]
        else:
            lora = getattr(layer.mlp, "lora", None)
            if lora is not None:
                for t in lora.A:
                    yield pre + f"mlp.{t}", lora.A[t], lora.B[t]


def adapter_state_dict(model) -> dict[str, torch.Tensor]:
    """This rank's pairs under PEFT names."""
    out = {}
    for path, a, b in _module_adapters(model):
        out[f"base_model.model.{path}.lora_A.weight"] = a.detach()
        out[f"base_model.model.{path}.lora_B.weight"] = b.detach()
    return out


def save_adapters(model, directory: str, base_model: str = "", is_writer: bool = True, group=None) -> None:
    """COLLECTIVE over the expert group when routed experts carry adapters: their pairs are gathered on the writer.
    Writes ``adapter_config.json`` and ``adapter_model.safetensors``."""
    import torch.distributed as dist
    from safetensors.torch import save_file

    from halo_b200.checkpoint.atomic import atomic_write_json, staged_path

    state = {k: v.cpu().contiguous() for k, v in adapter_state_dict(model).items()}
    tr = model.transport
    if getattr(tr, "n_ranks", 1) > 1 and model.lora_spec.expert_targets:
        mine = {k: v for k, v in state.items() if ".experts." in k}
        gathered = [None] * tr.n_ranks
        dist.all_gather_object(gathered, mine, group=getattr(tr, "group", None))
        for part in gathered:
            state.update(part)
    if not is_writer:
        return
    os.makedirs(directory, exist_ok=True)
    with staged_path(os.path.join(directory, ADAPTER_WEIGHTS)) as tmp:
        save_file(state, tmp, metadata={"format": "pt"})
    atomic_write_json(os.path.join(directory, ADAPTER_CONFIG), model.lora_spec.peft_config(base_model))


@torch.no_grad()
def load_adapters(model, directory: str, strict: bool = True) -> int:
    """Fill the model's pairs from a directory :func:`save_adapters` wrote (each rank takes its own experts)."""
    from safetensors import safe_open

    n = 0
    with safe_open(os.path.join(directory, ADAPTER_WEIGHTS), "pt") as f:
        keys = set(f.keys())
        for path, a, b in _module_adapters(model):
            for suffix, dst in (("lora_A", a), ("lora_B", b)):
                key = f"base_model.model.{path}.{suffix}.weight"
                if key not in keys:
                    if strict:
                        raise KeyError(f"{key} is absent from {directory!r}")
                    continue
                dst.copy_(f.get_tensor(key).to(dst.dtype))
                n += 1
    return n


def read_adapter_spec(directory: str) -> LoraSpec:
    return LoraSpec.from_peft_config(json.load(open(os.path.join(directory, ADAPTER_CONFIG))))


@torch.no_grad()
def merge_adapters_into_weights(model) -> None:
    """Fold every pair into its frozen base weight (``W += scale * B A``) and reset ``B`` to zero: the model computes
    the same function with plain weights."""
    cfg = model.cfg
    D = cfg.head_dim
    q_rows, kv_rows = cfg.num_attention_heads * D, cfg.num_key_value_heads * D
    for layer in model.layers:
        lora = getattr(layer.self_attn, "lora", None)
        if lora is not None:
            rows = {"q_proj": (0, q_rows), "k_proj": (q_rows, q_rows + kv_rows), "v_proj": (q_rows + kv_rows, q_rows + 2 * kv_rows)}
            for t in lora.A:
                delta = (lora.B[t].float() @ lora.A[t].float()) * lora.scale
                if t == "o_proj":
                    layer.self_attn.o_proj.add_(delta.to(layer.self_attn.o_proj.dtype))
                else:
                    lo, hi = rows[t]
                    layer.self_attn.qkv_proj[lo:hi].add_(delta.to(layer.self_attn.qkv_proj.dtype))
                lora.B[t].zero_()
        mlps = [layer.mlp.shared_expert] if hasattr(layer.mlp, "experts_gate_up") else [layer.mlp]
        for mlp in mlps:
            lora = getattr(mlp, "lora", None) if mlp is not None else None
            if lora is None:
                continue
            width = mlp.gate_up_proj.shape[0] // 2
            for t in lora.A:
                delta = (lora.B[t].float() @ lora.A[t].float()) * lora.scale
                if t == "down_proj":
                    mlp.down_proj.add_(delta.to(mlp.down_proj.dtype))
                else:
                    lo = 0 if t == "gate_proj" else width
                    mlp.gate_up_proj[lo:lo + width].add_(delta.to(mlp.gate_up_proj.dtype))
                lora.B[t].zero_()
        ex = getattr(layer.mlp, "expert_lora", None)
        if ex is not None:
            gu, dn = ex.effective_banks(layer.mlp.experts_gate_up, layer.mlp.experts_down)
            layer.mlp.experts_gate_up.copy_(gu)
            layer.mlp.experts_down.copy_(dn)
            for t in ex.targets:
                getattr(ex, f"B_{t}").zero_()


def is_adapter_parameter(name: str) -> bool:
    return ".lora." in name or ".expert_lora." in name


@torch.no_grad()
def merged_weight(model, name: str, p: torch.Tensor) -> torch.Tensor:
    """The base parameter ``name`` with its adapters folded in (the parameter itself when it has none); the model
    is left as it is. Used by merged saves."""
    parts = name.split(".")
    if parts[0] != "layers":
        return p.detach()
    layer = model.layers[int(parts[1])]
    rest = ".".join(parts[2:])
    cfg = model.cfg
    D = cfg.head_dim
    q_rows, kv_rows = cfg.num_attention_heads * D, cfg.num_key_value_heads * D

    def folded(lora, pieces):
        out = p.detach().clone()
        for t, lo, hi in pieces:
            if lora is not None and t in lora:
                out[lo:hi].add_(((lora.B[t].float() @ lora.A[t].float()) * lora.scale).to(out.dtype))
        return out

    if rest == "self_attn.qkv_proj":
        return folded(getattr(layer.self_attn, "lora", None),
                      [("q_proj", 0, q_rows), ("k_proj", q_rows, q_rows + kv_rows), ("v_proj", q_rows + kv_rows, q_rows + 2 * kv_rows)])
    if rest == "self_attn.o_proj":
        return folded(getattr(layer.self_attn, "lora", None), [("o_proj", 0, p.shape[0])])
    for prefix, mlp in (("mlp.shared_expert.", getattr(layer.mlp, "shared_expert", None)), ("mlp.", layer.mlp)):
        if mlp is None or not rest.startswith(prefix) or not hasattr(mlp, "gate_up_proj"):
            continue
        tail = rest[len(prefix):]
        if tail == "gate_up_proj":
            width = p.shape[0] // 2
            return folded(getattr(mlp, "lora", None), [("gate_proj", 0, width), ("up_proj", width, 2 * width)])
        if tail == "down_proj":
            return folded(getattr(mlp, "lora", None), [("down_proj", 0, p.shape[0])])
    ex = getattr(layer.mlp, "expert_lora", None)
    if ex is not None and rest in ("mlp.experts_gate_up", "mlp.experts_down"):
        gate_up, down = ex.effective_banks(layer.mlp.experts_gate_up, layer.mlp.experts_down)
        return (gate_up if rest == "mlp.experts_gate_up" else down).detach()
    return p.detach()
