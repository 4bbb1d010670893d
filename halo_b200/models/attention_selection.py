"""Which attention path serves a model, decided once from its configuration and device and logged at load time
(the role of halo/models/attention/selection.py:383-462, with one in-tree kernel family instead of five backends).

* ``flash``     - the sm_100a flash kernels: bf16 on CUDA, head_dim 128 (64 runs zero-padded to 128), causal attention
                  inside packed documents, grouped-query heads; optionally a sliding window (work lists cut to the
                  window, its left edge masked in the kernels), attention sinks (one logit per head added to the
                  denominator in the forward's last step; the backward kernels are unchanged) and a configured softmax
                  scale; deterministic forward and backward (no atomics), so a determinism request changes nothing.
* ``masked``    - the masked-attention op (query tiles under an explicit ``[T, T]`` mask): soft-capped scores, latent
                  attention, tree packing, and windows / sinks wherever the flash kernels cannot take them (CPU, fp32,
                  other head dims, context-parallel rows); element-wise half on the masked-softmax kernel, products on
                  library GEMMs.
* ``reference`` - tensor ops: CPU runs, fp32 models, head dims the kernels are not built for.
"""

from __future__ import annotations

import torch


def attention_path(cfg, device, dtype, tree_packing: bool = False) -> tuple[str, str]:
    device = torch.device(device)
    if getattr(cfg, "kv_lora_rank", 0):
        return "masked", "latent attention: query / key width differs from the value width"
    if getattr(cfg, "attn_logit_softcapping", 0.0):
        return "masked", "soft-capped attention scores: the flash kernel has no tanh between scores and softmax"
    if tree_packing:
        return "masked", "tree packing: branches attend a shared trunk"
    extras = []
    if cfg.sliding_window:
        mixed = " on the layers named sliding_attention" if getattr(cfg, "layer_types", None) else ""
        extras.append(f"sliding_window={cfg.sliding_window}{mixed} in the windowed kernels")
    if getattr(cfg, "attention_sinks", False):
        extras.append("sink logits added to the denominator in the forward kernel")
    if (getattr(cfg, "query_pre_attn_scalar", 0) or cfg.head_dim) != cfg.head_dim:
        extras.append(f"softmax scale {cfg.query_pre_attn_scalar}^-0.5")
    flash_ok = device.type == "cuda" and dtype == torch.bfloat16 and cfg.head_dim in (64, 128)
    if not flash_ok:
        why = (f"device {device.type}" if device.type != "cuda" else f"dtype {dtype} (the kernels take bf16)"
               if dtype != torch.bfloat16 else f"head_dim {cfg.head_dim} (the kernels are built for 128, and 64 zero-padded)")
        return ("masked" if extras else "reference"), why + ("; " + "; ".join(extras) if extras else "")
    width = "head_dim 128" if cfg.head_dim == 128 else "head_dim 64 zero-padded to the 128-wide kernels"
    return "flash", f"bf16, {width}, packed causal rows" + ("; " + "; ".join(extras) if extras else "")


def describe(cfg, device, dtype, tree_packing: bool = False) -> str:
    path, why = attention_path(cfg, device, dtype, tree_packing)
    rotary = "fused QK-norm + RoPE kernel" if path == "flash" and cfg.partial_rotary_factor == 1.0 and cfg.head_dim == 128 else "rotary as tensor ops"
    return f"attention path: {path} ({why}); {rotary}"
