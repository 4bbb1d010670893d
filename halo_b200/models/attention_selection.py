"""Which attention path serves a model, decided once from its configuration and device and logged at load time
(the role of halo/models/attention/selection.py:383-462, with one in-tree kernel family instead of five backends).

* ``flash``     - the sm_100a flash kernels: bf16 on CUDA, head_dim 128, causal attention inside packed documents,
                  grouped-query heads, optionally a sliding window (work lists cut to the window, its left edge masked
                  in the kernels); deterministic forward and backward (no atomics), so a determinism request changes
                  nothing.
* ``masked``    - the masked-attention op (query tiles under an explicit ``[T, T]`` mask): attention sinks, soft-capped
                  scores, tree packing, and sliding windows wherever the flash kernels cannot take them (CPU, fp32,
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
    if (getattr(cfg, "query_pre_attn_scalar", 0) or cfg.head_dim) != cfg.head_dim and not cfg.sliding_window:
        return "masked", f"softmax scale {cfg.query_pre_attn_scalar}^-0.5: the flash kernel scales by head_dim^-0.5"
    if getattr(cfg, "attention_sinks", False):
        return "masked", "attention sinks: the flash kernel's softmax has no extra logit"
    if tree_packing:
        return "masked", "tree packing: branches attend a shared trunk"
    if cfg.sliding_window:
        mixed = " on the layers named sliding_attention" if getattr(cfg, "layer_types", None) else ""
        flash_ok = device.type == "cuda" and dtype == torch.bfloat16 and cfg.head_dim == 128
        if not flash_ok:
            return "masked", f"sliding_window={cfg.sliding_window}{mixed}: windowed flash kernels need bf16 on CUDA and head_dim 128"
        return "flash", f"bf16, head_dim 128, packed causal rows; sliding_window={cfg.sliding_window}{mixed} in the windowed kernels"
    if device.type != "cuda":
        return "reference", f"device {device.type}"
    if dtype != torch.bfloat16:
        return "reference", f"dtype {dtype} (the kernels take bf16)"
    if cfg.head_dim != 128:
        return "reference", f"head_dim {cfg.head_dim} (the kernels are built for 128)"
    return "flash", "bf16, head_dim 128, packed causal rows"


def describe(cfg, device, dtype, tree_packing: bool = False) -> str:
    path, why = attention_path(cfg, device, dtype, tree_packing)
    rotary = "fused QK-norm + RoPE kernel" if path == "flash" and cfg.partial_rotary_factor == 1.0 else "rotary as tensor ops"
    return f"attention path: {path} ({why}); {rotary}"
