"""How many (query, key) pairs each layer's attention visits in a packed row: the attention term of the model-FLOPs
count. A full layer visits every causal pair inside a document, ``n (n + 1) / 2``; a windowed layer visits at most
``window`` keys per query, ``w (w + 1) / 2 + (n - w) w`` for a document longer than the window. Families that mix
windowed and full layers (gpt-oss, Qwen2 with ``max_window_layers``) get one figure per layer.
(The role of halo/models/attention/layout.py: the per-layer keys-visited model behind the MFU attention term.)"""

from __future__ import annotations

import numpy as np


def causal_pairs(doc_lengths, window: int = 0) -> float:
    n = np.asarray(doc_lengths, dtype=np.float64)
    if not window:
        return float((n * (n + 1) / 2).sum())
    w = float(window)
    short = n * (n + 1) / 2
    long = w * (w + 1) / 2 + (n - w) * w
    return float(np.where(n <= w, short, long).sum())


def layer_windows(cfg) -> list[int]:
    """The window of every layer (0 = full attention)."""
    kinds = getattr(cfg, "layer_types", None)
    w = int(getattr(cfg, "sliding_window", 0) or 0)
    if not w:
        return [0] * cfg.num_hidden_layers
    if not kinds:
        return [w] * cfg.num_hidden_layers
    return [w if (i >= len(kinds) or kinds[i] == "sliding_attention") else 0 for i in range(cfg.num_hidden_layers)]


def keys_visited_per_layer(cfg, cu_seqlens) -> list[float]:
    lengths = np.diff(np.asarray(cu_seqlens, dtype=np.float64))
    by_window = {}
    kinds = getattr(cfg, "layer_types", None) or []
    # a short-convolution or linear-attention layer does a fixed amount of work per token: no pair count
    return [0.0 if i < len(kinds) and kinds[i] in ("conv", "linear_attention") else by_window.setdefault(w, causal_pairs(lengths, w))
            for i, w in enumerate(layer_windows(cfg))]


def attention_flops(cfg, cu_seqlens) -> float:
    """Forward + backward FLOPs of the score and value products: 12 * head_dim * heads per visited pair (latent
    attention: 6 * (query/key width + value width), the two products have different widths there)."""
    width = (cfg.qk_nope_head_dim + cfg.qk_rope_head_dim + cfg.v_head_dim) / 2.0 if getattr(cfg, "kv_lora_rank", 0) else cfg.head_dim
    return 12.0 * width * cfg.num_attention_heads * sum(keys_visited_per_layer(cfg, cu_seqlens))
