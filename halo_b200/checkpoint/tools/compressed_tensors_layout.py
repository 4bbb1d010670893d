"""The ``quantization_config`` block that compressed-tensors loaders (vLLM's among them) read from ``config.json``,
for a checkpoint whose matrices were written in a block-scaled format by ``lowp_convert export``.

Nothing here reads weights: the exporter passes the names of the modules it quantised; this module turns them into
``re:`` targets (one pattern per projection kind, so the block stays short on a 48-layer model) and names the format's
element type, group size and scale type. Counterpart of halo/checkpoint/tools/compressed_tensors_layout.py:1-126.
"""

from __future__ import annotations

import re

FORMAT_SCHEMES = {
    # element bits / type, group (block) size, scale storage
    "mxfp8": {"num_bits": 8, "type": "float", "group_size": 32, "scale_dtype": "e8m0", "format": "mxfp8-quantized"},
    "mxfp4": {"num_bits": 4, "type": "float", "group_size": 32, "scale_dtype": "e8m0", "format": "mxfp4-pack-quantized"},
    "nvfp4": {"num_bits": 4, "type": "float", "group_size": 16, "scale_dtype": "float8_e4m3fn", "format": "nvfp4-pack-quantized"},
}


def module_targets(module_names: list[str]) -> list[str]:
    """``re:`` patterns covering the given modules: layer and expert indices (purely numeric name parts) are generalised
    to ``\\d+``, so a 48-layer model needs one pattern per projection kind."""
    patterns = set()
    for name in module_names:
        parts = [r"\d+" if part.isdigit() else re.escape(part) for part in name.split(".")]
        patterns.add("re:" + r"\.".join(parts))
    return sorted(patterns)


def quantization_config(fmt: str, quantized_modules: list[str], kept_modules: list[str]) -> dict:
    if fmt not in FORMAT_SCHEMES:
        raise ValueError(f"no compressed-tensors scheme for {fmt!r}; known: {sorted(FORMAT_SCHEMES)}")
    s = FORMAT_SCHEMES[fmt]
    targets = module_targets(quantized_modules)
    compiled = [re.compile(t[3:] + r"$") for t in targets]
    # a generalised pattern must not sweep in a module the exporter kept in bf16
    ignore = sorted(k for k in kept_modules if any(c.match(k) for c in compiled))
    weights = {"num_bits": s["num_bits"], "type": s["type"], "strategy": "group", "group_size": s["group_size"],
               "symmetric": True, "dynamic": False, "scale_dtype": s["scale_dtype"]}
    return {"quant_method": "compressed-tensors", "format": s["format"], "quantization_status": "compressed",
            "config_groups": {"group_0": {"targets": targets, "weights": weights, "input_activations": None}},
            "ignore": ignore}
