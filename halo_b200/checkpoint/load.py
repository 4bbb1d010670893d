"""Lazy SafeTensors loading: every rank reads only the tensors (and expert slices) it owns, straight
into its parameters, from a standard hub-layout checkpoint - sharded or single file. A coverage
gate refuses a checkpoint that leaves any parameter untouched, so nothing is silently left at its
random initialisation (the role of halo/model_loading/lazy_safetensors/*,
halo/model_loading/parallel/ep.py and checkpoint_coverage.py)."""

from __future__ import annotations

import json
import os

import torch
from safetensors import safe_open

from .hub_layout import hub_sources
from .writing import INDEX_NAME, SINGLE_NAME


class CheckpointIndex:
    """hub tensor name -> file, for single-file and sharded checkpoints."""

    def __init__(self, directory: str):
        self.directory = directory
        idx = os.path.join(directory, INDEX_NAME)
        if os.path.isfile(idx):
            self.weight_map = json.load(open(idx))["weight_map"]
        elif os.path.isfile(os.path.join(directory, SINGLE_NAME)):
            with safe_open(os.path.join(directory, SINGLE_NAME), "pt") as f:
                self.weight_map = {k: SINGLE_NAME for k in f.keys()}
        else:
            raise FileNotFoundError(f"no SafeTensors checkpoint under {directory!r}")
        self._open: dict[str, object] = {}

    def __contains__(self, name: str) -> bool:
        return name in self.weight_map

    def get(self, name: str) -> torch.Tensor:
        fname = self.weight_map[name]
        f = self._open.get(fname)
        if f is None:
            f = safe_open(os.path.join(self.directory, fname), "pt")
            self._open[fname] = f
        return f.get_tensor(name)

    def close(self) -> None:
        self._open.clear()


@torch.no_grad()
def load_model_weights(model, directory: str, strict: bool = True) -> dict:
    """Fill ``model``'s parameters from ``directory``. Returns {"loaded": n, "missing": [...]}."""
    cfg = model.cfg
    index = CheckpointIndex(directory)
    tr = getattr(model, "transport", None)
    ep_rank = getattr(tr, "rank", 0) if tr is not None else 0
    first_layer = model.layer_range[0]
    missing, loaded = [], 0
    for name, p in model.named_parameters():
        is_expert = getattr(p, "is_expert", False)
        offset = ep_rank * p.shape[0] if is_expert else 0
        for hub, (e, lo, hi) in hub_sources(name, tuple(p.shape), cfg, first_layer, offset):
            if hub not in index:
                if hub == "lm_head.weight" and "model.embed_tokens.weight" in index:
                    hub = "model.embed_tokens.weight"   # tied checkpoints store the matrix once
                else:
                    missing.append(hub)
                    continue
            t = index.get(hub)
            dst = p[e, lo:hi] if e is not None else p[lo:hi]
            if tuple(t.shape) != tuple(dst.shape):
                raise ValueError(f"{hub}: checkpoint shape {tuple(t.shape)} does not fit {tuple(dst.shape)}")
            dst.copy_(t.to(dst.dtype))
            loaded += 1
    index.close()
    if strict and missing:
        raise KeyError(f"{len(missing)} tensors are absent from {directory!r}, e.g. {missing[:4]}: refusing to leave "
                       f"parameters at their random initialisation")
    return {"loaded": loaded, "missing": missing}


def from_pretrained(directory: str, device="cpu", dtype=None, transport=None, **kw):
    """Build the model described by ``directory/config.json`` and load its weights."""
    from halo_b200.models.config import ModelConfig
    from halo_b200.models.qwen3 import build_model

    cfg = ModelConfig.load(directory)
    model = build_model(cfg, device=device, dtype=dtype, transport=transport, init=False, **kw)
    for p in model.parameters():
        if p.dim() == 1:
            p.data.fill_(1.0)
    load_model_weights(model, directory)
    return model
