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

from .hub_layout import hub_sources, stored_with_unit_offset, whole_bank_source
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
    tp = getattr(model, "tensor_parallel", None)
    etp = getattr(model, "expert_tensor_parallel", None)
    # layer matrices that live as 1 / N slices (ZeRO-3): filled into host stand-ins of their full shape, from which every
    # rank then keeps its slices
    zero3 = getattr(model, "zero3", None)
    full_shapes = {n: shape for items in zero3.params for n, _, _, _, shape in items} if zero3 is not None else {}
    stand_ins: dict = {}
    for name, p in model.named_parameters():
        if name == "zero3_shard":
            continue
        if name in full_shapes:
            p = stand_ins.setdefault(name, torch.empty(full_shapes[name], dtype=zero3.dtype))
        is_expert = getattr(p, "is_expert", False)
        offset = ep_rank * p.shape[0] if is_expert else 0
        tp_kind = getattr(p, "tp_kind", None) if tp is not None else None
        etp_kind = getattr(p, "etp_kind", None) if etp is not None else None
        if tp_kind is not None or etp_kind is not None:
            # a width-sliced parameter: assemble the unsliced tensor from its hub pieces on the host, keep this
            # rank's slice
            n, got = _load_sliced(index, name, p, cfg, first_layer, offset, tp_kind, tp, etp_kind, etp, missing)
            loaded += got
            continue
        whole = whole_bank_source(name, cfg, first_layer)
        if whole is not None:
            # stored as one transformed tensor (transposed, gate / up interleaved): undone on the host
            hub, to_runtime = whole
            if hub in index:
                stored = index.get(hub)
            elif hub + "_blocks" in index and hub + "_scales" in index:
                # a release with packed MXFP4 banks ([E, out, G, 16] codes, one power-of-two scale per 32 values): unpacked
                # to the bf16 form [E, in, out] the release's own bf16 twin stores
                from halo_b200.ops.lowp import unpack_mxfp4_blocks

                stored = unpack_mxfp4_blocks(index.get(hub + "_blocks"), index.get(hub + "_scales")).transpose(1, 2)
            else:
                missing.append(hub)
                continue
            t = to_runtime(stored)
            if is_expert and t.shape[0] != p.shape[0]:
                t = t[offset:offset + p.shape[0]]          # an expert-parallel rank keeps its experts of the whole bank
            if tuple(t.shape) != tuple(p.shape):
                raise ValueError(f"{hub}: checkpoint shape {tuple(t.shape)} does not fit {tuple(p.shape)}")
            p.copy_(t.to(p.dtype))
            loaded += 1
            continue
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
            if stored_with_unit_offset(name, cfg):
                dst.add_(1)
            loaded += 1
    index.close()
    if stand_ins:
        zero3.load_full(stand_ins)              # collective: ends with a barrier
    if strict and missing:
        raise KeyError(f"{len(missing)} tensors are absent from {directory!r}, e.g. {missing[:4]}: refusing to leave "
                       f"parameters at their random initialisation")
    return {"loaded": loaded, "missing": missing}


def _full_shape(p, cfg, tp_kind, tp, etp_kind, etp):
    if tp_kind in ("qkv", "qkv_bias"):
        return (cfg.qkv_dim, *p.shape[1:])
    if tp_kind == "gate_up":
        return (p.shape[0] * tp.size, p.shape[1])
    if tp_kind in ("o", "down"):
        return (p.shape[0], p.shape[1] * tp.size)
    if etp_kind == "gate_up":
        return (p.shape[0], p.shape[1] * etp.size, p.shape[2])
    return (p.shape[0], p.shape[1], p.shape[2] * etp.size)


def _load_sliced(index, name, p, cfg, first_layer, offset, tp_kind, tp, etp_kind, etp, missing):
    shape = _full_shape(p, cfg, tp_kind, tp, etp_kind, etp)
    full = torch.empty(shape, dtype=p.dtype)
    got = 0
    for hub, (e, lo, hi) in hub_sources(name, shape, cfg, first_layer, offset):
        if hub not in index:
            missing.append(hub)
            continue
        t = index.get(hub)
        dst = full[e, lo:hi] if e is not None else full[lo:hi]
        if tuple(t.shape) != tuple(dst.shape):
            raise ValueError(f"{hub}: checkpoint shape {tuple(t.shape)} does not fit {tuple(dst.shape)}")
        dst.copy_(t.to(dst.dtype))
        got += 1
    if tp_kind is not None:
        from halo_b200.parallel.tensor_parallel import slice_for_rank

        p.copy_(slice_for_rank(tp_kind, full, cfg, tp.rank, tp.size))
    else:
        from halo_b200.parallel.expert_tensor_parallel import slice_expert_bank

        p.copy_(slice_expert_bank(etp_kind, full, etp.rank, etp.size))
    return 1, got


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
