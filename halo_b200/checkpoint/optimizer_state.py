"""Optimizer state on disk: one shard per rank (``optimizer_shard_<rank>.pt``) plus a topology
fingerprint. Exact resume requires the fingerprint of the run to match the one saved; otherwise the
load fails loudly unless a warm restart (fresh moments) was explicitly allowed (the role of
halo/checkpoint/parallel/optimizer.py and optimizer_meta.py)."""

from __future__ import annotations

import os

import torch

from .atomic import atomic_torch_save, atomic_write_json

META_NAME = "optimizer_meta.json"


class FingerprintMismatch(RuntimeError):
    pass


def shard_name(rank: int) -> str:
    return f"optimizer_shard_{rank:05d}.pt"


def _named_state(optimizer) -> dict:
    out = {}
    for gi, group in enumerate(optimizer.param_groups):
        names = group.get("param_names") or [f"group{gi}.{i}" for i in range(len(group["params"]))]
        for name, p in zip(names, group["params"]):
            st = optimizer.state.get(p)
            if st:
                out[name] = {k: (v.detach().to("cpu") if torch.is_tensor(v) else v) for k, v in st.items()}
    return out


def save_optimizer_shard(optimizer, directory: str, rank: int, fingerprint: dict, write_meta: bool) -> None:
    if hasattr(optimizer, "synchronize_state"):
        optimizer.synchronize_state()
    hyper = [{k: v for k, v in g.items() if k not in ("params", "param_names")} for g in optimizer.param_groups]
    atomic_torch_save({"state": _named_state(optimizer), "hyper": hyper}, os.path.join(directory, shard_name(rank)))
    if write_meta:
        atomic_write_json(os.path.join(directory, META_NAME), {"fingerprint": fingerprint, "format": 1})


def load_optimizer_shard(optimizer, directory: str, rank: int, fingerprint: dict, allow_warm_restart: bool = False) -> bool:
    """Returns True when the state was restored, False on an allowed warm restart."""
    import json

    meta_path = os.path.join(directory, META_NAME)
    path = os.path.join(directory, shard_name(rank))
    saved = json.load(open(meta_path))["fingerprint"] if os.path.isfile(meta_path) else None
    if saved != fingerprint or not os.path.isfile(path):
        if allow_warm_restart:
            return False
        raise FingerprintMismatch(
            f"optimizer shards under {directory!r} were written for {saved}, this run is {fingerprint}; exact resume "
            f"is impossible. Set allow_optimizer_warm_restart=true to restart with fresh moments.")
    blob = torch.load(path, map_location="cpu", weights_only=False)
    for gi, (group, hyper) in enumerate(zip(optimizer.param_groups, blob["hyper"])):
        for k, v in hyper.items():
            if k != "lr":
                group[k] = v
        names = group.get("param_names") or [f"group{gi}.{i}" for i in range(len(group["params"]))]
        for name, p in zip(names, group["params"]):
            st = blob["state"].get(name)
            if st is None:
                continue
            live = optimizer._state_for(p, group) if hasattr(optimizer, "_state_for") else optimizer.state[p]
            for k, v in st.items():
                if torch.is_tensor(v) and torch.is_tensor(live.get(k)):
                    live[k].copy_(v.to(live[k].dtype))
                else:
                    live[k] = v.to(p.device) if torch.is_tensor(v) and v.dim() > 0 else v
    return True
