"""Model saves. The ladder picks the saver from the parallel layout (pipeline stages -> expert
parallel (gathered | sharded) -> data parallel / single process), and every saver ends in the same
standard layout: ``config.json`` + SafeTensors shards under hub names, loadable by
``transformers.AutoModelForCausalLM.from_pretrained`` (halo/checkpoint/parallel/save.py:63-104,
halo/checkpoint/parallel/ep.py:134-325).

Gathered expert-parallel save: the non-expert tensors come from the writer rank's replica; then,
layer by layer, each expert bank is all-gathered over the expert group and converted to per-expert
hub tensors on the writer, so peak extra memory is one layer's experts.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from halo_b200.runtime.consensus import DeferredRankFailure

from .atomic import atomic_write_json, remove_stale_staged
from .hub_layout import runtime_to_hub, whole_bank_source
from .writing import StreamingShardWriter

COMPLETE_MARKER = "trainer_state.json"


def _ep_info(model):
    tr = getattr(model, "transport", None)
    n = getattr(tr, "n_ranks", 1) if tr is not None else 1
    r = getattr(tr, "rank", 0) if tr is not None else 0
    g = getattr(tr, "group", None)
    return n, r, g


def _gather_expert_bank(t: torch.Tensor, n_ranks: int, group) -> torch.Tensor:
    if n_ranks == 1:
        return t
    out = torch.empty((n_ranks * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, t.contiguous(), group=group)
    return out


def save_model(model, directory: str, is_writer: bool | None = None, save_dtype: torch.dtype | None = torch.bfloat16,
               max_shard_bytes: int = 5 * 1024**3, sharded_experts: bool = False, extra_state: dict | None = None,
               group=None, adapters: str = "auto") -> None:
    """COLLECTIVE over the expert group when experts are sharded. ``is_writer``: this rank writes the
    files (default: global rank 0). ``sharded_experts``: every rank writes only its own experts to
    ``ep_shard_<rank>/`` (merge offline with halo_b200.checkpoint.tools.merge_ep_shards). ``group``: the
    ranks that take part in the save (default: the whole job); failures are agreed over it. ``adapters``: a model
    that carries low-rank adapters saves only them in the PEFT layout (``"auto"``), or its weights with the adapters
    folded in (``"merge"``)."""
    cfg = model.cfg
    lora = getattr(model, "lora_spec", None)
    if lora is not None and adapters != "merge":
        from halo_b200.peft.lora import save_adapters

        live = dist.is_available() and dist.is_initialized()
        writer_rank = (dist.get_rank(group) == 0) if live else True
        guard = DeferredRankFailure()
        with guard.catch():
            save_adapters(model, directory, base_model=getattr(model, "base_model_path", ""),
                          is_writer=writer_rank if is_writer is None else is_writer)
            if extra_state is not None and (writer_rank if is_writer is None else is_writer):
                atomic_write_json(os.path.join(directory, "halo_state.json"), extra_state)
        guard.raise_if_any(None if not live else (group or dist.group.WORLD), "saving the adapters failed")
        return

    def saved_tensor(name, p):
        if lora is None:
            return p.detach()
        from halo_b200.peft.lora import merged_weight

        return merged_weight(model, name, p)

    def base_parameters():
        if lora is None:
            yield from model.named_parameters()
            return
        from halo_b200.peft.lora import is_adapter_parameter

        for name, p in model.named_parameters():
            if not is_adapter_parameter(name):
                yield name, p

    n_ep, ep_rank, ep_group = _ep_info(model)
    live = dist.is_available() and dist.is_initialized()
    rank = dist.get_rank(group) if live else 0
    if is_writer is None:
        is_writer = rank == 0
    guard = DeferredRankFailure()
    first_layer = model.layer_range[0]
    writer = None
    with guard.catch():
        if sharded_experts and n_ep > 1:
            directory_w = os.path.join(directory, f"ep_shard_{ep_rank:05d}")
            writer = StreamingShardWriter(directory_w, max_shard_bytes, save_dtype)
        elif is_writer:
            remove_stale_staged(directory)
            writer = StreamingShardWriter(directory, max_shard_bytes, save_dtype)
    # 1. non-expert tensors (replicated: taken from the writer's copy; layer matrices sharded over the data-parallel
    #    ranks are assembled one layer at a time, a collective every rank takes part in)
    tp = getattr(model, "tensor_parallel", None)
    zero3 = getattr(model, "zero3", None)
    zero3_layer, zero3_full = -1, {}
    for name, p in base_parameters():
        if getattr(p, "is_expert", False) or name == "zero3_shard":
            continue
        if zero3 is not None and getattr(p, "zero3_managed", False):
            li = int(name.split(".")[1])
            if li != zero3_layer:
                zero3_layer, zero3_full = li, zero3.full_tensors(li)
            t_full = zero3_full[name]
        else:
            t_full = saved_tensor(name, p)
        if tp is not None and getattr(p, "tp_kind", None) is not None:
            from halo_b200.parallel.tensor_parallel import gather_full_weight

            t_full = gather_full_weight(p.tp_kind, t_full, cfg, tp)     # collective: every rank takes part
        with guard.catch():
            if writer is not None and is_writer:
                for hub, t in runtime_to_hub(name, t_full, cfg, first_layer).items():
                    writer.add(hub, t)
    # 2. expert banks, one layer at a time
    for name, p in base_parameters():
        if not getattr(p, "is_expert", False):
            continue
        if sharded_experts and n_ep > 1:
            if whole_bank_source(name, cfg, first_layer) is not None:
                raise NotImplementedError(f"{name}: this family stores an expert bank as ONE tensor, which per-rank shards "
                                          "cannot hold under one name; save unsharded (save_sharded_ep: false)")
            with guard.catch():
                for hub, t in runtime_to_hub(name, saved_tensor(name, p), cfg, first_layer, ep_rank * p.shape[0]).items():
                    writer.add(hub, t)
            continue
        local = saved_tensor(name, p)
        etp = getattr(model, "expert_tensor_parallel", None)
        if etp is not None and getattr(p, "etp_kind", None) is not None:
            from halo_b200.parallel.expert_tensor_parallel import unslice_expert_bank

            parts = [torch.empty_like(local) for _ in range(etp.size)]
            dist.all_gather(parts, local.contiguous(), group=etp.group)       # collective over the width-cut group
            local = unslice_expert_bank(p.etp_kind, parts)
        full = _gather_expert_bank(local, n_ep, ep_group)   # collective: every rank takes part
        with guard.catch():
            if is_writer and writer is not None:
                for hub, t in runtime_to_hub(name, full, cfg, first_layer, 0).items():
                    writer.add(hub, t)
        del full
    with guard.catch():
        if writer is not None:
            writer.finish()
        if is_writer:
            cfg.save(directory)
            head = getattr(model, "head", None)
            if head is not None and hasattr(head, "score"):
                # a model with a sequence-level head is written as the family's sequence-classification architecture
                import json

                path = os.path.join(directory, "config.json")
                d = json.load(open(path))
                d["architectures"] = [a.replace("ForCausalLM", "ForSequenceClassification") for a in d["architectures"]]
                d["num_labels"] = int(head.score.weight.shape[0])
                d.setdefault("pad_token_id", 0)
                atomic_write_json(path, d)
            if extra_state is not None:
                atomic_write_json(os.path.join(directory, "halo_state.json"), extra_state)
    guard.raise_if_any(None if not live else (group or dist.group.WORLD), "saving the model failed")


def save_pipeline_stages(model, directory: str, stage_index: int, n_stages: int, group=None,
                         save_dtype: torch.dtype | None = torch.bfloat16, max_shard_bytes: int = 5 * 1024**3,
                         is_writer: bool = True) -> None:
    """COLLECTIVE over the pipeline group (one rank per stage). Every stage writes its own layers - complete tensors
    under hub names - into shard files of its own stem in ``directory``; the first stage then merges the stages'
    tensor lists into the one ``model.safetensors.index.json`` and writes ``config.json``, so the result is an
    ordinary checkpoint (halo/checkpoint/parallel/pp.py).

    With expert-sharded stages every rank of a stage calls this: the stage's expert banks are gathered over its
    expert-parallel group (a collective of the whole stage), and only the rank with ``is_writer`` (one per stage: the
    members of one chain) writes and takes part in the collectives over ``group``."""
    cfg = model.cfg
    n_ep, _, ep_group = _ep_info(model)
    if not is_writer:
        # a stage's other replicas only hand their expert shards to the writer
        for name, p in model.named_parameters():
            if getattr(p, "is_expert", False) and n_ep > 1:
                _gather_expert_bank(p.detach(), n_ep, ep_group)
        return
    guard = DeferredRankFailure()
    first_layer = model.layer_range[0]
    weight_map, total = {}, 0
    live = dist.is_available() and dist.is_initialized()
    with guard.catch():
        if stage_index == 0:
            remove_stale_staged(directory)       # leftovers of an interrupted save, before any stage stages a new file
    guard.raise_if_any(None if not live else (group or dist.group.WORLD), "preparing the checkpoint directory failed")
    with guard.catch():
        writer = StreamingShardWriter(directory, max_shard_bytes, save_dtype, prefix=f"model-stage{stage_index:03d}")
        for name, p in model.named_parameters():
            t_full = p.detach()
            if getattr(p, "is_expert", False) and n_ep > 1:
                t_full = _gather_expert_bank(t_full, n_ep, ep_group)      # collective over the stage's expert group
            for hub, t in runtime_to_hub(name, t_full, cfg, first_layer).items():
                writer.add(hub, t)
        writer.finish(write_index=False)
        weight_map, total = writer.weight_map, writer.total_bytes
    guard.raise_if_any(None if not live else (group or dist.group.WORLD), "a pipeline stage failed to write its tensors")
    parts = [None] * n_stages
    if live and n_stages > 1:
        dist.all_gather_object(parts, (weight_map, total), group=group)
    else:
        parts = [(weight_map, total)]
    with guard.catch():
        if stage_index == 0:
            merged: dict[str, str] = {}
            for wm, _ in parts:
                clash = set(merged) & set(wm)
                if clash:
                    raise KeyError(f"tensors written by two stages: {sorted(clash)[:3]}")
                merged.update(wm)
            atomic_write_json(os.path.join(directory, "model.safetensors.index.json"),
                              {"metadata": {"total_size": sum(t for _, t in parts)}, "weight_map": merged})
            cfg.save(directory)
    guard.raise_if_any(None if not live else (group or dist.group.WORLD), "merging the pipeline stages' index failed")


def mark_complete(directory: str, trainer_state: dict) -> None:
    """Written last: a checkpoint without it is incomplete and never resumed from."""
    atomic_write_json(os.path.join(directory, COMPLETE_MARKER), trainer_state)


def is_complete(directory: str) -> bool:
    return os.path.isfile(os.path.join(directory, COMPLETE_MARKER))
