"""The lifecycle every training script shares (halo/entrypoints/script.py:84-317):

``parse_script_args``  YAML + CLI -> dataclasses, distributed init, output_dir pattern expanded once
``init_training_script``  device, seed, ParallelismConfig (validated the same on every rank), run log
``load_policy_model``  from a checkpoint directory or from a preset (random init), expert-sharded
``run_trainer``  train with resume, final save
``with_distributed_teardown``  destroy the process group on success; on an exception leave at once so
                               the launcher reaps the peers instead of letting them hang in a collective
"""

from __future__ import annotations

import functools
import logging
import os
import sys

import torch
import torch.distributed as dist

from halo_b200 import log as hlog
from halo_b200.configs.arguments import (DataArguments, ModelArguments, ParallelismArguments, TrainingArguments)
from halo_b200.configs.parser import ArgumentParser, expand_output_dir
from halo_b200.parallel.rules import reject_model_layout
from halo_b200.runtime.collectives import broadcast_object
from halo_b200.runtime.consensus import reject_across_ranks
from halo_b200.runtime.process_group import destroy_distributed, init_distributed

log = logging.getLogger(__name__)


def parse_script_args(*extra_dataclasses, argv=None):
    hlog.configure_logging()
    device = init_distributed()
    if dist.is_initialized():
        from halo_b200.runtime import filesystem
        from halo_b200.runtime.consensus import reject_divergent_environment

        reject_divergent_environment()
        filesystem.resolve_consensus()
    parser = ArgumentParser(ModelArguments, DataArguments, TrainingArguments, ParallelismArguments, *extra_dataclasses)
    parsed = parser.parse(argv)
    train_args = parsed[2]
    train_args.output_dir = broadcast_object(expand_output_dir(train_args.output_dir), 0)
    return device, parsed


def init_training_script(device, model_args, train_args, par_args, world_size: int = 0, global_rank: int = -1):
    torch.manual_seed(train_args.seed)
    reason = None
    pc = None
    try:
        pc = par_args.to_config(world_size=world_size, global_rank=global_rank, init_from_scratch=model_args.init_from_scratch)
    except ValueError as exc:
        reason = str(exc)
    reject_across_ranks(reason, what="parallelism configuration")
    from halo_b200.runtime import filesystem

    if dist.is_initialized() and torch.device(device).type == "cuda":
        # the declared NVLink domain against what the GPUs report (placement, fabric cliques, multi-node prerequisites)
        from halo_b200.parallel import nvlink_fabric

        nvlink_fabric.validate_domain(pc.nvlink_domain_size, pc.world_size, pc.gpus_per_node)
        nvlink_fabric.verify_mnnvl_prerequisites(pc.nvlink_domain_size, pc.gpus_per_node)
    if dist.is_initialized():
        # the writer of each scope (rank 0 on shared storage, local rank 0 per node otherwise) creates the directory;
        # a multi-node job then checks the declaration against what the mounts do
        filesystem.makedirs_on_writer(train_args.output_dir)
        filesystem.verify_job_directories(train_args.output_dir)
    elif hlog.is_main_process():
        os.makedirs(train_args.output_dir, exist_ok=True)
    try:
        # `cli run stack-dump <output_dir>` then shows where every rank of a running (or hung) job stands
        from halo_b200.diagnostics import stack_dump

        stack_dump.install(train_args.output_dir)
    except (OSError, ValueError, RuntimeError) as exc:     # a read-only directory, a non-main thread: diagnostics only
        log.warning("stack-dump handler not installed: %s", exc)
    return pc


def build_runtime(pc, device, group=None):
    """Process groups + transports for the layout (expert parallel over all trainer ranks is the wired
    path). ``group``: the trainer subgroup when some ranks of the job serve rollouts instead."""
    if pc.world_size == 1 or not dist.is_initialized():
        return None
    from halo_b200.parallel.runtime import ParallelRuntime

    group = group if group is not None else dist.group.WORLD
    if pc.pp_size > 1:
        return _pipeline_runtime(pc, device, group)
    if pc.tp_size > 1 or pc.cp_size > 1:
        return _token_cutting_runtime(pc, device, group)
    if pc.ep_size == pc.world_size and device.type == "cuda":
        return ParallelRuntime.for_expert_parallel(pc.world_size, device, group=group)
    if pc.ep_size > 1:
        from halo_b200.parallel.expert_parallel import CollectiveTransport

        return ParallelRuntime(device, dp_group=group, ep_group=group, transport=CollectiveTransport(group))
    return ParallelRuntime(device, dp_group=group)


def _pipeline_runtime(pc, device, group):
    """Pipeline parallelism: stage s is the contiguous block of ``world / pp`` ranks starting at ``s * world / pp``; the
    ranks at one position of every stage form a chain (the pipeline group, NCCL / gloo point-to-point), the ranks of
    one stage are its replicas (data parallel, with the experts sharded over them when ``ep_size`` equals the stage
    width). Every rank creates every subgroup, in the same order. Finished by :func:`load_policy_model`, which knows
    the model's sizes."""
    from halo_b200.parallel.runtime import ParallelRuntime

    if pc.tp_size > 1 or pc.cp_size > 1:
        raise ValueError("pipeline parallelism together with tensor / context parallelism is not wired into the entry points")
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    width = world // pc.pp_size
    if device.type == "cuda" and rank == 0:
        log.warning("pipeline stages on GPUs carry an open defect: a 4-GPU run of the tiny preset completed its schedule but "
                    "reported non-finite gradient norms from the first step (first loss exactly ln(vocabulary): the last "
                    "stage computed on all-zero activations). The multi-process CPU runs of the same engine are sound; "
                    "watch the gradient norm of this run")
    if pc.ep_size not in (1, width):
        raise ValueError(f"with pipeline stages of {width} ranks, expert_parallel_size must be 1 or {width}, got {pc.ep_size}")
    ranks = [dist.get_global_rank(group, r) for r in range(world)] if group is not dist.group.WORLD else list(range(world))
    stage, pos = rank // width, rank % width
    chain = chain_up = stage_group = None
    for j in range(width):                                # chains: one rank of every stage
        g = dist.new_group(ranks[j::width])
        # a second communicator over the same ranks for the gradients that travel up the pipeline: activations and
        # gradients cross in the steady state, and on one NCCL communicator their sends would wait behind each other
        g_up = dist.new_group(ranks[j::width]) if device.type == "cuda" else g
        if j == pos:
            chain, chain_up = g, g_up
    for s in range(pc.pp_size):                           # stages: their replicas
        g = dist.new_group(ranks[s * width:(s + 1) * width]) if width > 1 else None
        if s == stage:
            stage_group = g
    parallel = None
    if width > 1:
        if pc.ep_size == width and device.type == "cuda":
            parallel = ParallelRuntime.for_expert_parallel(width, device, group=stage_group)
        elif pc.ep_size == width:
            from halo_b200.parallel.expert_parallel import CollectiveTransport

            parallel = ParallelRuntime(device, dp_group=stage_group, ep_group=stage_group, transport=CollectiveTransport(stage_group))
        else:
            parallel = ParallelRuntime(device, dp_group=stage_group)
    return {"kind": "pp", "chain": chain, "chain_up": chain_up, "stage": stage, "n_stages": pc.pp_size, "position": pos, "width": width,
            "parallel": parallel, "device": device, "schedule": pc.pp_schedule, "split": pc.pp_split, "pc": pc}


def finish_pipeline_runtime(spec: dict, model, optimizer, row_len: int, max_grad_norm: float, lr_scheduler=None):
    """The stage object and the training engine of one pipeline rank, once its model slice and optimizer exist."""
    from halo_b200.parallel.pipeline import PipelineStage
    from halo_b200.trainers.pipeline_engine import PipelineEngine

    stage = PipelineStage(model, spec["chain"], row_len, up_group=spec.get("chain_up"))
    return PipelineEngine(stage, optimizer, max_grad_norm, spec["schedule"], lr_scheduler, parallel=spec["parallel"],
                          min_microbatches=spec["n_stages"] if spec["schedule"] == "1f1b" else 1)


def _token_cutting_runtime(pc, device, group):
    """Tensor or context parallelism (both cut a row's tokens over consecutive ranks), optionally times data
    parallelism. Every rank creates every subgroup, in the same order."""
    from halo_b200.parallel.runtime import ParallelRuntime

    world, rank = dist.get_world_size(group), dist.get_rank(group)
    width = pc.tp_size if pc.tp_size > 1 else pc.cp_size
    if pc.tp_size > 1 and pc.cp_size > 1:
        raise ValueError("tensor and context parallelism together are not wired into the entry points")
    if pc.ep_size > 1 and pc.ep_size != world:
        raise ValueError("with tensor or context parallelism the experts are sharded over every rank of the job "
                         f"(expert_parallel_size = {world}), got {pc.ep_size}")
    ranks = [dist.get_global_rank(group, r) for r in range(world)] if group is not dist.group.WORLD else list(range(world))
    mine = replica = None
    for b in range(world // width):                       # blocks of consecutive ranks share a row
        g = dist.new_group(ranks[b * width:(b + 1) * width])
        if b == rank // width:
            mine = g
    for j in range(width):                                # ranks with the same position hold the same weight slices
        g = dist.new_group(ranks[j::width])
        if j == rank % width:
            replica = g
    return {"group": group, "axis_group": mine, "replica_group": replica if world > width else None,
            "kind": "tp" if pc.tp_size > 1 else "cp", "device": device, "runtime_cls": ParallelRuntime,
            "expert_parallel": pc.ep_size > 1}


def finish_token_cutting_runtime(spec: dict, cfg, max_tokens: int):
    """Second half of :func:`_token_cutting_runtime`, once the model config and the row length are known."""
    from halo_b200.parallel.context_parallel import ContextParallel
    from halo_b200.parallel.tensor_parallel import TensorParallel

    tp = cp = None
    if spec["kind"] == "tp":
        tp = TensorParallel(spec["axis_group"], spec["device"], hidden=cfg.hidden_size, max_tokens=max_tokens)
    else:
        cp = ContextParallel(spec["axis_group"], spec["device"], cfg, max_tokens)
    if spec.get("expert_parallel"):
        # experts sharded over every rank, rows cut over blocks of consecutive ranks: to the expert layer a rank's tokens
        # are just tokens (it dispatches whatever it holds), and replicated parameters sum their gradients over the job
        if spec["device"].type == "cuda":
            from halo_b200.parallel.runtime import SymmetricTransport

            transport = SymmetricTransport(spec["group"], spec["device"])
        else:
            from halo_b200.parallel.expert_parallel import CollectiveTransport

            transport = CollectiveTransport(spec["group"])
        return spec["runtime_cls"](spec["device"], dp_group=spec["group"], ep_group=spec["group"], transport=transport,
                                   context_parallel=cp, tensor_parallel=tp,
                                   tp_replica_group=spec["replica_group"] if tp is not None else None)
    return spec["runtime_cls"](spec["device"], dp_group=spec["group"], tensor_parallel=tp, context_parallel=cp,
                               tp_replica_group=spec["replica_group"] if tp is not None else None)


def load_policy_model(model_args, pc, device, runtime, gradient_checkpointing=True, max_tokens=0):
    from halo_b200.checkpoint.load import from_pretrained
    from halo_b200.models.config import PRESETS, ModelConfig
    from halo_b200.models.qwen3 import build_model

    dtype = torch.bfloat16 if model_args.torch_dtype == "bfloat16" and device.type == "cuda" else torch.float32
    cfg = PRESETS[model_args.model_preset]() if model_args.init_from_scratch else ModelConfig.load(model_args.model_name_or_path)
    new_mtp_head = False
    if getattr(model_args, "enable_mtp_head", False):
        import dataclasses

        new_mtp_head = not cfg.num_nextn_predict_layers      # the checkpoint has none yet: the head starts from its initialisation
        cfg = dataclasses.replace(cfg, num_nextn_predict_layers=1, mtp_loss_weight=model_args.mtp_loss_weight,
                                  mtp_objective=model_args.mtp_objective)
    reject_model_layout(pc, cfg)
    if isinstance(runtime, dict) and runtime.get("kind") == "pp":
        # this rank's stage: its layer range (head-weighted unless pipeline_split says otherwise), the embedding on the
        # first stage, the final norm and the head on the last; from a checkpoint every stage reads only its own tensors
        from halo_b200.parallel.pipeline import stage_layer_range

        spec = runtime
        lo, hi = stage_layer_range(cfg, spec["stage"], spec["n_stages"], spec["split"])
        par = spec["parallel"]
        transport = par.transport if par is not None else None
        if transport is not None and hasattr(transport, "configure") and cfg.is_moe:
            transport.configure(max_tokens=max_tokens, top_k=cfg.num_experts_per_tok, hidden=cfg.hidden_size,
                                n_local_experts=cfg.num_experts // transport.n_ranks)
        kw = dict(device=device, dtype=dtype, transport=transport, gradient_checkpointing=gradient_checkpointing,
                  layer_range=(lo, hi), has_embed=spec["stage"] == 0, has_head=spec["stage"] == spec["n_stages"] - 1)
        model = build_model(cfg, **kw) if model_args.init_from_scratch else from_pretrained(model_args.model_name_or_path, **kw)
        model.parallel_runtime = spec
        log.info("pipeline stage %d of %d: decoder layers [%d, %d)", spec["stage"], spec["n_stages"], lo, hi)
        return model
    if isinstance(runtime, dict):          # tensor / context parallelism: needs the model's sizes to finish
        runtime = finish_token_cutting_runtime(runtime, cfg, max_tokens)
        transport = runtime.transport
        if transport is not None and hasattr(transport, "configure") and cfg.is_moe:
            # a rank holds its share of a row (plus what the tile-aligned cuts add)
            share = max_tokens // max(pc.cp_size, pc.tp_size, 1) + 512
            transport.configure(max_tokens=share, top_k=cfg.num_experts_per_tok, hidden=cfg.hidden_size,
                                n_local_experts=cfg.num_experts // transport.n_ranks)
        model = build_model(cfg, device=device, dtype=dtype, gradient_checkpointing=gradient_checkpointing,
                            tensor_parallel=runtime.tensor_parallel, transport=transport) if model_args.init_from_scratch else \
            from_pretrained(model_args.model_name_or_path, device=device, dtype=dtype, transport=transport,
                            gradient_checkpointing=gradient_checkpointing, tensor_parallel=runtime.tensor_parallel)
        model.context_parallel = runtime.context_parallel
        model.parallel_runtime = runtime
        return model
    transport = runtime.transport if runtime is not None else None
    if transport is not None and hasattr(transport, "configure") and cfg.is_moe:
        transport.configure(max_tokens=max_tokens, top_k=cfg.num_experts_per_tok, hidden=cfg.hidden_size,
                            n_local_experts=cfg.num_experts // transport.n_ranks)
    if model_args.init_from_scratch:
        model = build_model(cfg, device=device, dtype=dtype, transport=transport,
                            gradient_checkpointing=gradient_checkpointing)
    elif new_mtp_head:
        from halo_b200.checkpoint.load import load_model_weights

        model = build_model(cfg, device=device, dtype=dtype, transport=transport, gradient_checkpointing=gradient_checkpointing)
        report = load_model_weights(model, model_args.model_name_or_path, strict=False)
        head_prefix = f"model.layers.{cfg.num_hidden_layers}."
        stray = [n for n in report["missing"] if not n.startswith(head_prefix)]
        if stray:
            raise KeyError(f"{len(stray)} tensors are absent from {model_args.model_name_or_path!r}, e.g. {stray[:4]}")
        log.info("multi-token-prediction head: %d tensors start from their initialisation", len(report["missing"]))
    else:
        model = from_pretrained(model_args.model_name_or_path, device=device, dtype=dtype, transport=transport,
                                gradient_checkpointing=gradient_checkpointing)
    if getattr(pc, "fsdp_reshard_after_forward", False) and runtime is not None and runtime.dp_world > 1:
        # ZeRO-3: the decoder layers' replicated matrices live as 1 / N slices and are gathered per layer pass
        from halo_b200.parallel.zero3 import shard_layers

        if not gradient_checkpointing:
            raise ValueError("fsdp_reshard_after_forward gathers a layer's weights for each of its passes: it needs "
                             "gradient_checkpointing: true")
        if getattr(model_args, "use_peft", False):
            raise ValueError("fsdp_reshard_after_forward with use_peft is not wired: the frozen base would be sharded, the "
                             "adapters are tiny")
        z = shard_layers(model, runtime.dp_group, device, ep_world=runtime.ep_world)
        log.info("ZeRO-3: %d layer matrices sharded over %d ranks, %.1f M parameters per rank (plus two layers of staging)",
                 sum(len(x) for x in z.params), z.world, z.shard_total / 1e6)
    from halo_b200.models.attention_selection import describe

    log.info(describe(model.cfg, device, dtype))
    if model.cfg.attention_sinks:
        from halo_b200.models.attention_sinks import apply_sinks_policy, policy_from_flags

        policy = policy_from_flags(getattr(model_args, "reset_sinks", True), getattr(model_args, "train_sinks", False))
        n = apply_sinks_policy(model, policy, pretrained=not model_args.init_from_scratch)
        log.info("attention sinks: %d tensors, policy %s", n, model.sinks_policy)
    if getattr(model_args, "lowp_format", ""):
        from halo_b200.models.qwen3 import apply_lowp_compute

        log.info("quantisation-aware training: %d modules round their products to %s",
                 apply_lowp_compute(model, model_args.lowp_format), model_args.lowp_format)
    if getattr(model_args, "use_peft", False):
        from halo_b200.peft.lora import apply_lora, load_adapters

        stats = apply_lora(model, model_args.lora_spec(), seed=0)
        model.base_model_path = model_args.model_name_or_path
        model.merge_adapters_on_save = model_args.merge_adapters_on_save
        if model_args.adapter_path:
            load_adapters(model, model_args.adapter_path)
        log.info("low-rank adapters: %d trainable parameters on %d frozen", stats["trainable"], stats["frozen"])
        if getattr(model_args, "load_in_4bit", False):
            from halo_b200.peft.qlora import quantize_base_weights

            q = quantize_base_weights(model, model_args.bnb_4bit_quant_type, model_args.use_bnb_nested_quant)
            log.info("quantised base (%s): %d matrices, %.1f M parameters in %.1f MB", model_args.bnb_4bit_quant_type, q["matrices"],
                     q["parameters"] / 1e6, q["bytes"] / 1e6)
    if model_args.freeze_patterns or model_args.train_only_patterns:
        from halo_b200.models.freeze import apply_freeze_patterns

        stats = apply_freeze_patterns(model, model_args.freeze_patterns, model_args.train_only_patterns)
        log.info("frozen %d parameters, training %d", stats["frozen"], stats["trainable"])
    return model


def pin_tokenizer(tokenizer, max_length: int = 0):
    """The settings every entry point relies on: a pad token (the end-of-sequence token when the tokenizer ships none -
    packed rows never score it, padded evaluation batches need one), right-side truncation and padding, and
    ``model_max_length`` equal to the run's ``max_length`` so that truncation warnings refer to the run's limit
    (the role of halo/model_loading/tokenizer_setup.py)."""
    if tokenizer.pad_token_id is None and tokenizer.eos_token is not None:
        tokenizer.pad_token = tokenizer.eos_token
        log.info("tokenizer has no pad token: using the end-of-sequence token %r", tokenizer.eos_token)
    tokenizer.padding_side = "right"
    tokenizer.truncation_side = "right"
    if max_length:
        tokenizer.model_max_length = int(max_length)
    return tokenizer


def load_tokenizer(model_args):
    if not model_args.model_name_or_path:
        return None
    try:
        from transformers import AutoTokenizer

        return pin_tokenizer(AutoTokenizer.from_pretrained(model_args.model_name_or_path), getattr(model_args, "max_length", 0))
    except Exception as exc:   # a checkpoint directory without tokenizer files: pre-tokenised data still works
        log.warning("no tokenizer at %s (%s)", model_args.model_name_or_path, exc)
        return None


def run_trainer(trainer, train_args):
    result = trainer.train()
    final = os.path.join(train_args.output_dir, "final")
    from halo_b200.checkpoint.save import save_model

    spec = getattr(trainer.model, "parallel_runtime", None)
    if isinstance(spec, dict) and spec.get("kind") == "pp":
        from halo_b200.checkpoint.save import save_pipeline_stages

        # one chain writes (position 0 of every stage); the other replicas of a stage only hand over their expert shards
        sharded = spec["parallel"] is not None and spec["parallel"].ep_world > 1
        if spec["position"] == 0 or sharded:
            save_pipeline_stages(trainer.model, final, spec["stage"], spec["n_stages"], group=spec["chain"],
                                 is_writer=spec["position"] == 0)
        return result

    save_model(trainer.model, final, group=trainer.group, is_writer=trainer.is_main,
               adapters="merge" if getattr(trainer.model, "merge_adapters_on_save", False) else "auto")
    return result


def with_distributed_teardown(main):
    @functools.wraps(main)
    def wrapped(*a, **kw):
        try:
            out = main(*a, **kw)
        except BaseException:
            import traceback

            traceback.print_exc()
            sys.stderr.flush()
            os._exit(1)   # peers may be inside a collective: do not wait for them
        destroy_distributed()
        return out

    return wrapped
