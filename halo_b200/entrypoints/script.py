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
    if hlog.is_main_process():
        os.makedirs(train_args.output_dir, exist_ok=True)
    return pc


def build_runtime(pc, device, group=None):
    """Process groups + transports for the layout (expert parallel over all trainer ranks is the wired
    path). ``group``: the trainer subgroup when some ranks of the job serve rollouts instead."""
    if pc.world_size == 1 or not dist.is_initialized():
        return None
    from halo_b200.parallel.runtime import ParallelRuntime

    group = group if group is not None else dist.group.WORLD
    if pc.ep_size == pc.world_size and device.type == "cuda":
        return ParallelRuntime.for_expert_parallel(pc.world_size, device, group=group)
    if pc.ep_size > 1:
        from halo_b200.parallel.expert_parallel import CollectiveTransport

        return ParallelRuntime(device, dp_group=group, ep_group=group, transport=CollectiveTransport(group))
    return ParallelRuntime(device, dp_group=group)


def load_policy_model(model_args, pc, device, runtime, gradient_checkpointing=True, max_tokens=0):
    from halo_b200.checkpoint.load import from_pretrained
    from halo_b200.models.config import PRESETS, ModelConfig
    from halo_b200.models.qwen3 import build_model

    dtype = torch.bfloat16 if model_args.torch_dtype == "bfloat16" and device.type == "cuda" else torch.float32
    transport = runtime.transport if runtime is not None else None
    cfg = PRESETS[model_args.model_preset]() if model_args.init_from_scratch else ModelConfig.load(model_args.model_name_or_path)
    reject_model_layout(pc, cfg)
    if transport is not None and hasattr(transport, "configure") and cfg.is_moe:
        transport.configure(max_tokens=max_tokens, top_k=cfg.num_experts_per_tok, hidden=cfg.hidden_size,
                            n_local_experts=cfg.num_experts // transport.n_ranks)
    if model_args.init_from_scratch:
        return build_model(cfg, device=device, dtype=dtype, transport=transport,
                           gradient_checkpointing=gradient_checkpointing)
    return from_pretrained(model_args.model_name_or_path, device=device, dtype=dtype, transport=transport,
                           gradient_checkpointing=gradient_checkpointing)


def load_tokenizer(model_args):
    if not model_args.model_name_or_path:
        return None
    try:
        from transformers import AutoTokenizer

        return AutoTokenizer.from_pretrained(model_args.model_name_or_path)
    except Exception as exc:   # a checkpoint directory without tokenizer files: pre-tokenised data still works
        log.warning("no tokenizer at %s (%s)", model_args.model_name_or_path, exc)
        return None


def run_trainer(trainer, train_args):
    result = trainer.train()
    final = os.path.join(train_args.output_dir, "final")
    from halo_b200.checkpoint.save import save_model

    save_model(trainer.model, final, group=trainer.parallel.dp_group if trainer.parallel is not None else None)
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
