"""Translate a recipe written for the reference toolkit into this framework's keys:

    python -m halo_b200.configs.convert_recipe <reference.yaml> <out.yaml> [--method sft|dpo|kto|smpo|reward|...|grpo]

Keys with the same meaning are kept or renamed, keys whose job is done differently here are dropped with a note saying
what does it instead, and keys that ask for something this framework does not have stop the conversion with the
reason (``--lenient`` turns those into notes). The notes are written as comments at the top of the output, so the
converted recipe documents its own differences.
"""

from __future__ import annotations

import argparse
import os
import sys

import yaml

# same name, same meaning
KEPT = {
    "model_name_or_path", "per_device_train_batch_size", "learning_rate", "output_dir", "lr_scheduler_type", "logging_steps",
    "gradient_accumulation_steps", "report_to", "warmup_steps", "warmup_ratio", "eval_steps", "use_peft", "save_total_limit",
    "num_train_epochs", "save_steps", "max_length", "moe_balancing", "packing", "fp32_grad_reduce", "max_steps", "gradient_checkpointing",
    "fsdp_reshard_after_forward", "fsdp_reshard_after_backward", "lora_alpha", "lora_target_modules", "lora_r", "lora_dropout", "fp32_router",
    "fp32_experts", "fp32_non_ep_params", "weight_decay", "max_prompt_length", "max_completion_length", "num_generations", "num_iterations",
    "epsilon", "epsilon_high", "scale_rewards", "beta", "expert_parallel_size", "tensor_parallel_size", "context_parallel_size",
    "pipeline_parallel_size", "pipeline_microbatches", "expert_tensor_parallel_size", "ep_scope", "ep_buffer_backend", "max_concurrent_loading",
    "trust_remote_code", "optim", "seed", "routing_replay", "mtp_loss_weight", "environment_type", "max_grad_norm", "adam_beta1",
    "adam_beta2", "adam_epsilon", "router_aux_loss_coef", "resume_from_checkpoint", "gradient_checkpointing_plan", "temperature",
    "rollout_backend", "save_sharded_ep", "label_smoothing", "center_rewards_coefficient", "num_labels", "text_field",
    "reset_sinks", "train_sinks", "load_in_4bit", "load_in_8bit", "use_bnb_nested_quant", "bnb_4bit_quant_type",
}
# renamed: reference key -> (our key, optional value transform)
RENAMED = {
    "dataset_num_proc": ("num_proc", None),
    "dataloader_num_workers": ("num_proc", None),
    "packed_microbatch_tokens": ("token_budget", None),
    "max_train_row_tokens": ("packed_row_length", None),
    "rollout_temperature": ("temperature", None),
    "rollout_top_p": ("top_p", None),
    "rollout_max_tokens": ("max_completion_length", None),
    "environment_kwargs": ("environment_options", None),
    "scale_rewards_std_floor": ("std_floor", None),
    "skip_update_masked_frac": ("trust_region_mask_fraction", None),
    "rewards": ("reward_terms", None),
    "merge_expert_lora_on_save": ("merge_adapters_on_save", None),
    "train_on_last_assistant_only": ("assistant_only_loss", None),
    "mtp_loss_type": ("mtp_objective", lambda v: {"joint": "joint", "detached": "detached"}.get(v, "joint")),
    "target_margin": ("smpo_margin", None),
    "teacher_model": ("teacher_model_name_or_path", None),
    "distill_alpha": ("kd_weight", None),
    "desirable_weight": ("kto_desirable_weight", None),
    "undesirable_weight": ("kto_undesirable_weight", None),
    "chosen_sft_ratio": ("sft_loss_weight", None),
}
# dropped: what does the job here
DROPPED = {
    "attn_implementation": "attention is the built-in kernel family, chosen from the configuration at load time",
    "liger_kernel_config": "the fused norm / rotary / GLU / linear-cross-entropy kernels are the model's own ops",
    "use_liger_kernel": "the fused kernels are always on",
    "gradient_checkpointing_kwargs": "recomputation is the framework's own per-layer node (no reentrant / non-reentrant choice)",
    "logging_first_step": "the first step is logged whenever logging_steps divides 1",
    "eval_strategy": "evaluation runs every eval_steps when an eval dataset is given",
    "save_strategy": "saving runs every save_steps",
    "save_only_model": "checkpoints hold weights, optimizer shards and resume state; prune with save_total_limit",
    "per_device_eval_batch_size": "evaluation uses the packed rows of the eval dataset as they are",
    "remove_unused_columns": "records are read by field name; nothing is dropped implicitly",
    "dataloader_drop_last": "packed rows have a fixed length; there is no ragged last batch",
    "use_chunked_grpo_logprobs": "log-probabilities always come from the fused row-chunked head",
    "model_init_kwargs": "the model is built from config.json; dtype comes from torch_dtype",
    "force_chat_template": "set the tokenizer's chat_template (halo_b200.data.chat_render.load_chat_template) before training",
    "pad_token": "packed rows need no pad token; the tail of a row is a never-scored document",
    "eos_token": "the tokenizer's own eos_token_id ends generations",
    "run_name": "runs are named by output_dir",
    "enable_prefetch": "set rollout_prefetch: 1 to sample one round ahead",
    "log_completions": "GenerateExamplesCallback logs sample generations",
    "num_completions_to_print": "GenerateExamplesCallback logs sample generations",
    "text_only_model": "only text decoders are built",
    "eval_on_start": "not offered; run the evaluation CLI on the starting checkpoint",
    "batch_sampler": "rows are dealt to ranks by stride after a seeded shuffle",
    "lora_task_type": "adapters are always for causal language models",
    "use_grouped_gemm": "routed experts always run as grouped GEMMs",
    "train_sampling_strategy": "rows are dealt to ranks by stride after a seeded shuffle",
    "use_rlrr": "rank-shaped rewards are available as halo_b200.trainers.grpo.objective.dense_rank_rewards; there is no recipe switch",
    "use_vllm": "no generation server: add rollout_gpus: N (rollout ranks sample from a serving copy inside the job) or rollout_backend: in_process",
    "vllm_mode": "see use_vllm",
    "vllm_server_host": "see use_vllm",
    "rollout_server_configs": "no generation servers: add rollout_gpus: N, one rollout rank per former server GPU",
    "rollout_actor_budget": "episodes run as coroutines on the rollout rank; there is no actor pool to size",
}
# asks for something that does not exist here
UNSUPPORTED = {
    "images_field": "vision-language rows are not built",
    "lora_modules_to_save": "adapters are saved alone or merged; extra full modules beside them are not built",
    "pooling_mode": "embeddings are the last token's hidden state",
}
# hub datasets need a local copy: there is no downloader
DATA_KEYS = {"dataset", "conversation_field", "assistant_message_template", "test_size", "prompt_field", "answer_field", "chat_template",
             "system_prompt"}


VALUE_MAPS = {
    "routing_replay": ({"rollout": True, "recompute": True, "none": False, "off": False},
                       "the sampler's routing is replayed (one form: keyed by layer, safe under recomputation)"),
    "moe_balancing": ({"bias_update_transient": "bias_update"}, "the bias is kept across saves; there is no transient form"),
    "optim": ({"flash_adamw": "adamw_bf16", "adamw_torch_fused": "adamw_torch", "adamw_8bit": "adamw_bf16"},
              "bf16 moments with stochastic rounding are the memory-lean optimizer here"),
}
PREFERENCE_LOSSES = {"sigmoid": "dpo", "dpo": "dpo", "ipo": "ipo", "kto": "kto", "smpo": "smpo", "smooth_lower_bound": "smpo"}


def convert(recipe: dict, lenient: bool = False, method: str = "") -> tuple[dict, list[str]]:
    method = method or guess_method(recipe)
    out, notes, refused = {}, [], []
    for key, value in recipe.items():
        if value is None:
            notes.append(f"dropped {key}: it was unset (null) in the source; the default applies")
        elif key in ("max_prompt_length", "max_completion_length") and method != "grpo":
            notes.append(f"dropped {key}={value!r}: rows are bounded by packed_row_length; pairs that do not fit a row are skipped")
        elif key in VALUE_MAPS and value in VALUE_MAPS[key][0]:
            out[key] = VALUE_MAPS[key][0][value]
            notes.append(f"{key}: {value} -> {out[key]} ({VALUE_MAPS[key][1]})")
        elif key == "beta" and method == "grpo":
            out["grpo_beta"] = value
            notes.append("beta -> grpo_beta")
        elif key == "loss_type" and method == "embedding":
            notes.append(f"dropped loss_type={value!r}: embeddings train with the in-batch-negatives contrastive loss")
        elif key in KEPT:
            out[key] = value
        elif key in RENAMED:
            new, fn = RENAMED[key]
            out[new] = fn(value) if fn else value
            notes.append(f"{key} -> {new}")
        elif key in DROPPED:
            notes.append(f"dropped {key}: {DROPPED[key]}")
        elif key in UNSUPPORTED:
            refused.append(f"{key}: {UNSUPPORTED[key]}")
        elif key == "dataset":
            entries = value if isinstance(value, list) else [value]
            local = [e for e in entries if isinstance(e, str) and os.path.exists(e.split("@")[0])]
            if len(entries) == 1 and local:
                out["dataset_path"] = local[0]
            else:
                notes.append(f"dataset {entries}: copy the data to local JSONL / parquet files (or prepare it with the prepare-dataset "
                             f"tool) and set dataset_path; hub and S3 sources are not read")
        elif key == "conversation_field":
            notes.append(f"conversation_field {value!r}: records are read from a 'messages' field; rename the column when preparing the data")
        elif key == "assistant_message_template":
            out["completion_only_loss"] = True
            notes.append("assistant_message_template -> completion_only_loss: assistant spans come from the tokenizer's chat template")
        elif key == "loss_type" and value in PREFERENCE_LOSSES and method != "grpo":
            out["preference_loss"] = PREFERENCE_LOSSES[value]
            notes.append(f"loss_type {value} -> preference_loss {out['preference_loss']}")
        elif key == "loss_type" and method == "grpo":
            out["loss_type"] = value
        elif key == "loss_type":
            notes.append(f"dropped loss_type={value!r}: no counterpart for this method")
        elif key in DATA_KEYS:
            notes.append(f"dropped {key}: applied when the dataset is prepared, not at training time")
        elif key.startswith(("isr_", "early_stop_", "reasoning_", "rollout_", "eval_rollout", "num_generations_eval", "max_concurrent_rollouts",
                             "max_retries", "request_timeout", "episode_timeout", "max_turns", "drop_degenerate_groups", "balance_token_mass",
                             "top_entropy_quantile", "mask_truncated_completions", "sdpg_", "initial_", "mtp_train_scope", "model_revision",
                             "model_name", "generation_max_prompt_length", "num_eval_examples")):
            notes.append(f"dropped {key}={value!r}: no counterpart; see docs/grpo.md for the controls that exist")
        else:
            refused.append(f"{key}: unknown to the converter")
    if refused and not lenient:
        raise ValueError("the recipe asks for what this framework does not have:\n  " + "\n  ".join(refused))
    notes += [f"NOT CONVERTED {r}" for r in refused]
    return out, notes


def guess_method(recipe: dict) -> str:
    if "num_generations" in recipe:
        return "grpo"
    if recipe.get("loss_type") in ("kto", "smpo", "smooth_lower_bound"):
        return "kto" if recipe["loss_type"] == "kto" else "smpo"
    if recipe.get("loss_type") == "mnrl" or "pooling_mode" in recipe:
        return "embedding"
    if "beta" in recipe or recipe.get("loss_type") in ("dpo", "ipo", "sigmoid"):
        return "dpo"
    if "num_labels" in recipe:
        return "classification" if int(recipe["num_labels"]) > 1 else "reward"
    return "sft"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--method", default="")
    ap.add_argument("--lenient", action="store_true")
    args = ap.parse_args(argv)
    recipe = yaml.safe_load(open(args.src))
    method = args.method or guess_method(recipe)
    out, notes = convert(recipe, args.lenient, method)
    with open(args.dst, "w") as f:
        f.write(f"# converted from {os.path.basename(args.src)}; launch with:  python -m halo_b200.cli launch {method} {os.path.basename(args.dst)}\n")
        for n in notes:
            f.write(f"#   {n}\n")
        yaml.safe_dump(out, f, sort_keys=False)
    print(f"wrote {args.dst} ({len(out)} keys, {len(notes)} notes); method: {method}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
